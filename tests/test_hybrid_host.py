"""Host-side pieces of the hybrid decoder that need no GPU: the oracle's mechanisms checked against independent closed forms,
the configuration reader, the safetensors reader / writer, the registry, and the page + state-slot manager's bookkeeping."""
import json

import pytest
import torch

from oracle import hybrid_oracle as O
from tests import hybrid_util as U


def test_visibility_rule():
    assert O.visible(10, 10, 1, 0) and not O.visible(10, 9, 1, 0)
    assert O.visible(10, 6, 5, 0) and not O.visible(10, 5, 5, 0)
    assert O.visible(10, 1, 5, 2) and not O.visible(10, 2, 5, 2)
    assert not O.visible(3, 4, 100, 100)


def test_oracle_attention_is_softmax_with_an_extra_denominator_term():
    g = torch.Generator().manual_seed(0)
    T, H, G, dk, dv = 9, 4, 2, 6, 5
    q, k, v = (torch.randn(T, n, d, generator=g, dtype=torch.float64) for n, d in ((H, dk), (G, dk), (G, dv)))
    sink = torch.randn(H, generator=g, dtype=torch.float64)
    out = O.window_sink_attention(q, k, v, scale=0.4, window=4, keep_first=2, sink=sink)
    kk, vv = k.repeat_interleave(H // G, 1), v.repeat_interleave(H // G, 1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * 0.4
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    mask = (j <= i) & ((i - j < 4) | (j < 2))
    s = s.masked_fill(~mask, float("-inf"))
    s = torch.cat([s, sink[:, None, None].expand(H, T, 1)], dim=-1)       # the sink as one more column without a value
    p = torch.softmax(s, -1)[..., :T]
    ref = torch.einsum("hij,jhd->ihd", p, vv)
    assert torch.allclose(out, ref, atol=1e-12)


def test_oracle_lightning_equals_the_explicit_sum():
    g = torch.Generator().manual_seed(1)
    T, H, dk, dv = 11, 2, 4, 3
    q, k, v = (torch.randn(T, H, d, generator=g, dtype=torch.float64) for d in (dk, dk, dv))
    decay = [0.7, 0.99]
    out = O.lightning_attention(q, k, v, decay)
    for h in range(H):
        for t in range(T):
            ref = sum(decay[h] ** (t - s) * (q[t, h] @ k[s, h]) * v[s, h] for s in range(t + 1))
            assert torch.allclose(out[t, h], ref, atol=1e-12)


def test_oracle_delta_rule_without_decay_and_full_strength_projects_out_old_values():
    g = torch.Generator().manual_seed(2)
    dk, dv = 5, 4
    k = O.unit(torch.randn(3, 1, dk, generator=g, dtype=torch.float64), eps=0.0)
    k[2] = k[0]
    v = torch.randn(3, 1, dv, generator=g, dtype=torch.float64)
    out = O.gated_delta_rule(k, k, v, torch.ones(3, 1, dk, dtype=torch.float64), torch.ones(3, 1, dtype=torch.float64))
    assert torch.allclose(out[0, 0], v[0, 0], atol=1e-12)     # read-out sees the current token's write
    assert torch.allclose(out[2, 0], v[2, 0], atol=1e-12)     # rewriting k_0 replaces what it held


def test_oracle_conv_last_column_is_the_current_token():
    x = torch.arange(1.0, 6.0, dtype=torch.float64)[:, None]
    w = torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64)
    y = O.causal_conv(x, w, act=None)[:, 0]
    assert y.tolist() == [1.0, 12.0, 123.0, 234.0, 345.0]


def test_config_reader_and_implied_shapes():
    from vyomai_b200 import GelutarConfig, GelutarForCausalLM
    cfg = GelutarConfig(U.small_config())
    shapes = cfg.tensor_shapes()
    assert shapes["l0.mix.left.k"] == (2 * 16, 96) and shapes["l0.mix.left.g"] == (4, 96) and shapes["l0.mix.right.v.conv"] == (4 * 24, 3)
    assert shapes["l3.mix.right.q"] == (1 * 24, 96) and shapes["l3.mix.right.dt_bias"] == (2 * 24,)
    assert "l2.norm2" not in shapes and "l2.mlp.up" not in shapes and "l1.mlp.up" in shapes
    w = GelutarForCausalLM.random_weights(cfg, seed=0, low_rank=(5, 7))
    assert set(w) == set(shapes)
    assert w["l0.mix.right.a1"].shape == (5, 96) and w["l0.mix.right.g2"].shape == (4 * 24, 7)
    with pytest.raises(ValueError):
        GelutarConfig({**U.small_config(), "architecture": "Other"})
    bad = U.small_config()
    bad["layers"][0]["type"] = "unknown"
    with pytest.raises(ValueError):
        GelutarConfig(bad)


def test_safetensors_round_trip_and_registry(tmp_path):
    from vyomai_b200 import registry
    from vyomai_b200.checkpoint import load_safetensors, save_safetensors
    t = {"a.b": torch.randn(3, 5).bfloat16(), "i": torch.arange(7, dtype=torch.int32), "f": torch.randn(2, 2, 2)}
    save_safetensors(str(tmp_path / "x.safetensors"), t)
    back = load_safetensors(str(tmp_path / "x.safetensors"))
    assert set(back) == set(t) and all(back[k].dtype == t[k].dtype and torch.equal(back[k], t[k]) for k in t)
    assert "Gelutar" in registry.architectures()
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Nope"}))
    with pytest.raises(KeyError):
        registry.load_model(str(tmp_path))


class _FakeModel:
    device = torch.device("cpu")

    def cache_specs(self):
        return [[{"pages": (2, 4, 6), "states": {}}, {"pages": None, "states": {"S": (2, 3, 5), "conv_q": (8, 2)}}],
                [{"pages": None, "states": {"S": (1, 4, 4)}}]]


def test_manager_hands_out_grows_and_takes_back_pages_and_slots():
    from vyomai_b200 import HybridCacheManager, HybridSequence
    mgr = HybridCacheManager(_FakeModel(), max_tokens=8, block_size=4, max_seqs=1, device="cpu")
    assert mgr.views[0][0].k_pool.shape[1:] == (4, 2, 4) and mgr.views[0][0].v_pool.shape[1:] == (4, 2, 6)
    assert mgr.views[0][1].states["S"].shape == (1, 2, 3, 5) and mgr.views[1][0].k_pool is None
    a, b = HybridSequence("a", []), HybridSequence("b", [])
    mgr.allocate(a, 5)
    assert len(a.blocks) == 2 and a.slot == 0
    mgr.views[0][1].states["S"][a.slot] = 7.0
    mgr.views[0][0].k_pool[a.blocks[0]] = 3.0
    mgr.allocate(b, 9)                       # needs a second slot and more pages than are left: both pools grow, contents stay
    assert b.slot == 1 and len(b.blocks) == 3 and not set(a.blocks) & set(b.blocks)
    assert float(mgr.views[0][1].states["S"][a.slot].min()) == 7.0 and float(mgr.views[0][0].k_pool[a.blocks[0]].min()) == 3.0
    mgr.allocate(a, 6)                       # still inside its second page
    assert len(a.blocks) == 2
    mgr.allocate(a, 9)
    assert len(a.blocks) == 3
    total = mgr.num_blocks
    mgr.free(a)
    mgr.free(b)
    assert a.slot == -1 and not a.blocks and len(mgr.free_blocks) == total and len(mgr.free_slots) == mgr.num_slots
    assert mgr.can_allocate(4 * total) and not mgr.can_allocate(4 * total + 1)
