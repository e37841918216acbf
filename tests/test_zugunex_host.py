"""Host-side pieces of the Zugunex family that need no GPU: the configuration's checks and tensor list, the registry, the cache
manager's handling of layers that read another layer's pages, and the oracle's own mechanisms against brute-force loops."""
import math

import pytest
import torch

from oracle import zugunex_oracle as O
from tests import zugunex_util as U


def test_config_lists_the_tensors_of_every_layer_kind():
    from vyomai_b200 import ZugunexConfig
    cfg = ZugunexConfig(U.small_config())
    shapes = cfg.tensor_shapes()
    assert shapes["l0.mix.dkv"] == (20 + 6, 40) and "l1.mix.dkv" not in shapes and "l1.mix.dkv.norm" not in shapes
    assert shapes["l1.mix.q"] == (2 * (6 + 6), 40) and shapes["l1.mix.uk"] == (2 * 6, 20) and shapes["l1.mix.uv"] == (2 * 7, 20)
    assert "l2.norm2" not in shapes and "l2.mlp.up" not in shapes
    assert shapes["l1.mlp.e4.down"] == (40, 12) and shapes["l1.mlp.shared.sg"] == (1, 40) and "l3.mlp.shared.up" not in shapes
    assert shapes["l3.mlp.router"] == (3, 40)


@pytest.mark.parametrize("bad", ["forward", "chain", "rank", "kind", "type"])
def test_config_rejects_what_the_design_does_not_have(bad):
    from vyomai_b200 import ZugunexConfig
    d = U.small_config()
    if bad == "forward":
        d["layers"][1]["mixer"]["kv_from"] = 2
    elif bad == "chain":
        d["layers"][4]["mixer"]["kv_from"] = 1
    elif bad == "rank":
        d["layers"][1]["mixer"]["kv_rank"] = 21
    elif bad == "kind":
        d["layers"][0]["mlp"]["kind"] = "gated"
    else:
        d["layers"][0]["type"] = "lightning"
    with pytest.raises(ValueError):
        ZugunexConfig(d)


def test_registry_knows_the_architecture():
    from vyomai_b200.registry import architectures
    assert "Zugunex" in architectures()


class _FakeModel:
    device = "cpu"

    def cache_specs(self):
        own = {"pages": (1, 12, 0), "states": {}}
        return [[own], [{"pages": None, "states": {}, "pages_from": (0, 0)}], [dict(own)], [{"pages": None, "states": {}, "pages_from": (2, 0)}]]


def test_sharing_layers_see_their_owner_s_pool_also_after_growth():
    from vyomai_b200.paged import HybridCacheManager, HybridSequence
    mgr = HybridCacheManager(_FakeModel(), max_tokens=8, block_size=4, max_seqs=1, device="cpu")
    assert mgr.views[1][0] is mgr.views[0][0] and mgr.views[3][0] is mgr.views[2][0] and mgr.views[2][0] is not mgr.views[0][0]
    assert mgr.views[0][0].v_pool is None and mgr.views[0][0].k_pool.shape[1:] == (4, 1, 12)
    before = mgr.views[0][0].k_pool
    before[0, 0, 0, 0] = 5.0
    seq = HybridSequence("a", [])
    mgr.allocate(seq, 200)   # far beyond the hint: the pools are replaced by larger ones
    assert mgr.views[1][0].k_pool is mgr.views[0][0].k_pool and mgr.views[1][0].k_pool is not before
    assert float(mgr.views[1][0].k_pool[0, 0, 0, 0]) == 5.0 and len(seq.blocks) == 50


def test_sharing_must_name_an_owner():
    from vyomai_b200.paged import HybridCacheManager

    class Bad(_FakeModel):
        def cache_specs(self):
            return [[{"pages": None, "states": {}, "pages_from": (0, 0)}]]
    with pytest.raises(ValueError):
        HybridCacheManager(Bad(), device="cpu")


# ---- the oracle against brute force ----
def test_oracle_rotation_by_hand():
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0]], [[1.0, 0.0, 0.0, 1.0, -1.0]]], dtype=torch.float64)   # [T=2, 1, 5], dims 4
    y = O.rotate_pairs(x, 16.0, 4, pos0=3)
    for t in range(2):
        p = 3 + t
        for i, f in enumerate((1.0, 16.0 ** -0.5)):
            u, v = x[t, 0, 2 * i], x[t, 0, 2 * i + 1]
            a = p * f
            assert abs(float(y[t, 0, 2 * i]) - float(u * math.cos(a) - v * math.sin(a))) < 1e-12
            assert abs(float(y[t, 0, 2 * i + 1]) - float(v * math.cos(a) + u * math.sin(a))) < 1e-12
        assert float(y[t, 0, 4]) == float(x[t, 0, 4])


def test_oracle_attention_against_token_loops():
    m = U.attn(heads=2, dim=3, rot_dim=2, vdim=4, rank=5, window=3, scale=0.7)
    g = torch.Generator().manual_seed(0)
    W = 8
    w = {"q": torch.randn(2 * 5, W, generator=g), "dkv": torch.randn(7, W, generator=g), "dkv.norm": torch.rand(5, generator=g) + 0.5,
         "uk": torch.randn(6, 5, generator=g), "uv": torch.randn(8, 5, generator=g), "sink": torch.randn(2, generator=g),
         "g": torch.randn(2, W, generator=g), "o": torch.randn(W, 8, generator=g)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(9, W, generator=g).double()
    c, kr = O.latent_kv(h, w, m, 1e-6)
    got = O.latent_attention(h, w, m, c, kr)
    q = (h @ w["q"].T).view(9, 2, 5)
    for i in range(9):
        heads = []
        for hd in range(2):
            qn, qr = q[i, hd, :3], O.rotate_pairs(q[i:i + 1, hd:hd + 1, 3:], 100.0, 2, pos0=i)[0, 0]
            js = [j for j in range(9) if 0 <= i - j < 3]
            s = torch.stack([(qn @ (w["uk"][hd * 3:(hd + 1) * 3] @ c[j]) + qr @ kr[j]) * 0.7 for j in js])
            e = torch.exp(s)
            den = e.sum() + torch.exp(w["sink"][hd])
            o = sum(e[n] / den * (w["uv"][hd * 4:(hd + 1) * 4] @ c[j]) for n, j in enumerate(js))
            heads.append(o * torch.sigmoid(w["g"][hd] @ h[i]))
        want = w["o"] @ torch.cat(heads)
        assert float((got[i] - want).abs().max()) < 1e-10


def test_oracle_router_weights_sum_to_the_scale():
    g = torch.Generator().manual_seed(1)
    idx, wt = O.route(torch.randn(6, 8, generator=g).double(), torch.randn(5, 8, generator=g).double(), 2, 1.5)
    assert idx.shape == (6, 2) and float((wt.sum(-1) - 1.5).abs().max()) < 1e-12
