"""The hybrid decoder end to end on the GPU: GelutarForCausalLM through HybridBatchEngine / HybridCacheManager (the engine a
user generates with, and the one bin/trace_run drives) against oracle/hybrid_oracle.py's float64 forward of the same seeded
weights. Whole prompts, portions down to two tokens, token-by-token decoding, mixed batches of unequal requests, pages and
slots that are freed and handed out again, long decoding across window edges, other sizes, greedy generation, the replayer's
command line. float32 models are held to 2e-4 of the largest logit, bfloat16 ones to 3e-2."""
import json
import os
import subprocess
import sys

import pytest
import torch

from oracle import hybrid_oracle as O
from tests import hybrid_util as U

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {torch.float32: 2e-4, torch.bfloat16: 3e-2}


def _oracle_logits(cfg, W, toks):
    return O.forward(cfg, W, list(toks))


def test_residual_stream_layer_by_layer():
    cfg = U.small_config()
    model, W = U.build(cfg)
    eng, _ = U.engine_for(model)
    toks = U.tokens(19, cfg["vocab"], 1)
    ref_res = []
    ref = O.forward(cfg, W, toks, residuals=ref_res)
    model.debug_residuals = []
    got = eng.feed([("a", toks, list(range(len(toks))))]).float().cpu()
    for i, (x, r) in enumerate(zip(model.debug_residuals, ref_res)):
        assert U.rel_err(x.cpu(), r) < 1e-4, f"layer {i}"
    model.debug_residuals = None
    assert U.rel_err(got, ref) < TOL[torch.float32]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cuts", [[40], [2, 2, 2, 30], [1], [17, 3, 5], [33]])
def test_prompt_portions_and_decoding_agree_with_the_oracle(dtype, cuts):
    cfg = U.small_config()
    model, W = U.build(cfg, dtype=dtype)
    eng, _ = U.engine_for(model)
    toks = U.tokens(40, cfg["vocab"], 2)
    ref = _oracle_logits(cfg, W, toks)
    got = U.feed_in_portions(eng, "s", toks, cuts)
    assert U.rel_err(got, ref) < TOL[dtype]


def test_cutting_changes_nothing_beyond_rounding():
    cfg = U.small_config()
    model, _ = U.build(cfg)
    eng, _ = U.engine_for(model)
    toks = U.tokens(48, cfg["vocab"], 3)
    whole = U.feed_in_portions(eng, "w", toks, [48])
    for cuts in ([2] * 24, [1], [5, 9, 2, 20], [47]):
        eng.release(["p"])
        assert U.rel_err(U.feed_in_portions(eng, "p", toks, cuts), whole) < 2e-5, cuts


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mixed_batch_equals_each_request_alone(dtype):
    cfg = U.small_config()
    model, W = U.build(cfg, dtype=dtype)
    eng, _ = U.engine_for(model, max_seqs=1, max_tokens=16)     # pools must grow under the batch
    lens = {"a": 31, "b": 3, "c": 12, "d": 1}
    toks = {k: U.tokens(n + 6, cfg["vocab"], 10 + i) for i, (k, n) in enumerate(lens.items())}
    ref = {k: _oracle_logits(cfg, W, t) for k, t in toks.items()}
    got = {k: [] for k in lens}
    # prompts of unequal length in one step, then decode together; "b" and "d" end early and drop out
    out = eng.feed([(k, toks[k][:n], list(range(n))) for k, n in lens.items()]).float().cpu()
    at = 0
    for k, n in lens.items():
        got[k].append(out[at:at + n])
        at += n
    live = list(lens)
    for step in range(6):
        if step == 3:
            eng.release(["b", "d"])
            live = ["a", "c"]
        out = eng.feed([(k, [toks[k][lens[k] + step]], [0]) for k in live]).float().cpu()
        for j, k in enumerate(live):
            got[k].append(out[j:j + 1])
    for k in lens:
        g = torch.cat(got[k])
        assert U.rel_err(g, ref[k][: g.shape[0]]) < TOL[dtype], k


def test_freed_pages_and_slots_are_reused_without_leaking_state():
    cfg = U.small_config()
    model, W = U.build(cfg)
    eng, mgr = U.engine_for(model, max_seqs=2, max_tokens=64)
    first = U.tokens(30, cfg["vocab"], 20)
    U.feed_in_portions(eng, "old", first, [25])
    held = eng.active["old"]
    old_slot, old_blocks = held.slot, list(held.blocks)
    eng.release(["old"])
    blocks0, slots0 = mgr.num_blocks, mgr.num_slots
    seen_slots, seen_blocks = set(), set()
    for r in range(4):      # later requests land on the freed slot / pages (free lists are FIFO over a small pool)
        toks = U.tokens(22, cfg["vocab"], 30 + r)
        got = U.feed_in_portions(eng, f"n{r}", toks, [2, 15])
        seen_slots.add(eng.active[f"n{r}"].slot)
        seen_blocks.update(eng.active[f"n{r}"].blocks)
        eng.release([f"n{r}"])
        assert U.rel_err(got, _oracle_logits(cfg, W, toks)) < TOL[torch.float32], r
    assert old_slot in seen_slots and seen_blocks & set(old_blocks)
    assert (mgr.num_blocks, mgr.num_slots) == (blocks0, slots0)
    assert len(mgr.free_slots) == mgr.num_slots and len(mgr.free_blocks) == mgr.num_blocks


def test_long_decode_across_window_and_page_edges():
    """Window 5 / 7 with pages of 4: 70 decoded tokens pass many window and page borders; the slow decay heads keep the prompt."""
    cfg = U.small_config()
    model, W = U.build(cfg)
    eng, _ = U.engine_for(model)
    toks = U.tokens(80, cfg["vocab"], 40)
    assert U.rel_err(U.feed_in_portions(eng, "s", toks, [10]), _oracle_logits(cfg, W, toks)) < TOL[torch.float32]


@pytest.mark.parametrize("seed,layers,width,vocab", [
    (1, [U.lightning(heads=2, dim=32, vdim=32, decay=(0.8, 0.99))], 64, 50),
    (2, [U.parallel(heads=1, kv_heads=1, dim=32, vdim=8, window=3, keep_first=1, r_heads=1, r_kv=1, r_dim=8, r_vdim=40, taps=1, ff=0)], 40, 33),
    (3, [U.parallel(heads=8, kv_heads=1, dim=8, vdim=8, window=64, keep_first=4, r_heads=6, r_kv=2, r_dim=16, r_vdim=16, taps=5),
         U.parallel(window=2, keep_first=5)], 128, 257),
    (4, [U.lightning(heads=4, dim=64, vdim=64, decay=(0.5, 0.9, 0.99, 0.999), ff=256), U.parallel(heads=2, kv_heads=2, dim=64, vdim=64, window=16,
                                                                                                   keep_first=1, r_heads=2, r_kv=2, r_dim=64,
                                                                                                   r_vdim=64, taps=4, ff=256)], 256, 512),
])
def test_other_sizes(seed, layers, width, vocab):
    cfg = U.config(layers, width=width, vocab=vocab, eps=1e-6, emb_scale=0.8, logit_scale=1.3)
    for dtype in (torch.float32, torch.bfloat16):
        model, W = U.build(cfg, dtype=dtype, seed=seed, ranks=(3, 9))
        eng, _ = U.engine_for(model, block_size=16)
        toks = U.tokens(36, vocab, seed)
        ref = _oracle_logits(cfg, W, toks)
        assert U.rel_err(U.feed_in_portions(eng, "s", toks, [21, 2]), ref) < TOL[dtype]


def test_wide_heads_and_a_prompt_longer_than_a_tile():
    """128-wide heads (the kernels' 16-byte load paths and widest templates), a 150-token prompt fed as 70 + 2 + 65 and the rest decoded,
    window 40 with 2 kept tokens: the prompt crosses the tiled kernels' 64-token tiles and chunks inside and between portions."""
    layers = [U.lightning(heads=2, dim=128, vdim=128, decay=(0.9, 0.999), ff=128),
              U.parallel(heads=2, kv_heads=1, dim=128, vdim=128, window=40, keep_first=2, scale=0.09, r_heads=2, r_kv=1, r_dim=128, r_vdim=128,
                         taps=4, ff=128)]
    cfg = U.config(layers, width=256, vocab=300, eps=1e-6, emb_scale=1.0, logit_scale=0.5)
    for dtype in (torch.float32, torch.bfloat16):
        model, W = U.build(cfg, dtype=dtype, seed=7, ranks=(8, 8))
        eng, _ = U.engine_for(model, block_size=16)
        toks = U.tokens(150, 300, 8)
        ref = _oracle_logits(cfg, W, toks)
        assert U.rel_err(U.feed_in_portions(eng, "s", toks, [70, 2, 65]), ref) < TOL[dtype]


def test_greedy_generation_through_the_engine():
    """generate(): waiting room (batch limit 2 for 3 prompts), prompts and decoding tokens in the same packed step. Tokens must
    equal the oracle's greedy continuation wherever its top-1 / top-2 margin is not at rounding level."""
    cfg = U.small_config()
    model, W = U.build(cfg)
    eng, mgr = U.engine_for(model, max_batch_size=2)
    prompts = [U.tokens(n, cfg["vocab"], 50 + n) for n in (9, 2, 17)]
    outs = eng.generate(prompts, max_new_tokens=8)
    for p, o in zip(prompts, outs):
        assert o[: len(p)] == p and len(o) == len(p) + 8
        ref, margins = O.greedy(cfg, W, p, 8)
        for i, m in enumerate(margins):
            if m < 1e-3:
                break
            assert o[len(p) + i] == ref[len(p) + i]
    assert not eng.active and len(mgr.free_slots) == mgr.num_slots and len(mgr.free_blocks) == mgr.num_blocks


def test_trace_replayer_command_line(tmp_path):
    from vyomai_b200 import GelutarConfig, GelutarForCausalLM
    from vyomai_b200.checkpoint import save_safetensors
    cfg = U.small_config()
    w = GelutarForCausalLM.random_weights(GelutarConfig(cfg), seed=5, low_rank=(4, 6))
    mdir, odir = tmp_path / "model", tmp_path / "out"
    mdir.mkdir()
    (mdir / "config.json").write_text(json.dumps(cfg))
    save_safetensors(str(mdir / "model.safetensors"), w)
    a, b = U.tokens(14, cfg["vocab"], 60), U.tokens(6, cfg["vocab"], 61)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:11], "want": [0, 10]}, {"id": "b", "tokens": b[:5], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[11]], "want": []}, {"id": "b", "tokens": [b[5]], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[12:], "want": [1]}], "end": ["a"]}]
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(mdir), "--dtype", "float32", "--out", str(odir),
                        "--max-tokens", "32"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [ln for ln in p.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    W = U.f64(w)
    ra, rb = _oracle_logits(cfg, W, a), _oracle_logits(cfg, W, b)
    import numpy as np
    rd = lambda s: torch.from_numpy(np.fromfile(str(odir / f"{s}.f32"), dtype="<f4").reshape(-1, cfg["vocab"]))  # noqa: E731
    assert U.rel_err(rd(0), ra[[0, 10]]) < TOL[torch.float32]
    assert U.rel_err(rd(1), rb[[5]]) < TOL[torch.float32]
    assert U.rel_err(rd(2), ra[[13]]) < TOL[torch.float32]
