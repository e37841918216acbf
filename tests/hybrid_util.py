"""Shared pieces of the hybrid-decoder tests: small configurations (none of them a shipped model's sizes), float64 copies
of seeded weights for the oracle, and a driver that feeds a schedule of token portions through the batching engine."""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import torch


def lightning(heads=3, dim=8, vdim=40, decay=(0.55, 0.9, 0.995), ff=72):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def parallel(heads=4, kv_heads=2, dim=16, vdim=24, window=5, keep_first=2, scale=0.3, r_heads=4, r_kv=2, r_dim=16, r_vdim=24, taps=3, ff=72):
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                               "mask": {"size": window, "keep_first": keep_first}},
                      "right": {"heads": r_heads, "kv_heads": r_kv, "dim": r_dim, "vdim": r_vdim, "conv": taps}},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(layers, width=96, vocab=131, eps=1e-5, emb_scale=1.7, logit_scale=0.3) -> dict:
    return {"architecture": "Gelutar", "vocab": vocab, "width": width, "embedding": {"scale": emb_scale}, "norm": {"eps": eps},
            "logit_scale": logit_scale, "layers": layers}


def small_config() -> dict:
    """Attention first, a layer without feed-forward, grouped heads on both sides, dim != vdim, odd vocabulary."""
    return config([parallel(), lightning(), lightning(ff=0), parallel(heads=6, kv_heads=3, dim=8, vdim=16, window=7, keep_first=0, r_heads=2,
                                                                      r_kv=1, r_dim=24, r_vdim=8, taps=2), lightning(heads=1, dim=16, vdim=16, decay=(0.97,))])


def f64(weights: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    return {k: v.double() for k, v in weights.items()}


def build(cfg_dict: dict, dtype=torch.float32, seed=0, ranks=(5, 7), **kw):
    """(model on the GPU, float64 weights). The two low-rank projections of the delta mixer get different ranks."""
    from vyomai_b200 import GelutarConfig, GelutarForCausalLM
    cfg = GelutarConfig(cfg_dict)
    w = GelutarForCausalLM.random_weights(cfg, seed=seed, low_rank=ranks)
    return GelutarForCausalLM(cfg, w, dtype=dtype, device="cuda", **kw), f64(w)


def engine_for(model, max_tokens=256, block_size=4, max_seqs=2, **kw):
    from vyomai_b200 import HybridBatchEngine, HybridCacheManager
    mgr = HybridCacheManager(model, max_tokens=max_tokens, block_size=block_size, max_seqs=max_seqs)
    return HybridBatchEngine(model, mgr, **kw), mgr


def feed_in_portions(engine, key, tokens: Sequence[int], cuts: Sequence[int]) -> torch.Tensor:
    """Feeds one sequence portion by portion (cuts = portion sizes, the rest one token at a time) asking for every position;
    returns logits [len(tokens), vocab] on the CPU."""
    rows, at = [], 0
    sizes = list(cuts)
    while at < len(tokens):
        n = sizes.pop(0) if sizes else 1
        n = min(n, len(tokens) - at)
        rows.append(engine.feed([(key, list(tokens[at:at + n]), list(range(n)))]).float().cpu())
        at += n
    return torch.cat(rows)


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    return float((got.double() - want.double()).abs().max() / want.double().abs().max().clamp_min(1e-30))


def tokens(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def shuffled_batch(lengths: Sequence[int], pos0: Sequence[int], block_size: int, device, seed=0) -> Tuple:
    """A PackedBatch whose sequences own shuffled pages and slots (pages for pos0 + length positions each)."""
    from vyomai_b200 import ops
    g = torch.Generator().manual_seed(seed)
    n = len(lengths)
    need = [(p + l + block_size - 1) // block_size for p, l in zip(pos0, lengths)]
    perm = torch.randperm(sum(need) + 3, generator=g).tolist()
    width = max(need)
    table, at = [], 0
    for k in need:
        table.append(perm[at:at + k] + [0] * (width - k))
        at += k
    slots = torch.randperm(n + 2, generator=g)[:n].tolist()
    cu = [0]
    for l in lengths:
        cu.append(cu[-1] + l)
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=device)  # noqa: E731
    batch = ops.PackedBatch(t(cu), t(list(pos0)), t(slots), max(lengths), t(table).view(n, width), block_size)
    return batch, table, slots, sum(need) + 3, n + 2
