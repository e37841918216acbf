"""Shared pieces of the Zugunex tests: small configurations (none of them a shipped model's sizes), float64 copies of seeded
weights for the oracle, an engine builder."""
from __future__ import annotations

from typing import Dict, Optional

import torch


def attn(heads=3, dim=8, rot_dim=6, vdim=10, rank=20, window=5, scale=0.3, base=100.0, kv_from: Optional[int] = None, rot_dims=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale, "mask": {"size": window},
         "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def dense(ff=44):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, top=2, ff=12, scale=1.3, shared_ff: Optional[int] = 20):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if shared_ff:
        f["shared"] = {"ff": shared_ff}
    return f


def layer(mixer, mlp):
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def config(layers, width=40, vocab=97, eps=1e-5) -> dict:
    return {"architecture": "Zugunex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


def small_config() -> dict:
    """Odd sizes throughout (nothing a multiple of 4), a sharing layer with its own head count and window, a layer without
    feed-forward, experts with and without a shared one, top 1 and a single head."""
    return config([
        layer(attn(), dense()),
        layer(attn(heads=2, dim=6, vdim=7, window=9, scale=0.2, kv_from=0), moe()),
        layer(attn(heads=1, dim=10, rot_dim=4, vdim=9, rank=11, window=3, base=7.0), None),
        layer(attn(heads=4, dim=5, rot_dim=4, vdim=6, rank=11, window=6, base=7.0, kv_from=2), moe(experts=3, top=1, ff=9, scale=0.7, shared_ff=None)),
        layer(attn(heads=3, dim=8, vdim=5, window=40, kv_from=0), moe(experts=4, top=4, ff=6, shared_ff=5)),
    ])


def aligned_config(width=128, window=24) -> dict:
    """Sizes the tensor-core products take (multiples of 8 and 32), for the bfloat16 path."""
    a = dict(heads=4, dim=32, rot_dim=16, vdim=24, rank=48, window=window, scale=0.15, base=1000.0)
    return config([
        layer(attn(**a), dense(ff=192)),
        layer(attn(**{**a, "heads": 2, "vdim": 40}, kv_from=0), moe(experts=6, top=2, ff=32, shared_ff=64)),
        layer(attn(**a), moe(experts=4, top=3, ff=40, scale=2.0, shared_ff=None)),
    ], width=width, vocab=203)


def many_heads_config() -> dict:
    """8 and 16 query heads over one latent row: single tokens take the heads-as-rows attention with the keys split over CTAs."""
    a = dict(dim=8, rot_dim=4, vdim=12, rank=20, window=70, scale=0.3, base=50.0)
    return config([layer(attn(heads=8, **a), dense(ff=48)), layer(attn(heads=16, **a, kv_from=0), moe(experts=4, top=2, ff=16, shared_ff=16))],
                  width=48, vocab=101)


def f64(weights: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    return {k: v.double() for k, v in weights.items()}


def build(cfg_dict: dict, dtype=torch.float32, seed=0, weights=None, **kw):
    """(model on the GPU, float64 weights)."""
    from vyomai_b200 import ZugunexConfig, ZugunexForCausalLM
    cfg = ZugunexConfig(cfg_dict)
    w = weights if weights is not None else ZugunexForCausalLM.random_weights(cfg, seed=seed)
    kw.setdefault("sorted_min_rows", 8)   # both forms of the experts' sum come up at test sizes
    kw.setdefault("force_sorted", True)
    return ZugunexForCausalLM(cfg, w, dtype=dtype, device="cuda", **kw), f64(w)


def random_config(seed: int, experts: bool = True) -> dict:
    """A configuration drawn from the design's whole space: 3-6 layers in any order of owners and sharers, head counts from 1 to 12,
    unrelated channel counts, windows shorter and longer than the test sequences, every feed-forward kind (experts=False: the same
    draw with every mixture replaced by a dense feed-forward)."""
    g = torch.Generator().manual_seed(seed)
    pick = lambda xs: xs[int(torch.randint(0, len(xs), (1,), generator=g))]  # noqa: E731
    width = pick([48, 64, 96, 160])
    layers, owners = [], []
    for i in range(pick([3, 4, 5, 6])):
        own = not owners or pick([True, False])
        if own:
            geo = dict(rank=pick([12, 16, 40, 64, 96]), rot_dim=pick([2, 4, 8, 16, 32]), base=pick([10.0, 1000.0, 250000.0]))
            owners.append((i, geo))
            src = None
        else:
            src, geo = pick(owners)
        m = attn(heads=pick([1, 2, 3, 4, 6, 8, 12]), dim=pick([4, 8, 16, 24, 32]), vdim=pick([4, 8, 20, 32, 48]), window=pick([1, 3, 17, 50, 200]),
                 scale=pick([0.1, 0.25, 0.5]), kv_from=src, **geo)
        kind = pick(["none", "dense", "moe", "moe_shared"])
        mlp = None if kind == "none" else dense(ff=pick([24, 64, 100])) if kind == "dense" else \
            moe(experts=pick([2, 3, 8, 16]), top=1, ff=pick([8, 12, 32]), scale=pick([0.5, 1.0, 2.5]), shared_ff=pick([8, 40]) if kind == "moe_shared" else None)
        if mlp and mlp["kind"] == "moe":
            mlp["router"]["top"] = pick(list(range(1, mlp["router"]["experts"] + 1)))
        if mlp and mlp["kind"] == "moe" and not experts:
            mlp = dense(ff=mlp["expert"]["ff"] * 2)
        layers.append(layer(m, mlp))
    return config(layers, width=width, vocab=pick([50, 131, 256]), eps=pick([1e-6, 1e-5]))
