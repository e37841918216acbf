"""Plain float64 statement of the Zugunex decoder's mechanisms, one function per mechanism, written from the equations and
sharing no code with vyomai_b200: interleaved partial rotation, latent attention (keys and values re-expanded from a
cached low-rank latent, one rotated key part shared by the heads, sliding window, softmax sink, per-head output gate),
latent sharing between layers, output-side RMS norms, the tanh-GELU feed-forward and the sigmoid-routed mixture of
squared-ReLU experts with a gated shared expert. Every function takes a WHOLE sequence from position 0 (time along dim 0);
the tests compare the CUDA path (whole prompts, portions, single-token decoding, mixed batches) against these.

Notation: T tokens, H heads, dn / dr unrotated / rotated query-key sizes per head, dv value size, R latent size.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_pairs(x: torch.Tensor, base: float, dims: int, pos0: int = 0) -> torch.Tensor:
    """x [T, ..., n]: the first `dims` entries of the last axis are rotated pairwise, (2i, 2i + 1) by the angle
    p * base^(-2i / dims) at position p = pos0 + t; the others pass."""
    T = x.shape[0]
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    a = (torch.arange(T, dtype=F64) + pos0)[:, None] * f[None, :]          # [T, half]
    shape = [T] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(a).view(shape), torch.sin(a).view(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def window_mask(T: int, window: int) -> torch.Tensor:
    """[T, T] bool: query i sees key j iff 0 <= i - j < window."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (i - j >= 0) & (i - j < window)


def sink_softmax_attention(scores: torch.Tensor, values: torch.Tensor, mask: torch.Tensor, sink: Optional[torch.Tensor]) -> torch.Tensor:
    """scores [H, T, T] (already scaled), values [H, T, dv], mask [T, T]; the denominator also holds exp(sink_h)."""
    s = scores.masked_fill(~mask[None], float("-inf"))
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink.view(-1, 1, 1))
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink.view(-1, 1, 1) - m)
    return (e / den) @ values


def latent_kv(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float):
    """The cached pair of a layer that owns a down-projection: latent c [T, R] (RMS-normed, plain weight) and the rotated
    shared key part kr [T, dr]."""
    R, dr = m["kv_rank"], m["rot_dim"]
    d = h @ w["dkv"].T
    c = rms(d[:, :R], eps) * w["dkv.norm"]
    kr = rotate_pairs(d[:, R:R + dr], m["rot"]["base"], m["rot"]["dims"])
    return c, kr


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, c: torch.Tensor, kr: torch.Tensor) -> torch.Tensor:
    """h [T, W] -> [T, W]: queries of this layer against keys / values expanded from (c, kr)."""
    T = h.shape[0]
    H, dn, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    q = (h @ w["q"].T).view(T, H, dn + dr)
    qn = q[..., :dn]
    qr = rotate_pairs(q[..., dn:], m["rot"]["base"], m["rot"]["dims"])
    kn = (c @ w["uk"].T).view(T, H, dn)
    v = (c @ w["uv"].T).view(T, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", qn, kn) + torch.einsum("ihd,jd->hij", qr, kr)) * m["scale"]
    o = sink_softmax_attention(scores, v.transpose(0, 1), window_mask(T, m["mask"]["size"]), w.get("sink"))   # [H, T, dv]
    gate = torch.sigmoid(h @ w["g"].T)                                                                       # [T, H]
    o = o.transpose(0, 1) * gate[:, :, None]
    return o.reshape(T, H * dv) @ w["o"].T


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor]) -> torch.Tensor:
    return gelu_tanh(h @ w["up"].T) @ w["down"].T


def relu2_expert(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return torch.relu(h @ up.T) ** 2 @ down.T


def route(h: torch.Tensor, router: torch.Tensor, top: int, scale: float):
    """-> (chosen experts [T, top], their weights [T, top]): sigmoid scores, the `top` largest, divided by their sum, times scale."""
    s = torch.sigmoid(h @ router.T)
    val, idx = torch.topk(s, top, dim=-1)
    return idx, val / (val.sum(-1, keepdim=True) + 1e-20) * scale


def moe_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], mlp: dict) -> torch.Tensor:
    r = mlp["router"]
    idx, wt = route(h, w["router"], r["top"], r["scale"])
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for n in range(idx.shape[1]):
            e = int(idx[t, n])
            out[t] += wt[t, n] * relu2_expert(h[t:t + 1], w[f"e{e}.up"], w[f"e{e}.down"])[0]
    if mlp.get("shared"):
        out = out + torch.sigmoid(h @ w["shared.sg"].T) * relu2_expert(h, w["shared.up"], w["shared.down"])
    return out


def _sub(w: Dict[str, torch.Tensor], pre: str) -> Dict[str, torch.Tensor]:
    return {k[len(pre):]: v for k, v in w.items() if k.startswith(pre)}


def forward(cfg: dict, w: Dict[str, torch.Tensor], ids: List[int], residuals: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from position 0; w maps tensor names to float64 tensors."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(ids)]
    kept = {}
    for i, L in enumerate(cfg["layers"]):
        m, mw = L["mixer"], _sub(w, f"l{i}.mix.")
        if "kv_from" in m and m["kv_from"] is not None:
            c, kr = kept[int(m["kv_from"])]
        else:
            c, kr = kept[i] = latent_kv(x, mw, m, eps)
        x = x + rms(latent_attention(x, mw, m, c, kr), eps) * w[f"l{i}.norm1"]
        if L.get("mlp"):
            fw = _sub(w, f"l{i}.mlp.")
            y = dense_ff(x, fw) if L["mlp"]["kind"] == "dense" else moe_ff(x, fw, L["mlp"])
            x = x + rms(y, eps) * w[f"l{i}.norm2"]
        if residuals is not None:
            residuals.append(x.clone())
    return (rms(x, eps) * w["final.norm"]) @ w["head"].T
