"""Plain, slow float64 statement of the hybrid decoder family's mechanisms (the Gelutar architecture), one function per
mechanism, written from the equations and sharing no code with vyomai_b200. Every function takes a WHOLE sequence from
position 0 (time along dim 0) and loops over tokens where the mechanism is a recurrence; the tests compare the CUDA path
— whole prompts, portions, single-token decoding, mixed batches — against these.

Notation: T tokens, H heads, G key/value heads, dk / dv per-head key and value sizes.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dim."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    return rms(x, eps) * (1.0 + w)


def silu(x):
    return x * torch.sigmoid(x)


def visible(i: int, j: int, window: int, keep_first: int) -> bool:
    """Does the query at position i see the key at position j?"""
    return j <= i and (i - j < window or j < keep_first)


def window_sink_attention(q, k, v, *, scale: float, window: int, keep_first: int, sink: Optional[torch.Tensor], gate_logits=None):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] -> [T, H, dv]. Softmax over the visible keys with exp(sink_h) added to the
    denominator; the head's output times sigmoid(gate_logits[t, h])."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            js = [j for j in range(i + 1) if visible(i, j, window, keep_first)]
            s = torch.stack([(q[i, h] * k[j, g]).sum() * scale for j in js])
            m = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            den = e.sum() + (torch.exp(sink[h] - m) if sink is not None else 0.0)
            o = sum(e[n] / den * v[j, g] for n, j in enumerate(js))
            if gate_logits is not None:
                o = o * torch.sigmoid(gate_logits[i, h])
            out[i, h] = o
    return out


def causal_conv(x, w, act=silu):
    """x [T, C], w [C, taps] with the LAST column multiplying the current token; zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    y = torch.zeros(T, C, dtype=F64)
    for t in range(T):
        for d in range(taps):
            if t - d >= 0:
                y[t] += w[:, taps - 1 - d] * x[t - d]
    return act(y) if act is not None else y


def lightning_attention(q, k, v, decay: List[float]):
    """q, k [T, H, dk], v [T, H, dv]: S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t."""
    T, H, dk = q.shape
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for h in range(H):
        S = torch.zeros(dk, v.shape[2], dtype=F64)
        for t in range(T):
            S = decay[h] * S + torch.outer(k[t, h], v[t, h])
            out[t, h] = S.T @ q[t, h]
    return out


def gated_delta_rule(q, k, v, g, beta):
    """q, k [T, G, dk] (already unit-normed / scaled), v [T, H, dv], g [T, H, dk] decay per key channel, beta [T, H].
    S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T, G, dk = q.shape
    H, dv = v.shape[1], v.shape[2]
    out = torch.zeros(T, H, dv, dtype=F64)
    for h in range(H):
        c = h // (H // G)
        S = torch.zeros(dk, dv, dtype=F64)
        for t in range(T):
            S = g[t, h][:, None] * S
            u = beta[t, h] * (v[t, h] - S.T @ k[t, c])
            S = S + torch.outer(k[t, c], u)
            out[t, h] = S.T @ q[t, c]
    return out


def unit(x, eps=1e-6):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


def relu2_mlp(h, up, down):
    return torch.relu(h @ up.T) ** 2 @ down.T


# ---- mixers and the model ----
def lightning_mixer(h, W: Dict[str, torch.Tensor], m: dict, eps: float):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ W["q"].T).view(T, H, dk)
    k = silu(h @ W["k"].T).view(T, H, dk)
    v = silu(h @ W["v"].T).view(T, H, dv)
    o = lightning_attention(q, k, v, m["decay"]).reshape(T, H * dv)
    o = rms(o, eps) * W["norm"] * torch.sigmoid(h @ W["g"].T)
    return o @ W["o"].T


def attention_mixer(h, W, m, eps):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (rms(h @ W["q"].T, eps) * W["q.norm"]).view(T, H, dk)
    k = (rms(h @ W["k"].T, eps) * W["k.norm"]).view(T, G, dk)
    v = (h @ W["v"].T).view(T, G, dv)
    o = window_sink_attention(q, k, v, scale=m["scale"], window=m["mask"]["size"], keep_first=m["mask"]["keep_first"], sink=W["sink"],
                              gate_logits=h @ W["g"].T)
    return o.reshape(T, H * dv) @ W["o"].T


def delta_mixer(h, W, m, eps):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv(h @ W["q"].T, W["q.conv"]).view(T, G, dk)
    k = causal_conv(h @ W["k"].T, W["k.conv"]).view(T, G, dk)
    v = causal_conv(h @ W["v"].T, W["v.conv"]).view(T, H, dv)
    q = unit(q) * dk ** -0.5
    k = unit(k)
    beta = torch.sigmoid(h @ W["b"].T)
    a = (h @ W["a1"].T) @ W["a2"].T + W["dt_bias"]
    g = torch.exp(-torch.exp(W["A_log"])[None, :, None] * torch.nn.functional.softplus(a).view(T, H, dk))
    o = gated_delta_rule(q, k, v, g, beta)
    o = rms(o, eps) * W["norm"] * torch.sigmoid((h @ W["g1"].T) @ W["g2"].T).view(T, H, dv)
    return o.reshape(T, H * dv) @ W["o"].T


def _sub(W, pre):
    return {k[len(pre):]: v for k, v in W.items() if k.startswith(pre)}


def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: List[int], residuals: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence. W: name -> float64 tensor."""
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = norm_one_plus(x, W[p + "norm1"], eps)
        if L["type"] == "lightning":
            y = lightning_mixer(h, _sub(W, p + "mix."), L["mixer"], eps)
        else:
            a = attention_mixer(h, _sub(W, p + "mix.left."), L["mixer"]["left"], eps)
            b = delta_mixer(h, _sub(W, p + "mix.right."), L["mixer"]["right"], eps)
            y = 0.5 * (rms(a, eps) * W[p + "mix.left.out"] + rms(b, eps) * W[p + "mix.right.out"])
        x = x + y
        if L.get("mlp"):
            x = x + relu2_mlp(norm_one_plus(x, W[p + "norm2"], eps), W[p + "mlp.up"], W[p + "mlp.down"])
        if residuals is not None:
            residuals.append(x.clone())
    return norm_one_plus(x, W["final.norm"], eps) @ W["head"].T * cfg["logit_scale"]


def greedy(cfg, W, prompt: List[int], n_new: int):
    """Greedy continuation by re-running the whole sequence; also returns each step's top-1 / top-2 margin."""
    toks, margins = list(prompt), []
    for _ in range(n_new):
        lg = forward(cfg, W, toks)[-1]
        top = lg.topk(2).values
        margins.append(float(top[0] - top[1]))
        toks.append(int(lg.argmax()))
    return toks, margins
