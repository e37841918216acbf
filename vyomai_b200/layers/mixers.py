"""Sequence mixers and the squared-ReLU feed-forward of the hybrid decoder family (models/gelutar.py), on the packed-batch
kernels of csrc/seqmix.cu. Each mixer is built from its config block and its weights, declares what it keeps per sequence
(`cache_spec`: pages of keys / values, recurrent state slots) and maps the normed layer input h [rows, width] to its
output; the constants of a mechanism (window, kept tokens, scale, sink, decay, taps, head counts) are constructor
arguments, so another architecture can reuse a mixer with other values.

Precision: projections run on the tensor cores in bf16 with fp32 accumulation and fp32 results (`Projection`), or in true
fp32 when the model is built with dtype float32; everything between two projections (norms, scores, softmax, gates,
convolutions, decays, recurrences, the residual) is fp32, and only a projection's INPUT is rounded to bf16.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .. import _lib, ops


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class Projection:
    """y = act(x W^T + bias) * scale + addend for a weight stored [out, in]. bf16 weights with 16-byte-aligned rows go to the
    tcgen05 / small-batch GEMM (vy_gemm, fp32 result); fp32 weights and every other shape go to the fp32-FMA kernel."""

    def __init__(self, weight: torch.Tensor, tensor_cores: bool = True):
        self.weight = weight.contiguous()
        self.out_features, self.in_features = weight.shape
        self.tensor_cores = bool(tensor_cores) and weight.dtype == torch.bfloat16 and self.in_features % 8 == 0 and self.in_features >= 32 \
            and self.out_features >= 16

    def __call__(self, x: torch.Tensor, *, act: Optional[str] = None, bias: Optional[torch.Tensor] = None, scale: float = 1.0,
                 addend: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.float32, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        N = self.out_features
        if out is None:
            out = torch.empty((x.shape[0], _round_up(N, 8)), device=x.device, dtype=out_dtype)[:, :N]
        tc = self.tensor_cores and x.dtype == torch.bfloat16 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and bias is None \
            and act in (None, "none", "relu2")
        if tc:
            ops.gemm(x, self.weight, act=act, addend=addend, out=out, out_scale=scale, swap_ab=x.shape[0] <= 32)
        else:
            ops.linear_plain(x, self.weight, bias=bias, act=act, scale=scale, addend=addend, out=out)
        return out


def pack_rows(tensors: List[torch.Tensor], align: int = 8) -> Tuple[torch.Tensor, List[Tuple[int, int]]]:
    """Stacks weights that read the same input into one [sum out, in] matrix (each block padded with zero rows to a multiple
    of `align` outputs, so every block of the product starts at an aligned column). Returns the matrix and (offset, rows)
    of each block."""
    K = tensors[0].shape[1]
    spans, off = [], 0
    for t in tensors:
        spans.append((off, t.shape[0]))
        off += _round_up(t.shape[0], align)
    w = torch.zeros((off, K), dtype=tensors[0].dtype, device=tensors[0].device)
    for t, (o, n) in zip(tensors, spans):
        w[o:o + n] = t
    return w, spans


class Mixer:
    """Common surface: `cache_spec()` -> {"pages": (kv_heads, dim, vdim) | None, "states": {name: per-slot shape}};
    `input_weights()` -> the [out, in] matrices that read the layer input (packed by the layer into one projection);
    `forward(parts, batch, cache)` with `parts` the list of product blocks in the same order."""

    def cache_spec(self) -> dict:
        return {"pages": None, "states": {}}


class LightningMixer(Mixer):
    """Linear attention with one fixed decay per head: q, k, v = silu(projections), S_t = decay_h S_(t-1) + k_t v_t^T,
    o_t = S_t^T q_t; the heads' outputs are RMS-normed together, gated by sigmoid(W_g h) and projected."""

    def __init__(self, cfg: dict, w: Dict[str, torch.Tensor], eps: float, act_dtype: torch.dtype, tensor_cores: bool):
        self.heads, self.dim, self.vdim = int(cfg["heads"]), int(cfg["dim"]), int(cfg["vdim"])
        if len(cfg["decay"]) != self.heads:
            raise ValueError("lightning mixer: one decay per head expected")
        self.eps, self.act_dtype = eps, act_dtype
        dev = w["q"].device
        self.decay = torch.tensor([float(d) for d in cfg["decay"]], dtype=torch.float32, device=dev)
        self._in = [w["q"], w["k"], w["v"], w["g"]]
        self.norm = w["norm"].contiguous()
        self.o = Projection(w["o"], tensor_cores)

    def input_weights(self):
        return self._in

    def cache_spec(self):
        return {"pages": None, "states": {"S": (self.heads, self.dim, self.vdim)}}

    def forward(self, parts, batch, cache, x_residual: Optional[torch.Tensor] = None):
        q, k, v, g = parts
        o = ops.linear_attn(batch, q, k, v, self.decay, cache.states["S"], heads=self.heads, dim=self.dim, vdim=self.vdim, in_act="silu")
        og = ops.rms_norm(o, self.norm, eps=self.eps, w_mode="plain", gate=g, gate_act="sigmoid", out_dtype=self.act_dtype)
        if x_residual is not None:  # x += W_o(...) in the projection's epilogue
            return self.o(og, addend=x_residual, out=x_residual)
        return self.o(og)


class WindowSinkAttention(Mixer):
    """Softmax attention without rotation: whole-projection RMS norm of q and k (plain weights), score = q.k * scale, causal
    sliding window that also keeps the first tokens, a learned per-head sink in the denominator, and a per-head sigmoid
    output gate read from the layer input. Keys / values live in pages."""

    def __init__(self, cfg: dict, w: Dict[str, torch.Tensor], eps: float, act_dtype: torch.dtype, tensor_cores: bool,
                 kv_dtype: torch.dtype = torch.float32):
        self.heads, self.kv_heads = int(cfg["heads"]), int(cfg["kv_heads"])
        self.dim, self.vdim = int(cfg["dim"]), int(cfg["vdim"])
        if self.heads % self.kv_heads:
            raise ValueError("attention: heads must be a multiple of kv_heads")
        mask = cfg.get("mask") or {}
        self.window, self.keep_first = int(mask.get("size", 0)), int(mask.get("keep_first", 0))
        self.scale = float(cfg["scale"])
        self.eps, self.act_dtype, self.kv_dtype = eps, act_dtype, kv_dtype
        self._in = [w["q"], w["k"], w["v"], w["g"]]
        self.q_norm, self.k_norm = w["q.norm"].contiguous(), w["k.norm"].contiguous()
        self.sink = w["sink"].contiguous() if "sink" in w else None
        self.o = Projection(w["o"], tensor_cores)

    def input_weights(self):
        return self._in

    def cache_spec(self):
        return {"pages": (self.kv_heads, self.dim, self.vdim), "states": {}, "kv_dtype": self.kv_dtype}

    def forward(self, parts, batch, cache):
        q, k, v, g = parts
        qn = ops.rms_norm(q, self.q_norm, eps=self.eps, w_mode="plain", out_dtype=torch.float32)
        kn = ops.rms_norm(k, self.k_norm, eps=self.eps, w_mode="plain", out_dtype=torch.float32)
        ops.kv_page_write(batch, kn, v, cache.k_pool, cache.v_pool)
        a = ops.window_attn(batch, qn, cache.k_pool, cache.v_pool, heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim,
                            scale=self.scale, window=self.window, keep_first=self.keep_first, sink=self.sink, gate=g,
                            out_dtype=self.act_dtype)
        return self.o(a)


class GatedDeltaMixer(Mixer):
    """Gated delta rule: q / k / v pass a short causal depthwise convolution and silu, q and k become unit vectors per head
    (q also times dim^-1/2), a per-channel decay exp(-exp(A_log) softplus(W_a2 W_a1 h + dt_bias)) shrinks the state, a
    sigmoid write strength scales the delta update; the read-out is RMS-normed per head, gated by sigmoid(W_g2 W_g1 h) and
    projected."""

    def __init__(self, cfg: dict, w: Dict[str, torch.Tensor], eps: float, act_dtype: torch.dtype, tensor_cores: bool):
        self.heads, self.kv_heads = int(cfg["heads"]), int(cfg["kv_heads"])
        self.dim, self.vdim, self.taps = int(cfg["dim"]), int(cfg["vdim"]), int(cfg["conv"])
        if self.heads % self.kv_heads:
            raise ValueError("delta mixer: heads must be a multiple of kv_heads")
        self.eps, self.act_dtype = eps, act_dtype
        # q | k | v are adjacent blocks of the packed product (widths are multiples of the packing alignment or the last block),
        # so one convolution call covers all three when their channel counts need no padding; otherwise three calls
        self._in = [w["q"], w["k"], w["v"], w["b"], w["a1"], w["g1"]]
        self.conv_w = [w["q.conv"].contiguous(), w["k.conv"].contiguous(), w["v.conv"].contiguous()]
        self.a2 = Projection(w["a2"], False)  # contractions over the low rank: fp32 activations straight from the a1 / g1 blocks
        self.g2 = Projection(w["g2"], False)
        self.dt_bias = w["dt_bias"].contiguous()
        self.a_log = w["A_log"].contiguous()
        self.norm = w["norm"].contiguous()
        self.o = Projection(w["o"], tensor_cores)

    def input_weights(self):
        return self._in

    def cache_spec(self):
        qk, vv = self.kv_heads * self.dim, self.heads * self.vdim
        st = {"S": (self.heads, self.dim, self.vdim)}
        if self.taps > 1:
            st.update({"conv_q": (qk, self.taps - 1), "conv_k": (qk, self.taps - 1), "conv_v": (vv, self.taps - 1)})
        return {"pages": None, "states": st}

    def forward(self, parts, batch, cache):
        q, k, v, b, a1, g1 = parts
        dummy = cache.states["S"]
        qc = ops.causal_conv(batch, q, self.conv_w[0], cache.states.get("conv_q", dummy), act="silu", out_dtype=torch.float32)
        kc = ops.causal_conv(batch, k, self.conv_w[1], cache.states.get("conv_k", dummy), act="silu", out_dtype=torch.float32)
        vc = ops.causal_conv(batch, v, self.conv_w[2], cache.states.get("conv_v", dummy), act="silu", out_dtype=torch.float32)
        a = self.a2(a1, bias=self.dt_bias)
        g = self.g2(g1)
        o = ops.delta_rule(batch, qc, kc, vc, a, b, self.a_log, cache.states["S"], heads=self.heads, kv_heads=self.kv_heads, dim=self.dim,
                           vdim=self.vdim, unit_eps=1e-6)
        on = ops.rms_norm(o, self.norm, eps=self.eps, w_mode="plain", groups=self.heads, gate=g, gate_act="sigmoid", out_dtype=self.act_dtype)
        return self.o(on)


class ReluSquaredMLP:
    """W_down relu(W_up h)^2, the down projection adding into the fp32 residual in its epilogue."""

    def __init__(self, w: Dict[str, torch.Tensor], act_dtype: torch.dtype, tensor_cores: bool):
        self.up, self.down = Projection(w["up"], tensor_cores), Projection(w["down"], tensor_cores)
        self.act_dtype = act_dtype

    def forward(self, h: torch.Tensor, x_residual: torch.Tensor) -> torch.Tensor:
        u = self.up(h, act="relu2", out_dtype=self.act_dtype)   # squared on the fp32 accumulator in the epilogue, rounded once
        return self.down(u, addend=x_residual, out=x_residual)
