"""Zugunex: a decoder-only language model of latent-attention layers. Layers are listed in the configuration; each adds the
RMS-normed OUTPUT of its sublayers to the residual stream (x += norm1(mixer(x)); x += norm2(ff(x)), the sublayers reading x
itself, plain norm weights). The mixer is latent attention (layers/mixers.py LatentAttention: a cached low-rank latent plus
one rotated key part per token, pair rotation by position, sliding window, softmax sink, sigmoid output gate); a layer with
`kv_from: j` owns no down-projection and attends over layer j's cached rows with its own expansions and queries. The
feed-forward is dense (tanh-GELU) or a sigmoid-routed mixture of squared-ReLU experts with an optional gated shared expert
(layers/mixers.py MoEFeedForward). The reference package has no such model; it is served by the same pieces as the other
packed-step decoder here (models/gelutar.py): a configuration object read from config.json, weights loaded by tensor name, the
cache manager's pages (vyomai_b200/paged.py; a sharing layer is given the owner's pool), one `step` over a packed batch that
the batching engine, the CUDA-graph capture and the trace replayer all call, and greedy selection by vy_argmax_rows.

The residual stream, norms, rotation angles, attention scores, router scores and weights are fp32 in both dtypes; with
dtype=bfloat16 the projections read bf16 inputs on the tensor cores (fp32 results), with dtype=float32 they are fp32 FMA.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

import torch

from .. import _lib, ops
from ..layers.mixers import DenseMLP, LatentAttention, MoEFeedForward, Projection, pack_rows


class ZugunexConfig:
    """config.json of the architecture: vocab, width, norm.eps and `layers`, a list of
    {"type": "latent_attention", "mixer": {heads, dim, rot_dim, vdim, kv_rank, scale, rot: {base, dims}, mask: {size}, kv_from?},
     "mlp": null | {"kind": "dense", "ff"} | {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "scale"}, "shared": {"ff"}?}}."""

    architecture = "Zugunex"

    def __init__(self, d: dict):
        if d.get("architecture") != self.architecture:
            raise ValueError(f"not a {self.architecture} configuration: {d.get('architecture')!r}")
        self.raw = d
        self.vocab, self.width = int(d["vocab"]), int(d["width"])
        self.eps = float(d["norm"]["eps"])
        self.layers = list(d["layers"])
        for i, L in enumerate(self.layers):
            if L["type"] != "latent_attention":
                raise ValueError(f"layer {i}: unknown mixer type {L['type']!r}")
            m = L["mixer"]
            j = m.get("kv_from")
            if j is not None:
                j = int(j)
                if not 0 <= j < i or self.layers[j]["mixer"].get("kv_from") is not None:
                    raise ValueError(f"layer {i}: kv_from {j} must name an earlier layer that owns its latent")
                o = self.layers[j]["mixer"]
                if (o["kv_rank"], o["rot_dim"], o.get("rot")) != (m["kv_rank"], m["rot_dim"], m.get("rot")):
                    raise ValueError(f"layer {i}: kv_rank / rot_dim / rot differ from layer {j}'s, whose latent it reads")
            kind = (L.get("mlp") or {}).get("kind", "dense")
            if kind not in ("dense", "moe"):
                raise ValueError(f"layer {i}: unknown feed-forward kind {kind!r}")

    @classmethod
    def from_dir(cls, path: str) -> "ZugunexConfig":
        with open(os.path.join(path, "config.json")) as f:
            return cls(json.load(f))

    def tensor_shapes(self) -> Dict[str, tuple]:
        """Name -> shape of every weight the configuration implies (what a checkpoint must hold; also the recipe for random
        initialisation)."""
        W = self.width
        out: Dict[str, tuple] = {"embed": (self.vocab, W), "final.norm": (W,), "head": (self.vocab, W)}
        for i, L in enumerate(self.layers):
            p, m = f"l{i}.", L["mixer"]
            H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            out.update({p + "norm1": (W,), p + "mix.q": (H * (dn + dr), W), p + "mix.uk": (H * dn, R), p + "mix.uv": (H * dv, R),
                        p + "mix.sink": (H,), p + "mix.g": (H, W), p + "mix.o": (W, H * dv)})
            if m.get("kv_from") is None:
                out.update({p + "mix.dkv": (R + dr, W), p + "mix.dkv.norm": (R,)})
            f = L.get("mlp")
            if not f:
                continue
            out[p + "norm2"] = (W,)
            if f.get("kind", "dense") == "dense":
                out.update({p + "mlp.up": (f["ff"], W), p + "mlp.down": (W, f["ff"])})
            else:
                for e in range(f["router"]["experts"]):
                    out.update({p + f"mlp.e{e}.up": (f["expert"]["ff"], W), p + f"mlp.e{e}.down": (W, f["expert"]["ff"])})
                out[p + "mlp.router"] = (f["router"]["experts"], W)
                if f.get("shared"):
                    out.update({p + "mlp.shared.up": (f["shared"]["ff"], W), p + "mlp.shared.down": (W, f["shared"]["ff"]),
                                p + "mlp.shared.sg": (1, W)})
        return out


class _Layer:
    def __init__(self, idx: int, spec: dict, w: Dict[str, torch.Tensor], cfg: ZugunexConfig, act_dtype, tensor_cores: bool, kv_dtype,
                 sorted_min_rows: int, force_sorted: bool):
        p = f"l{idx}."
        sub = lambda pre: {k[len(pre):]: v for k, v in w.items() if k.startswith(pre)}  # noqa: E731
        self.eps, self.act_dtype = cfg.eps, act_dtype
        self.norm1 = w[p + "norm1"].contiguous()
        shared_from = spec["mixer"].get("kv_from")
        self.mixer = LatentAttention(spec["mixer"], sub(p + "mix."), cfg.eps, act_dtype, tensor_cores, kv_dtype,
                                     shared_from=None if shared_from is None else int(shared_from))
        packed, self.spans = pack_rows(self.mixer.input_weights())
        self.inp = Projection(packed, tensor_cores)   # every matrix that reads the layer input, as one product
        self.mlp, self.moe = None, False
        f = spec.get("mlp")
        if f:
            self.norm2 = w[p + "norm2"].contiguous()
            if f.get("kind", "dense") == "dense":
                self.mlp = DenseMLP(sub(p + "mlp."), act_dtype, tensor_cores, act="gelu_tanh")
            else:
                r = f["router"]
                self.mlp = MoEFeedForward(sub(p + "mlp."), r["experts"], r["top"], r.get("scale", 1.0), act_dtype, tensor_cores, act="relu2",
                                          shared=bool(f.get("shared")), sorted_min_rows=sorted_min_rows, force_sorted=force_sorted)
                self.moe = True

    def cache_specs(self):
        return [self.mixer.cache_spec()]

    def _round(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        """Room for the bf16 rounding of the residual that the next tensor-core product reads (None for fp32 models: they read x)."""
        return None if self.act_dtype == torch.float32 else torch.empty(x.shape, device=x.device, dtype=self.act_dtype)

    def forward(self, x: torch.Tensor, h: Optional[torch.Tensor], batch: ops.PackedBatch, caches, last: bool = False) -> Optional[torch.Tensor]:
        """x: the fp32 residual (updated in place); h: its rounding in the activation dtype (None: x itself is read). Every sublayer
        reads the residual itself; the norm that adds a sublayer's output into x also writes the rounding the next product reads.
        Returns the rounding of the layer's result (None for fp32 models and for the last layer, whose reader is the final norm)."""
        P = self.inp(x if h is None else h)
        y = self.mixer.forward([P[:, o:o + n] for o, n in self.spans], batch, caches[0])
        h = None if last and self.mlp is None else self._round(x)
        ops.rms_norm(y, self.norm1, eps=self.eps, w_mode="plain", accumulate=True, out=x, copy_out=h)
        if self.mlp is not None:
            hin = x if h is None else h
            y = self.mlp.forward(hin, batch) if self.moe else self.mlp.forward(hin)
            h = None if last else self._round(x)
            ops.rms_norm(y, self.norm2, eps=self.eps, w_mode="plain", accumulate=True, out=x, copy_out=h)
        return h


class ZugunexForCausalLM:
    """The model: `step(ids, batch, caches, want_rows)` runs the step's packed tokens through every layer, writing the
    sequences' latent rows into their pages in `caches` (one entry per layer: a list with the mixer's cache view; a sharing
    layer's view IS its owner's), and returns fp32 logits [len(want_rows), vocab] of the requested rows."""

    config_class = ZugunexConfig

    def __init__(self, config: ZugunexConfig, weights: Dict[str, torch.Tensor], dtype: torch.dtype = torch.bfloat16,
                 device: Optional[torch.device] = None, tensor_cores: bool = True, kv_dtype: torch.dtype = torch.float32,
                 sorted_min_rows: int = 128, force_sorted: bool = False):
        if dtype not in (torch.bfloat16, torch.float32):
            raise _lib.VyomError("ZugunexForCausalLM runs in bfloat16 or float32")
        self.config, self.dtype = config, dtype
        self.device = torch.device(device or "cuda")
        need = config.tensor_shapes()
        missing = [k for k in need if k not in weights]
        if missing:
            raise KeyError(f"checkpoint lacks {missing[:5]}{' ...' if len(missing) > 5 else ''}")
        for k, shp in need.items():
            if tuple(weights[k].shape) != tuple(shp):
                raise ValueError(f"{k}: shape {tuple(weights[k].shape)}, the configuration implies {tuple(shp)}")
        w = {k: v.to(device=self.device, dtype=dtype) for k, v in weights.items() if k in need}
        self.embed = w["embed"].contiguous()
        self.final_norm = w["final.norm"].contiguous()
        self.head = Projection(w["head"], tensor_cores)
        self.layers = [_Layer(i, L, w, config, dtype, tensor_cores, kv_dtype, sorted_min_rows, force_sorted) for i, L in enumerate(config.layers)]
        self.debug_residuals: Optional[list] = None   # set to [] to collect the residual stream after every layer

    @classmethod
    def from_pretrained(cls, path: str, dtype: torch.dtype = torch.bfloat16, device=None, **kw) -> "ZugunexForCausalLM":
        from ..checkpoint import load_safetensors
        return cls(ZugunexConfig.from_dir(path), load_safetensors(os.path.join(path, "model.safetensors")), dtype=dtype, device=device, **kw)

    @staticmethod
    def random_weights(config: ZugunexConfig, seed: int = 0) -> Dict[str, torch.Tensor]:
        """Seeded bf16 weights of the right shapes (tests, benchmarks): projections ~ N(0, 1/in), embeddings ~ N(0, 1), norm weights
        around 1, sinks ~ N(0, 1); routers ~ N(0, 1/(4 in)), so that router logits stay where an fp32 sigmoid still tells them apart
        (beyond |z| ~ 17 the scores of different experts round to the same number and the choice falls to the tie rule)."""
        g = torch.Generator().manual_seed(seed)
        out = {}
        for k, shp in config.tensor_shapes().items():
            leaf = k.split(".")[-1]
            if leaf == "embed":
                t = torch.randn(shp, generator=g)
            elif leaf == "router":
                t = torch.randn(shp, generator=g) * 0.5 / (shp[1] ** 0.5)
            elif len(shp) == 2:
                t = torch.randn(shp, generator=g) / (shp[1] ** 0.5)
            elif leaf == "sink":
                t = torch.randn(shp, generator=g)
            else:   # norm weights
                t = 1.0 + 0.1 * torch.randn(shp, generator=g)
            out[k] = t.to(torch.bfloat16)
        return out

    def cache_specs(self):
        return [L.cache_specs() for L in self.layers]

    @torch.no_grad()
    def step(self, ids: torch.Tensor, batch: ops.PackedBatch, caches, want_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        cfg = self.config
        x = ops.embed_rows(ids, self.embed, 1.0, torch.float32)
        h = None if self.dtype == torch.float32 else ops.unary(x, None, self.dtype)
        for i, (L, c) in enumerate(zip(self.layers, caches)):
            h = L.forward(x, h, batch, c, last=i == len(self.layers) - 1)
            if self.debug_residuals is not None:
                self.debug_residuals.append(x.clone())
        if want_rows is None or want_rows.numel() == 0:
            return None
        hn = ops.rms_norm(x, self.final_norm, eps=cfg.eps, w_mode="plain", row_index=want_rows, out_dtype=self.dtype)
        return self.head(hn)
