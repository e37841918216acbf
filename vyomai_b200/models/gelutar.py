"""Gelutar: a hybrid decoder-only language model. Layers are listed in the configuration; each is pre-norm
(x += mixer(norm1 x); x += ff(norm2 x)) with RMS norms whose weights are stored around zero (1 + w), a mixer that is
either `lightning` (linear attention with a fixed per-head decay) or `parallel` (windowed softmax attention with kept
first tokens and a sink, side by side with a gated delta rule; the two outputs are RMS-normed with plain weights and
averaged), and a squared-ReLU feed-forward. Embeddings are scaled on the way in, logits on the way out. The reference
package has no such model; it is served by the same pieces as the other decoders here: a configuration object read from
config.json, weights loaded by tensor name, a cache manager that gives every sequence pages and state slots
(vyomai_b200/paged.py), one `step` over a packed batch that the batching engine and the trace replayer both call, and greedy
selection by vy_argmax_rows.

The residual stream, all norms, attention scores, gates, decays and recurrent state are fp32 in both dtypes; with
dtype=bfloat16 the projections read bf16 inputs on the tensor cores (fp32 results), with dtype=float32 they are fp32 FMA.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

import torch

from .. import _lib, ops
from ..layers.mixers import GatedDeltaMixer, LightningMixer, Projection, ReluSquaredMLP, WindowSinkAttention, pack_rows


class GelutarConfig:
    """config.json of the architecture: vocab, width, embedding.scale, norm.eps, logit_scale and `layers`, a list of
    {"type": "lightning" | "parallel", "mixer": {...}, "mlp": {"kind": "dense", "ff": n} | null}."""

    architecture = "Gelutar"

    def __init__(self, d: dict):
        if d.get("architecture") != self.architecture:
            raise ValueError(f"not a {self.architecture} configuration: {d.get('architecture')!r}")
        self.raw = d
        self.vocab, self.width = int(d["vocab"]), int(d["width"])
        self.embedding_scale = float(d.get("embedding", {}).get("scale", 1.0))
        self.eps = float(d["norm"]["eps"])
        self.logit_scale = float(d.get("logit_scale", 1.0))
        self.layers = list(d["layers"])
        for i, L in enumerate(self.layers):
            if L["type"] not in ("lightning", "parallel"):
                raise ValueError(f"layer {i}: unknown mixer type {L['type']!r}")
            if L.get("mlp") and L["mlp"].get("kind", "dense") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {L['mlp'].get('kind')!r}")

    @classmethod
    def from_dir(cls, path: str) -> "GelutarConfig":
        with open(os.path.join(path, "config.json")) as f:
            return cls(json.load(f))

    def tensor_shapes(self) -> Dict[str, tuple]:
        """Name -> shape of every weight the configuration implies (what a checkpoint must hold; also the recipe for
        random initialisation)."""
        W = self.width
        out: Dict[str, tuple] = {"embed": (self.vocab, W), "final.norm": (W,), "head": (self.vocab, W)}
        for i, L in enumerate(self.layers):
            p = f"l{i}."
            out[p + "norm1"] = (W,)
            m = L["mixer"]
            if L["type"] == "lightning":
                H, dk, dv = m["heads"], m["dim"], m["vdim"]
                out.update({p + "mix.q": (H * dk, W), p + "mix.k": (H * dk, W), p + "mix.v": (H * dv, W), p + "mix.g": (H * dv, W),
                            p + "mix.o": (W, H * dv), p + "mix.norm": (H * dv,)})
            else:
                a, r = m["left"], m["right"]
                q = p + "mix.left."
                out.update({q + "q": (a["heads"] * a["dim"], W), q + "k": (a["kv_heads"] * a["dim"], W), q + "v": (a["kv_heads"] * a["vdim"], W),
                            q + "q.norm": (a["heads"] * a["dim"],), q + "k.norm": (a["kv_heads"] * a["dim"],), q + "sink": (a["heads"],),
                            q + "g": (a["heads"], W), q + "o": (W, a["heads"] * a["vdim"]), q + "out": (W,)})
                q = p + "mix.right."
                out.update({q + "q": (r["kv_heads"] * r["dim"], W), q + "k": (r["kv_heads"] * r["dim"], W), q + "v": (r["heads"] * r["vdim"], W),
                            q + "q.conv": (r["kv_heads"] * r["dim"], r["conv"]), q + "k.conv": (r["kv_heads"] * r["dim"], r["conv"]),
                            q + "v.conv": (r["heads"] * r["vdim"], r["conv"]), q + "b": (r["heads"], W), q + "A_log": (r["heads"],),
                            q + "norm": (r["vdim"],), q + "dt_bias": (r["heads"] * r["dim"],), q + "o": (W, r["heads"] * r["vdim"]),
                            q + "out": (W,)})
                # the two low ranks are not configuration: -1 stands for "whatever the checkpoint holds", and the pairs must agree
                out.update({q + "a1": (-1, W), q + "a2": (r["heads"] * r["dim"], -1), q + "g1": (-1, W), q + "g2": (r["heads"] * r["vdim"], -1)})
            if L.get("mlp"):
                out.update({p + "norm2": (W,), p + "mlp.up": (L["mlp"]["ff"], W), p + "mlp.down": (W, L["mlp"]["ff"])})
        return out


class _Layer:
    def __init__(self, idx: int, spec: dict, w: Dict[str, torch.Tensor], cfg: GelutarConfig, act_dtype, tensor_cores: bool, kv_dtype):
        p = f"l{idx}."
        sub = lambda pre: {k[len(pre):]: v for k, v in w.items() if k.startswith(pre)}  # noqa: E731
        self.kind = spec["type"]
        self.norm1 = w[p + "norm1"].contiguous()
        self.eps, self.act_dtype = cfg.eps, act_dtype
        if self.kind == "lightning":
            self.mixers = [LightningMixer(spec["mixer"], sub(p + "mix."), cfg.eps, act_dtype, tensor_cores)]
            self.out_norms = None
        else:
            self.mixers = [WindowSinkAttention(spec["mixer"]["left"], sub(p + "mix.left."), cfg.eps, act_dtype, tensor_cores, kv_dtype),
                           GatedDeltaMixer(spec["mixer"]["right"], sub(p + "mix.right."), cfg.eps, act_dtype, tensor_cores)]
            self.out_norms = [w[p + "mix.left.out"].contiguous(), w[p + "mix.right.out"].contiguous()]
        blocks: List[torch.Tensor] = []
        self.counts = []
        for m in self.mixers:
            ws = m.input_weights()
            self.counts.append(len(ws))
            blocks += ws
        packed, self.spans = pack_rows(blocks)
        self.inp = Projection(packed, tensor_cores)   # every matrix that reads norm1(x), as one product
        self.mlp = None
        if spec.get("mlp"):
            self.norm2 = w[p + "norm2"].contiguous()
            self.mlp = ReluSquaredMLP(sub(p + "mlp."), act_dtype, tensor_cores)

    def cache_specs(self):
        return [m.cache_spec() for m in self.mixers]

    def forward(self, x: torch.Tensor, batch: ops.PackedBatch, caches) -> None:
        h = ops.rms_norm(x, self.norm1, eps=self.eps, w_mode="one_plus", out_dtype=self.act_dtype)
        P = self.inp(h)
        parts = [P[:, o:o + n] for o, n in self.spans]
        if self.kind == "lightning":
            self.mixers[0].forward(parts, batch, caches[0], x_residual=x)
        else:
            at = 0
            for m, cnt, c, wn in zip(self.mixers, self.counts, caches, self.out_norms):
                y = m.forward(parts[at:at + cnt], batch, c)
                at += cnt
                ops.rms_norm(y, wn, eps=self.eps, w_mode="plain", coef=1.0 / len(self.mixers), accumulate=True, out=x)
        if self.mlp is not None:
            h2 = ops.rms_norm(x, self.norm2, eps=self.eps, w_mode="one_plus", out_dtype=self.act_dtype)
            self.mlp.forward(h2, x)


class GelutarForCausalLM:
    """The model: `step(ids, batch, caches, want_rows)` runs the step's packed tokens through every layer, updating the
    sequences' pages and state slots in `caches` (one entry per layer: a list with one cache view per mixer), and returns
    fp32 logits [len(want_rows), vocab] of the requested rows."""

    config_class = GelutarConfig

    def __init__(self, config: GelutarConfig, weights: Dict[str, torch.Tensor], dtype: torch.dtype = torch.bfloat16,
                 device: Optional[torch.device] = None, tensor_cores: bool = True, kv_dtype: torch.dtype = torch.float32):
        if dtype not in (torch.bfloat16, torch.float32):
            raise _lib.VyomError("GelutarForCausalLM runs in bfloat16 or float32")
        self.config, self.dtype = config, dtype
        self.device = torch.device(device or "cuda")
        need = config.tensor_shapes()
        missing = [k for k in need if k not in weights]
        if missing:
            raise KeyError(f"checkpoint lacks {missing[:5]}{' ...' if len(missing) > 5 else ''}")
        for k, shp in need.items():
            got = tuple(weights[k].shape)
            if len(got) != len(shp) or any(a != b for a, b in zip(got, shp) if b >= 0):
                raise ValueError(f"{k}: shape {got}, the configuration implies {tuple(shp)}")
            if k.endswith(("mix.right.a1", "mix.right.g1")) and weights[k[:-1] + "2"].shape[1] != got[0]:
                raise ValueError(f"{k}: rank {got[0]} does not match {k[:-1]}2")
        w = {k: v.to(device=self.device, dtype=dtype) for k, v in weights.items() if k in need}
        self.embed = w["embed"].contiguous()
        self.final_norm = w["final.norm"].contiguous()
        self.head = Projection(w["head"], tensor_cores)
        self.layers = [_Layer(i, L, w, config, dtype, tensor_cores, kv_dtype) for i, L in enumerate(config.layers)]
        self.debug_residuals: Optional[list] = None   # set to [] to collect the residual stream after every layer

    @classmethod
    def from_pretrained(cls, path: str, dtype: torch.dtype = torch.bfloat16, device=None, **kw) -> "GelutarForCausalLM":
        from ..checkpoint import load_safetensors
        return cls(GelutarConfig.from_dir(path), load_safetensors(os.path.join(path, "model.safetensors")), dtype=dtype, device=device, **kw)

    @staticmethod
    def random_weights(config: GelutarConfig, seed: int = 0, low_rank=16) -> Dict[str, torch.Tensor]:
        """Seeded bf16 weights of the right shapes (tests, benchmarks): projections ~ N(0, 1/in), norm weights and sinks small,
        A_log and dt_bias in the range that gives decays between ~0.5 and ~1. `low_rank`: one rank, or (decay rank, gate rank)
        of the delta mixer's two factored projections."""
        g = torch.Generator().manual_seed(seed)
        ranks = (low_rank, low_rank) if isinstance(low_rank, int) else tuple(low_rank)
        out = {}
        for k, shp in config.tensor_shapes().items():
            leaf = k.split(".")[-1]
            if -1 in shp:
                rank = ranks[0] if leaf in ("a1", "a2") else ranks[1]
                shp = tuple(rank if n < 0 else n for n in shp)
            if len(shp) == 2 and leaf != "conv":
                t = torch.randn(shp, generator=g) / (shp[1] ** 0.5)
                if leaf == "embed":
                    t = torch.randn(shp, generator=g)
            elif leaf == "conv":
                t = torch.randn(shp, generator=g) * 0.5
            elif leaf == "A_log":
                t = torch.rand(shp, generator=g) * 2.0 - 2.0
            elif leaf == "dt_bias":
                t = torch.rand(shp, generator=g) * 2.0 - 3.0
            elif leaf == "sink":
                t = torch.randn(shp, generator=g)
            elif k.endswith("q.norm") or k.endswith("k.norm") or leaf in ("out", "norm") and ".mix." in k:
                t = 1.0 + 0.1 * torch.randn(shp, generator=g)
            else:
                t = 0.1 * torch.randn(shp, generator=g)
            out[k] = t.to(torch.bfloat16)
        return out

    def cache_specs(self):
        return [L.cache_specs() for L in self.layers]

    @torch.no_grad()
    def step(self, ids: torch.Tensor, batch: ops.PackedBatch, caches, want_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        cfg = self.config
        x = ops.embed_rows(ids, self.embed, cfg.embedding_scale, torch.float32)
        for L, c in zip(self.layers, caches):
            L.forward(x, batch, c)
            if self.debug_residuals is not None:
                self.debug_residuals.append(x.clone())
        if want_rows is None or want_rows.numel() == 0:
            return None
        hn = ops.rms_norm(x, self.final_norm, eps=cfg.eps, w_mode="one_plus", row_index=want_rows, out_dtype=self.dtype)
        return self.head(hn, scale=cfg.logit_scale)
