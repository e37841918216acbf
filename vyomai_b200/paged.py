"""Paged kv-cache and continuous batching for the decoder family.

Host-side mirror of `Examples/simple_vllm.ipynb` cell 2 of the reference — `SequenceState`, `PagedKVManager`
(`can_allocate` / `allocate` / `free`, pools of shape (max_blocks, block_size, kv_heads, head_dim) per layer) and
`ContinuousBatchEngine` (`add_sequence`, `step`, waiting room, greedy next token, eos / length retirement) — on top of
`vy_attn_decode`'s paged mode: one kernel launch per layer does the new token's RoPE, writes its k/v into the
sequence's current block (the notebook's `k_cache[slots // block_size, slots % block_size] = k`) and attends over the
blocks named by the block table with a per-row context length (the notebook's
`flash_attn_with_kvcache(q, k_cache, v_cache, cache_seqlens=..., block_table=..., causal=True)`).

Differences from the notebook, on purpose:
  * the model is this package's `DecoderModel` (head_dim 64, LayerNorm / GELU blocks), not the notebook's Qwen3 clone;
  * a step that holds both prefilling and decoding sequences runs the prefills (one forward per new sequence, k/v
    scattered into its blocks) AND a proper paged decode for the others — the notebook sends such a mixed batch through
    `flash_attn_varlen_func` over the new tokens only, so a decoding sequence attends to nothing but its own token
    during that step;
  * eos ids are a constructor argument instead of the hard-wired Qwen ids.
"""
from __future__ import annotations

import itertools
from collections import deque

import numpy as np
from typing import Dict, Iterable, List

import torch

from . import functional as F
from . import ops
from .layers.kv_cache import StaticCacheOne


class SequenceState:
    """Runtime state of one request (notebook: SequenceState)."""

    def __init__(self, sid: int, prompt_ids: List[int], max_gen_len: int, block_size: int, device):
        self.id, self.device, self.block_size = sid, device, block_size
        p_len = len(prompt_ids)
        self.max_total_len = p_len + max_gen_len
        self.tokens = torch.zeros(self.max_total_len, dtype=torch.long, device=device)
        self.tokens[:p_len] = torch.tensor(prompt_ids, dtype=torch.long, device=device)
        self.num_tokens, self.is_prefill = p_len, True
        max_blocks = (self.max_total_len + block_size - 1) // block_size
        self.block_table = torch.zeros(max_blocks, dtype=torch.int32, device=device)  # which pool blocks hold this sequence
        self.block_count = 0

    def slots(self, start: int, end: int) -> torch.Tensor:
        """Pool slot (block * block_size + offset) of token positions [start, end)."""
        idx = torch.arange(start, end, device=self.device)
        return self.block_table[idx // self.block_size].long() * self.block_size + idx % self.block_size


class PagedKVManager:
    """Block pools (max_blocks, block_size, kv_heads, 64) per layer and a free list (notebook: PagedKVManager)."""

    def __init__(self, model, max_blocks: int, block_size: int, dtype=None, device=None):
        att = model.all_layer[0].attention
        self.block_size = block_size
        self.kv_heads, self.head_dim = att._kv_heads, F.HEAD_DIM
        dev = device or model.word_embeddings.weight.device
        dtype = dtype or model.word_embeddings.weight.dtype
        self.free_blocks = deque(range(max_blocks))
        shape = (max_blocks, block_size, self.kv_heads, self.head_dim)
        self.k_cache = [torch.zeros(shape, device=dev, dtype=dtype) for _ in model.all_layer]
        self.v_cache = [torch.zeros(shape, device=dev, dtype=dtype) for _ in model.all_layer]

    def can_allocate(self, num_tokens: int) -> bool:
        """Enough free blocks for a prompt of `num_tokens`?"""
        return len(self.free_blocks) >= (num_tokens + self.block_size - 1) // self.block_size

    def allocate(self, state: SequenceState) -> None:
        needed = (state.num_tokens + self.block_size - 1) // self.block_size
        while state.block_count < needed:
            if not self.free_blocks:
                raise RuntimeError("KV Cache full! (Engine should have prevented this)")
            state.block_table[state.block_count] = self.free_blocks.popleft()
            state.block_count += 1

    def free(self, state: SequenceState) -> None:
        for i in range(state.block_count):
            self.free_blocks.append(int(state.block_table[i]))
        state.block_count = 0


class ContinuousBatchEngine:
    """Greedy continuous batching over a paged cache (notebook: ContinuousBatchEngine)."""

    def __init__(self, model, kv_mgr: PagedKVManager, max_batch_size: int = 16, eos_token_ids: Iterable[int] = ()):
        if model._rope is None:
            raise ValueError("ContinuousBatchEngine supports RoPE models (positions enter only through the attention kernel)")
        self.model = model.eval()
        self.kv_mgr = kv_mgr
        self.active: Dict[int, SequenceState] = {}
        self.id_gen = itertools.count()
        self.device = model.word_embeddings.weight.device
        self.max_batch = max_batch_size
        self.eos = set(int(t) for t in eos_token_ids)
        self.waiting_room: deque = deque()

    def add_sequence(self, prompt_ids: List[int], max_gen_len: int = 128) -> int:
        """Queues a request; it becomes active when the pool has blocks for its prompt."""
        # every position the sequence can reach must have a row in the model's position / RoPE tables: the decode kernel
        # indexes them without passing through DecoderModel.forward's own check
        self.model._check_positions(len(prompt_ids) + max_gen_len)
        sid = next(self.id_gen)
        self.waiting_room.append({"sid": sid, "prompt_ids": list(prompt_ids), "max_gen_len": max_gen_len})
        return sid

    def _try_schedule_waiting(self) -> None:
        while self.waiting_room and len(self.active) < self.max_batch:
            req = self.waiting_room[0]
            if not self.kv_mgr.can_allocate(len(req["prompt_ids"])):
                break  # pool full: retry after some sequence retires
            self.waiting_room.popleft()
            self.active[req["sid"]] = SequenceState(req["sid"], req["prompt_ids"], req["max_gen_len"], self.kv_mgr.block_size,
                                                    self.device)

    # ---- one prompt: ordinary prefill, then its k/v rows are scattered into the sequence's blocks ----
    @torch.no_grad()
    def _prefill(self, s: SequenceState) -> int:
        m, mgr = self.model, self.kv_mgr
        P = s.num_tokens
        cache = StaticCacheOne(m.config, max_cache_len=P, batch_size=1, dtype=mgr.k_cache[0].dtype)
        if cache.heads != mgr.kv_heads:  # the cache sizes its heads from the config alone (quirk Q12): follow the model
            shape = (1, mgr.kv_heads, P, mgr.head_dim)
            cache.key_cache = [torch.zeros(shape, dtype=cache.dtype, device=cache.device) for _ in m.all_layer]
            cache.value_cache = [torch.zeros(shape, dtype=cache.dtype, device=cache.device) for _ in m.all_layer]
        ids = s.tokens[:P].view(1, P)
        out = m(ids, attention_mask=torch.ones_like(ids), use_cache=True, kv_cache=cache, start_pos=0)
        slots = s.slots(0, P)
        for li in range(len(m.all_layer)):
            mgr.k_cache[li].view(-1, mgr.kv_heads, mgr.head_dim)[slots] = cache.key_cache[li][0, :, :P].transpose(0, 1)
            mgr.v_cache[li].view(-1, mgr.kv_heads, mgr.head_dim)[slots] = cache.value_cache[li][0, :, :P].transpose(0, 1)
        return int(ops.argmax_rows(out.logits[0, -1:].contiguous())[0])

    # ---- all decoding sequences: one batched single-token step over the paged pools ----
    @torch.no_grad()
    def _decode(self, states: List[SequenceState]) -> List[int]:
        m, mgr = self.model, self.kv_mgr
        B = len(states)
        T = m.word_embeddings.weight.dtype
        tok = torch.stack([s.tokens[s.num_tokens - 1] for s in states])
        seqlens = torch.tensor([s.num_tokens - 1 for s in states], dtype=torch.int32, device=self.device)
        width = max(s.block_table.numel() for s in states)
        table = torch.zeros((B, width), dtype=torch.int32, device=self.device)
        for i, s in enumerate(states):
            table[i, : s.block_table.numel()] = s.block_table
        longest = max(s.num_tokens - 1 for s in states)
        x = m._embed(tok.view(B, 1), 0)  # [B, H]
        cos, sin = m._rope.get(x.device, T)
        for li, layer in enumerate(m.all_layer):
            att = layer.attention
            w_qkv, b_qkv = F.pack_linears(att._packed())
            qkv = F._lin(x, w_qkv, b_qkv)
            a = ops.attn_decode(qkv, mgr.k_cache[li], mgr.v_cache[li], longest, att.num_attention_heads, att._kv_heads, cos, sin,
                                out_dtype=T, seqlens=seqlens, block_table=table)
            y, _ = F.self_output(a, x, att.out.dense, att.out.layernorm)
            ff = layer.feed_forward
            x, _ = F.feed_forward(y, x, ff.intermediate, ff.out, ff.layernorm, act=ff._act_name)
        head = m.lm_head
        logits, _ = F.lm_head(x, head.dense, head.layer_norm, head.decoder.weight, head.bias)
        return ops.argmax_rows(logits).tolist()

    def step(self) -> Dict[int, List[int]]:
        """One engine iteration: schedule, grow block tables, prefill the new sequences, decode the others, retire the
        finished ones. Returns {sequence id: all its tokens} for the sequences that finished in this step."""
        self._try_schedule_waiting()
        if not self.active:
            return {}
        states = list(self.active.values())
        for s in states:
            self.kv_mgr.allocate(s)
        nxt: Dict[int, int] = {}
        decoding = [s for s in states if not s.is_prefill]
        for s in states:
            if s.is_prefill:
                nxt[s.id] = self._prefill(s)
        if decoding:
            for s, t in zip(decoding, self._decode(decoding)):
                nxt[s.id] = t
        finished: Dict[int, List[int]] = {}
        for s in states:
            token_id = nxt[s.id]
            s.is_prefill = False
            s.tokens[s.num_tokens] = token_id
            s.num_tokens += 1
            if token_id in self.eos or s.num_tokens >= s.max_total_len:
                finished[s.id] = s.tokens[: s.num_tokens].tolist()
                self.kv_mgr.free(s)
                del self.active[s.id]
        return finished


# ==== hybrid models: pages for attention layers, state slots for recurrent layers, packed steps ====
class LayerCacheView:
    """What one mixer sees of the manager: its page pools (attention) and / or its per-slot state tensors (recurrences)."""

    def __init__(self):
        self.k_pool: torch.Tensor = None
        self.v_pool: torch.Tensor = None
        self.states: Dict[str, torch.Tensor] = {}
        self.step_rows: torch.Tensor = None   # scratch of the running step (a mixer may leave its packed rows for layers that share its pages)


class HybridSequence:
    """One request of a hybrid model: its tokens (host side), how many of them the cache already holds, the pages that hold its
    keys / values and the slot that holds its recurrent state."""

    def __init__(self, sid, tokens: List[int], max_total_len: int = 0):
        self.id, self.tokens, self.max_total_len = sid, list(tokens), max_total_len
        self.num_cached = 0
        self.blocks: List[int] = []
        self.slot = -1
        self._blocks_np = None   # `blocks` as an int32 array, rebuilt when the list changed (single-token steps copy it every step)

    def blocks_array(self):
        if self._blocks_np is None or len(self._blocks_np) != len(self.blocks):
            self._blocks_np = np.asarray(self.blocks, dtype=np.int32)
        return self._blocks_np


class HybridCacheManager:
    """Pages and state slots for a model whose layers declare `cache_specs()` (per layer, per mixer:
    {"pages": (kv_heads, dim, vdim) | None, "states": {name: per-slot shape}}). Attention mixers get pools
    [num_blocks, block_size, kv_heads, dim | vdim] addressed through each sequence's block list — the same page scheme as
    PagedKVManager above (vdim 0: one pool only, for mixers whose values are part of the key row); a mixer that declares
    "pages_from": (layer, mixer) owns no pool and is handed the view of the mixer it names (layers that attend over another
    layer's cached rows); recurrent mixers get fp32 tensors [num_slots, *shape] addressed by the sequence's slot. Both
    grow on demand, so `max_tokens` / `max_seqs` are sizing hints, not limits. A slot or page handed out again is not
    cleared: a sequence whose first position is 0 never reads what its slot held, and pages are written before they are
    read."""

    def __init__(self, model, max_tokens: int = 4096, block_size: int = 16, max_seqs: int = 8, device=None):
        self.block_size = int(block_size)
        self.device = torch.device(device or model.device)
        self._specs = model.cache_specs()
        self.has_pages = any(s["pages"] for layer in self._specs for s in layer)
        self.views: List[List[LayerCacheView]] = [[LayerCacheView() for _ in layer] for layer in self._specs]
        for li, layer in enumerate(self._specs):
            for mi, spec in enumerate(layer):
                src = spec.get("pages_from")
                if src is None:
                    continue
                lj, mj = int(src[0]), int(src[1])
                if not (0 <= lj < len(self._specs) and 0 <= mj < len(self._specs[lj]) and self._specs[lj][mj].get("pages")):
                    raise ValueError(f"layer {li}: pages_from {src} does not name a mixer that owns pages")
                self.views[li][mi] = self.views[lj][mj]   # the same object: growing the owner's pools is seen here too
        self.num_blocks = 0
        self.num_slots = 0
        self.generation = 0
        self.free_blocks: deque = deque()
        self.free_slots: deque = deque()
        self._grow_slots(max(1, int(max_seqs)))
        if self.has_pages:
            self._grow_blocks((max(1, int(max_tokens)) + self.block_size - 1) // self.block_size + max(1, int(max_seqs)))

    def _grow_blocks(self, n_more: int) -> None:
        new_total = self.num_blocks + n_more
        for layer, views in zip(self._specs, self.views):
            for spec, view in zip(layer, views):
                if not spec["pages"]:
                    continue
                g, dk, dv = spec["pages"]
                dt = spec.get("kv_dtype", torch.float32)
                for name, d in (("k_pool", dk), ("v_pool", dv)):
                    if d == 0:
                        continue
                    new = torch.zeros((new_total, self.block_size, g, d), device=self.device, dtype=dt)
                    old = getattr(view, name)
                    if old is not None:
                        new[: self.num_blocks] = old
                    setattr(view, name, new)
        self.free_blocks.extend(range(self.num_blocks, new_total))
        self.num_blocks = new_total
        self.generation += 1   # pool tensors were replaced: captured steps that point at the old ones are stale

    def _grow_slots(self, n_more: int) -> None:
        new_total = self.num_slots + n_more
        for layer, views in zip(self._specs, self.views):
            for spec, view in zip(layer, views):
                for name, shape in spec["states"].items():
                    new = torch.zeros((new_total,) + tuple(shape), device=self.device, dtype=torch.float32)
                    if name in view.states:
                        new[: self.num_slots] = view.states[name]
                    view.states[name] = new
        self.free_slots.extend(range(self.num_slots, new_total))
        self.num_slots = new_total
        self.generation += 1

    def blocks_for(self, n_tokens: int) -> int:
        return (n_tokens + self.block_size - 1) // self.block_size if self.has_pages else 0

    def can_allocate(self, n_tokens: int) -> bool:
        """Room for a NEW sequence of n_tokens without growing?"""
        return len(self.free_blocks) >= self.blocks_for(n_tokens) and len(self.free_slots) >= 1

    def allocate(self, seq: HybridSequence, n_tokens: int) -> None:
        """Makes `seq` own a slot and enough pages for its first n_tokens positions (growing the pools if they ran out)."""
        if seq.slot < 0:
            if not self.free_slots:
                self._grow_slots(self.num_slots)
            seq.slot = self.free_slots.popleft()
        need = self.blocks_for(n_tokens) - len(seq.blocks)
        if need > len(self.free_blocks):
            self._grow_blocks(max(need - len(self.free_blocks), self.num_blocks // 2, 1))
        for _ in range(max(need, 0)):
            seq.blocks.append(self.free_blocks.popleft())
            seq._blocks_np = None

    def free(self, seq: HybridSequence) -> None:
        self.free_blocks.extend(seq.blocks)
        seq.blocks = []
        seq._blocks_np = None
        if seq.slot >= 0:
            self.free_slots.append(seq.slot)
            seq.slot = -1
        seq.num_cached = 0


class _CapturedStep:
    """One single-token step of `n` sequences with a block table `width` pages wide, captured into a CUDA graph. The step's
    integers (token rows, positions, slots, block table, ids) live in one static device buffer that every replay refreshes
    from pinned host memory; the logits of all n rows come back in a static tensor. Capturing runs nothing, so the states
    and pages advance only on replay. Valid for the pool tensors of the manager generation it was captured under."""

    def __init__(self, engine: "HybridBatchEngine", n: int, width: int):
        import os
        from . import _lib
        self.n = n
        _, total = engine._layout(n, width, n, n)
        self.flat = torch.zeros(total, dtype=torch.int32, device=engine.device)
        self.host = torch.zeros(total, dtype=torch.int32).pin_memory()
        self.host_np = self.host.numpy()   # the same pinned memory, filled in place by the engine
        self.copied = None
        batch, ids_t, rows_t = engine._views(self.flat, n, width, n, n, 1)
        self.graph = torch.cuda.CUDAGraph()
        pdl = os.environ.get("VY_DECODE_PDL", "1") != "0"   # each short kernel's launch overlaps its predecessor's tail
        prev = _lib.lib().vy_set_pdl(1) if pdl else None
        try:
            with torch.cuda.graph(self.graph), torch.no_grad():
                self.logits = engine.model.step(ids_t, batch, engine.cache.views, rows_t)
        finally:
            if pdl:
                _lib.lib().vy_set_pdl(prev)

    def begin(self):
        """The pinned staging array, free to be overwritten (the previous replay's upload has left it)."""
        if self.copied is not None:
            self.copied.synchronize()
        return self.host_np

    def launch(self) -> torch.Tensor:
        self.flat.copy_(self.host, non_blocking=True)
        self.copied = torch.cuda.Event()
        self.copied.record()
        self.graph.replay()
        return self.logits

    def replay(self, host_ints: torch.Tensor) -> torch.Tensor:
        self.begin()[:] = host_ints.numpy()
        return self.launch()


class HybridBatchEngine:
    """Continuous batching for hybrid models, the counterpart of ContinuousBatchEngine for models with a packed `step`
    (models/gelutar.py): every engine iteration is ONE model step over the concatenated new tokens of all live
    sequences — whole prompts of the sequences that start, one token of those that decode — so nothing is padded and
    a sequence's logits do not depend on its neighbours. `step()` is the greedy generation loop (waiting room, eos /
    length retirement as above); `feed()` / `release()` advance named sequences by GIVEN tokens and return the logits of
    chosen rows (replaying a recorded trace, scoring, teacher forcing) through the same step and manager."""

    def __init__(self, model, cache_mgr: HybridCacheManager, max_batch_size: int = 16, eos_token_ids: Iterable[int] = (),
                 use_graph: bool = True):
        self.model, self.cache = model, cache_mgr
        self.device = cache_mgr.device
        self.max_batch = max_batch_size
        self.eos = set(int(t) for t in eos_token_ids)
        self.active: Dict[object, HybridSequence] = {}
        self.waiting_room: deque = deque()
        self.id_gen = itertools.count()
        # single-token steps are a chain of short kernels whose arguments all live in device arrays: the second time a
        # (batch size, table width) shape comes up it is captured into a CUDA graph and replayed from then on
        self.use_graph = bool(use_graph) and self.device.type == "cuda"
        self._graphs: Dict[tuple, "_CapturedStep"] = {}
        self._seen: Dict[tuple, int] = {}

    # ---- the shared step ----
    @staticmethod
    def _layout(n: int, width: int, n_ids: int, n_rows: int):
        """Offsets of cu_tokens | pos0 | slot | block table | ids | wanted rows inside the step's one int32 staging buffer."""
        sizes = (n + 1, n, n, n * width, n_ids, n_rows)
        offs, at = [], 0
        for k in sizes:
            offs.append((at, k))
            at += k
        return offs, at

    def _views(self, flat: torch.Tensor, n: int, width: int, n_ids: int, n_rows: int, max_new: int, all_start: bool = False):
        offs, _ = self._layout(n, width, n_ids, n_rows)
        cu_t, pos_t, slot_t, table_t, ids_t, rows_t = (flat[o:o + k] for o, k in offs)
        batch = ops.PackedBatch(cu_t, pos_t, slot_t, max_new, table_t.view(n, width) if self.cache.has_pages else None, self.cache.block_size,
                                all_start=all_start)
        return batch, ids_t, rows_t

    @torch.no_grad()
    def _run(self, work: List, want: List[List[int]]) -> torch.Tensor:
        """work: [(sequence, new tokens)]; want[i]: offsets among sequence i's new tokens whose logits are returned
        (in order). Extends the sequences' pages, runs the model step, advances `num_cached`."""
        mgr = self.cache
        n = len(work)
        cu, pos0, slot, ids, rows = [0], [], [], [], []
        for (seq, toks), w in zip(work, want):
            if not toks:
                raise ValueError("a sequence in a step needs at least one new token")
            mgr.allocate(seq, seq.num_cached + len(toks))
            for o in w:
                if not 0 <= o < len(toks):
                    raise ValueError(f"wanted offset {o} outside the {len(toks)} new tokens")
                rows.append(cu[-1] + o)
            pos0.append(seq.num_cached)
            slot.append(seq.slot)
            ids += [int(t) for t in toks]
            cu.append(cu[-1] + len(toks))
        max_new = max(len(t) for _, t in work)
        width = max(1, max(len(seq.blocks) for seq, _ in work))
        single = max_new == 1 and self.use_graph
        if single:   # few distinct table widths, so few captures
            width = max(8, 1 << (width - 1).bit_length())
        if single:
            key = (n, width, mgr.generation)
            if self._graphs and next(iter(self._graphs))[2] != mgr.generation:
                self._graphs.clear()   # the pools were re-allocated: those captures point at freed tensors
            cap = self._graphs.get(key)
            if cap is None and self._seen.get(key, 0) >= 1:
                if len(self._graphs) >= 32:
                    self._graphs.clear()
                cap = self._graphs[key] = _CapturedStep(self, n, width)
            self._seen[key] = self._seen.get(key, 0) + 1
            # the step's integers go straight into the (pinned) staging array: no Python list of the block table per step
            offs, total = self._layout(n, width, n, n)
            buf = cap.begin() if cap is not None else np.empty(total, dtype=np.int32)
            (o_cu, _), (o_pos, _), (o_slot, _), (o_tab, _), (o_ids, _), (o_rows, _) = offs
            buf[o_cu:o_cu + n + 1] = np.arange(n + 1, dtype=np.int32)
            buf[o_pos:o_pos + n] = pos0
            buf[o_slot:o_slot + n] = slot
            tab = buf[o_tab:o_tab + n * width].reshape(n, width)
            tab[:] = 0
            for i, (seq, _) in enumerate(work):
                b = seq.blocks_array()
                tab[i, :len(b)] = b
            buf[o_ids:o_ids + n] = ids
            buf[o_rows:o_rows + n] = np.arange(n, dtype=np.int32)
            if cap is not None:
                all_rows = cap.launch()
            else:
                flat = torch.from_numpy(buf)
                flat = flat.pin_memory().to(self.device, non_blocking=True)
                batch, ids_t, rows_t = self._views(flat, n, width, n, n, 1)
                all_rows = self.model.step(ids_t, batch, mgr.views, rows_t)
            if not rows:
                logits = None
            elif rows == list(range(n)):
                logits = all_rows.clone() if cap is not None else all_rows   # every row wanted, in order (a replay's output buffer is reused)
            else:
                logits = all_rows[torch.tensor(rows, dtype=torch.long, device=self.device)]
        else:
            table = []
            for seq, _ in work:
                table += seq.blocks + [0] * (width - len(seq.blocks))
            flat = torch.tensor(cu + pos0 + slot + table + ids + rows, dtype=torch.int32)
            if self.device.type == "cuda":   # one pinned staging buffer, one host-to-device copy per step
                flat = flat.pin_memory().to(self.device, non_blocking=True)
            batch, ids_t, rows_t = self._views(flat, n, width, len(ids), len(rows), max_new, all_start=not any(pos0))
            logits = self.model.step(ids_t, batch, mgr.views, rows_t if rows else None)
        for seq, toks in work:
            seq.num_cached += len(toks)
        return logits

    # ---- given tokens ----
    def feed(self, entries: List) -> torch.Tensor:
        """entries: [(key, tokens, want offsets)]; unknown keys start new sequences. Returns fp32 logits [sum(len(want)), vocab]
        (None when nothing is wanted)."""
        work, want = [], []
        for key, toks, w in entries:
            seq = self.active.get(key)
            if seq is None:
                seq = self.active[key] = HybridSequence(key, [])
            seq.tokens += list(toks)
            work.append((seq, list(toks)))
            want.append(list(w))
        return self._run(work, want)

    def release(self, keys: Iterable) -> None:
        for key in keys:
            seq = self.active.pop(key, None)
            if seq is not None:
                self.cache.free(seq)

    # ---- greedy generation ----
    def add_sequence(self, prompt_ids: List[int], max_gen_len: int = 128) -> int:
        sid = next(self.id_gen)
        self.waiting_room.append(HybridSequence(sid, prompt_ids, len(prompt_ids) + max_gen_len))
        return sid

    def _try_schedule_waiting(self) -> None:
        while self.waiting_room and len(self.active) < self.max_batch:
            seq = self.waiting_room[0]
            if self.active and not self.cache.can_allocate(len(seq.tokens)):
                break  # pools full: retry after some sequence retires (an empty engine grows the pools instead)
            self.waiting_room.popleft()
            self.active[seq.id] = seq

    def step(self) -> Dict[int, List[int]]:
        """One iteration: admit waiting sequences, run prompts and single tokens as one packed step, pick each sequence's next
        token greedily, retire finished sequences. Returns {sequence id: all its tokens} for those that finished."""
        self._try_schedule_waiting()
        if not self.active:
            return {}
        seqs = list(self.active.values())
        work = [(s, s.tokens[s.num_cached:]) for s in seqs]
        logits = self._run(work, [[len(t) - 1] for _, t in work])
        nxt = ops.argmax_rows(logits).tolist()
        finished: Dict[int, List[int]] = {}
        for s, t in zip(seqs, nxt):
            s.tokens.append(int(t))
            if int(t) in self.eos or len(s.tokens) >= s.max_total_len:
                finished[s.id] = list(s.tokens)
                self.cache.free(s)
                del self.active[s.id]
        return finished

    def generate(self, prompts: List[List[int]], max_new_tokens: int = 16) -> List[List[int]]:
        """Greedy continuations of `prompts` (all queued at once; the waiting room and the batch limit decide the schedule)."""
        sids = [self.add_sequence(p, max_new_tokens) for p in prompts]
        done: Dict[int, List[int]] = {}
        while self.active or self.waiting_room:
            done.update(self.step())
        return [done[s] for s in sids]
