"""The hybrid decoder's mechanisms one at a time: each packed-batch kernel (csrc/seqmix.cu, csrc/linear_plain.cu) against the
float64 statement of the same mechanism in oracle/hybrid_oracle.py, on batches of unequal sequences that own shuffled pages
and slots, fed whole, in portions and token by token. Inputs are fp32, so the tolerance is fp32 rounding (1e-4 of the
output's largest magnitude). Where random data would hide a fault — a key far back, the first kept tokens, a window's edge,
the sink — the inputs are built so that one score dominates."""
import math

import pytest
import torch

from oracle import hybrid_oracle as O
from tests.hybrid_util import rel_err, shuffled_batch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ops():
    from vyomai_b200 import ops
    return ops


@pytest.mark.parametrize("groups,w_mode,gated", [(1, "one_plus", False), (3, "plain", True), (1, None, False), (2, "plain", False)])
def test_rms_norm_variants(groups, w_mode, gated):
    ops = _ops()
    g = torch.Generator().manual_seed(1)
    T, width = 7, 20
    x = torch.randn(T, groups * width, generator=g) * 3
    w = torch.randn(width, generator=g) * 0.3
    gate = torch.randn(T, groups * width, generator=g)
    ref = O.rms(x.double().view(T, groups, width), 1e-5)
    if w_mode == "plain":
        ref = ref * w.double()
    elif w_mode == "one_plus":
        ref = ref * (1 + w.double())
    ref = ref.reshape(T, -1)
    if gated:
        ref = ref * torch.sigmoid(gate.double())
    got = ops.rms_norm(x.to(DEV), w.to(DEV) if w_mode else None, eps=1e-5, w_mode=w_mode, groups=groups, gate=gate.to(DEV) if gated else None)
    assert rel_err(got.cpu(), ref) < 1e-5
    # accumulate with a coefficient, reading chosen rows
    idx = torch.tensor([5, 0, 5], dtype=torch.int32)
    acc = torch.randn(3, groups * width, generator=g)
    out = acc.to(DEV).clone()
    ops.rms_norm(x.to(DEV), w.to(DEV) if w_mode else None, eps=1e-5, w_mode=w_mode, groups=groups, coef=0.5, accumulate=True,
                 row_index=idx.to(DEV), out=out)
    ref2 = acc.double() + 0.5 * (ref[idx.long()] / (torch.sigmoid(gate.double()[idx.long()]) if gated else 1.0))
    assert rel_err(out.cpu(), ref2) < 1e-5


@pytest.mark.parametrize("M,N,K", [(1, 5, 3), (9, 33, 70), (40, 24, 7)])
def test_linear_plain_any_shape(M, N, K):
    ops = _ops()
    g = torch.Generator().manual_seed(2)
    x, w, b, add = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g), torch.randn(N, generator=g), torch.randn(M, N, generator=g)
    got = ops.linear_plain(x.to(DEV), w.to(DEV), bias=b.to(DEV), act="relu2", scale=0.7, addend=add.to(DEV))
    ref = torch.relu(x.double() @ w.double().T + b.double()) ** 2 * 0.7 + add.double()
    assert rel_err(got.cpu(), ref) < 1e-5
    gotb = ops.linear_plain(x.to(DEV).bfloat16(), w.to(DEV).bfloat16(), out_dtype=torch.float32)
    refb = x.bfloat16().double() @ w.bfloat16().double().T
    assert rel_err(gotb.cpu(), refb) < 1e-5


def _attend(ops, q, k, v, lengths, cuts_per_seq, *, H, G, dk, dv, scale, window, keep, sink, gate, bs=4):
    """Runs the sequences through page write + attention in the given portions (all sequences advance together; a sequence whose
    portions ran out drops out of the batch). q/k/v/gate are lists of per-sequence CPU tensors. Returns per-sequence outputs."""
    n = len(lengths)
    done = [0] * n
    outs = [[] for _ in range(n)]
    batch0, table, slots, n_blocks, _ = shuffled_batch(lengths, [0] * n, bs, DEV, seed=5)
    kp = torch.full((n_blocks, bs, G, dk), float("nan"), device=DEV)   # a page read before it is written shows as NaN
    vp = torch.full((n_blocks, bs, G, dv), float("nan"), device=DEV)
    cuts = [list(c) for c in cuts_per_seq]
    while any(d < L for d, L in zip(done, lengths)):
        live = [i for i in range(n) if done[i] < lengths[i]]
        take = [min(cuts[i].pop(0) if cuts[i] else 1, lengths[i] - done[i]) for i in live]
        cu = [0]
        for t in take:
            cu.append(cu[-1] + t)
        ti = lambda vals: torch.tensor(vals, dtype=torch.int32, device=DEV)  # noqa: E731
        width = len(table[0])
        batch = ops.PackedBatch(ti(cu), ti([done[i] for i in live]), ti([slots[i] for i in live]), max(take),
                                ti([table[i] for i in live]).view(len(live), width), bs)
        cat = lambda src: torch.cat([src[i][done[i]:done[i] + t] for i, t in zip(live, take)]).to(DEV).contiguous()  # noqa: E731
        ops.kv_page_write(batch, cat(k).view(-1, G * dk), cat(v).view(-1, G * dv), kp, vp)
        o = ops.window_attn(batch, cat(q).view(-1, H * dk), kp, vp, heads=H, kv_heads=G, dim=dk, vdim=dv, scale=scale, window=window,
                            keep_first=keep, sink=sink.to(DEV) if sink is not None else None, gate=cat(gate) if gate is not None else None,
                            out_dtype=torch.float32).cpu()
        for j, (i, t) in enumerate(zip(live, take)):
            outs[i].append(o[cu[j]:cu[j + 1]])
            done[i] += t
    return [torch.cat(o) for o in outs]


def _attention_case(lengths, H, G, dk, dv, seed, spikes=()):
    g = torch.Generator().manual_seed(seed)
    q = [torch.randn(L, H, dk, generator=g) for L in lengths]
    k = [torch.randn(L, G, dk, generator=g) for L in lengths]
    v = [torch.randn(L, G, dv, generator=g) for L in lengths]
    gate = [torch.randn(L, H, generator=g) for L in lengths]
    for s, i, j, h in spikes:   # key j of sequence s points along query (i, head h): its score stands out if it is visible
        k[s][j, h // (H // G)] = 6.0 * q[s][i, h] / q[s][i, h].norm()
        q[s][i, h] *= 3.0
    return q, k, v, gate


@pytest.mark.parametrize("window,keep", [(6, 2), (1, 0), (9, 9), (0, 0), (1000, 3)])
def test_window_attention_whole_and_pieces(window, keep):
    ops = _ops()
    H, G, dk, dv, scale = 4, 2, 12, 20, 0.25
    lengths = [23, 1, 14]
    # dominant keys just inside / just outside the window and the kept prefix, for the last query of sequence 0
    i = lengths[0] - 1
    spikes = [(0, i, min(max(i - window + 1, 0), i), 0), (0, i, min(max(i - window, 0), i), 1), (0, i, max(keep - 1, 0), 2), (0, i, keep, 3)]
    q, k, v, gate = _attention_case(lengths, H, G, dk, dv, 3, spikes)
    sink = torch.tensor([2.0, -1.0, 0.5, 3.0])
    ref = [O.window_sink_attention(q[s].double(), k[s].double(), v[s].double(), scale=scale, window=window if window > 0 else 10 ** 9,
                                   keep_first=keep, sink=sink.double(), gate_logits=gate[s].double()).reshape(lengths[s], -1) for s in range(3)]
    for cuts in ([[99], [99], [99]], [[5, 2, 9], [1], [3, 3]], [[1], [1], [1]], [[20], [1], [2, 11]]):
        got = _attend(ops, q, k, v, lengths, cuts, H=H, G=G, dk=dk, dv=dv, scale=scale, window=window, keep=keep, sink=sink, gate=gate)
        for s in range(3):
            assert rel_err(got[s], ref[s]) < 1e-4, (cuts, s)


def test_window_attention_far_key_kept_prefix_and_edges_in_long_context():
    """300 positions, window 64, 3 kept tokens, page size 16: the last queries (run as a prompt portion and decoded) have one
    dominant key each at: a kept token, the first dropped token, the window's oldest key, the key just past it, a page border."""
    ops = _ops()
    H, G, dk, dv, scale, window, keep = 2, 1, 16, 16, 0.25, 64, 3
    T = 300
    spikes = [(0, 299, 2, 0), (0, 299, 3, 1), (0, 298, 298 - 63, 0), (0, 298, 298 - 64, 1), (0, 297, 240, 0), (0, 297, 239, 1),
              (0, 150, 0, 0), (0, 150, 150 - 64, 1)]
    q, k, v, gate = _attention_case([T], H, G, dk, dv, 4, spikes)
    sink = torch.tensor([0.3, 1.5])
    ref = O.window_sink_attention(q[0].double(), k[0].double(), v[0].double(), scale=scale, window=window, keep_first=keep, sink=sink.double(),
                                  gate_logits=gate[0].double()).reshape(T, -1)
    for cuts in ([[300]], [[140, 158]], [[296]]):   # whole; two portions (the spiked queries inside the second); then decoded alone
        got = _attend(ops, q, k, v, [T], cuts, H=H, G=G, dk=dk, dv=dv, scale=scale, window=window, keep=keep, sink=sink, gate=gate, bs=16)
        assert rel_err(got[0], ref) < 1e-4, cuts
    # without the sink the same rows must differ visibly: the sink is not a rounding-level term
    nos = _attend(ops, q, k, v, [T], [[300]], H=H, G=G, dk=dk, dv=dv, scale=scale, window=window, keep=keep, sink=None, gate=gate, bs=16)
    assert rel_err(nos[0], ref) > 1e-2


def _recur(fn, lengths, cuts_per_seq, per_seq_inputs, state_shapes, n_slots=5):
    """Drives a recurrent op over the portions; `fn(batch, cat, states)` -> output rows. States start as NaN (a new sequence must
    not read its slot) and are shared by all portions."""
    from vyomai_b200 import ops
    n = len(lengths)
    g = torch.Generator().manual_seed(11)
    slots = torch.randperm(n_slots, generator=g)[:n].tolist()
    states = [torch.full((n_slots,) + tuple(s), float("nan"), device=DEV) for s in state_shapes]
    done, outs = [0] * n, [[] for _ in range(n)]
    cuts = [list(c) for c in cuts_per_seq]
    while any(d < L for d, L in zip(done, lengths)):
        live = [i for i in range(n) if done[i] < lengths[i]]
        take = [min(cuts[i].pop(0) if cuts[i] else 1, lengths[i] - done[i]) for i in live]
        cu = [0]
        for t in take:
            cu.append(cu[-1] + t)
        ti = lambda vals: torch.tensor(vals, dtype=torch.int32, device=DEV)  # noqa: E731
        batch = ops.PackedBatch(ti(cu), ti([done[i] for i in live]), ti([slots[i] for i in live]), max(take))
        cat = lambda name: torch.cat([per_seq_inputs[name][i][done[i]:done[i] + t] for i, t in zip(live, take)]).to(DEV).contiguous()  # noqa: E731
        o = fn(batch, cat, states).cpu()
        for j, (i, t) in enumerate(zip(live, take)):
            outs[i].append(o[cu[j]:cu[j + 1]])
            done[i] += t
    return [torch.cat(o) for o in outs]


SCHEDULES = ([[99], [99], [99]], [[7, 2, 30], [2, 2], [1, 40]], [[1], [1], [1]], [[37], [3], [2]])


@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_causal_conv_carries_its_taps(taps):
    ops = _ops()
    C, lengths = 37, [41, 5, 18]
    g = torch.Generator().manual_seed(6)
    x = [torch.randn(L, C, generator=g) for L in lengths]
    w = torch.randn(C, taps, generator=g)
    ref = [O.causal_conv(xi.double(), w.double()) for xi in x]
    for cuts in SCHEDULES:
        got = _recur(lambda b, cat, st: ops.causal_conv(b, cat("x"), w.to(DEV), st[0], act="silu", out_dtype=torch.float32), lengths, cuts,
                     {"x": x}, [(C, max(taps - 1, 1))])
        for s in range(3):
            assert rel_err(got[s], ref[s]) < 1e-5, (cuts, s)


@pytest.mark.parametrize("H,dk,dv", [(3, 8, 40), (1, 24, 8), (2, 64, 130)])
def test_linear_attention_with_fixed_decay(H, dk, dv):
    ops = _ops()
    lengths = [45, 4, 19]
    g = torch.Generator().manual_seed(7)
    mk = lambda d: [torch.randn(L, H * d, generator=g) for L in lengths]  # noqa: E731
    q, k, v = mk(dk), mk(dk), mk(dv)
    decay = [0.5, 0.93, 0.999][:H]
    ref = [O.lightning_attention(O.silu(q[s].double()).view(-1, H, dk), O.silu(k[s].double()).view(-1, H, dk), O.silu(v[s].double()).view(-1, H, dv),
                                 decay).reshape(lengths[s], -1) for s in range(3)]
    dec = torch.tensor(decay, device=DEV)
    for cuts in SCHEDULES:
        got = _recur(lambda b, cat, st: ops.linear_attn(b, cat("q"), cat("k"), cat("v"), dec, st[0], heads=H, dim=dk, vdim=dv, in_act="silu"),
                     lengths, cuts, {"q": q, "k": k, "v": v}, [(H, dk, dv)])
        for s in range(3):
            assert rel_err(got[s], ref[s]) < 1e-4, (cuts, s)


def test_linear_attention_long_prompt_in_chunks_and_long_decode():
    """700 tokens: whole, in uneven portions that straddle the kernel's chunking, and the last 150 decoded one by one; the slow
    head (decay 0.9995) still carries the first tokens at the end."""
    ops = _ops()
    H, dk, dv, T = 2, 16, 32, 700
    g = torch.Generator().manual_seed(8)
    q, k, v = [torch.randn(T, H * dk, generator=g)], [torch.randn(T, H * dk, generator=g)], [torch.randn(T, H * dv, generator=g)]
    decay = [0.9, 0.9995]
    ref = O.lightning_attention(O.silu(q[0].double()).view(T, H, dk), O.silu(k[0].double()).view(T, H, dk), O.silu(v[0].double()).view(T, H, dv),
                                decay).reshape(T, -1)
    dec = torch.tensor(decay, device=DEV)
    for cuts in ([[700]], [[63, 65, 129, 2, 300]], [[550]]):
        got = _recur(lambda b, cat, st: ops.linear_attn(b, cat("q"), cat("k"), cat("v"), dec, st[0], heads=H, dim=dk, vdim=dv, in_act="silu"),
                     [T], cuts, {"q": q, "k": k, "v": v}, [(H, dk, dv)])
        assert rel_err(got[0], ref) < 2e-4, cuts


@pytest.mark.parametrize("H,G,dk,dv", [(4, 2, 16, 24), (2, 2, 40, 8), (3, 1, 64, 72)])
def test_gated_delta_rule(H, G, dk, dv):
    ops = _ops()
    lengths = [45, 4, 19]
    g = torch.Generator().manual_seed(9)
    mk = lambda d: [torch.randn(L, d, generator=g) for L in lengths]  # noqa: E731
    q, k, v, a, b = mk(G * dk), mk(G * dk), mk(H * dv), mk(H * dk), mk(H)
    a_log = torch.randn(H, generator=g) * 0.5 - 1.0
    ref = []
    for s in range(3):
        L = lengths[s]
        qq = O.unit(q[s].double().view(L, G, dk)) * dk ** -0.5
        kk = O.unit(k[s].double().view(L, G, dk))
        gg = torch.exp(-torch.exp(a_log.double())[None, :, None] * torch.nn.functional.softplus(a[s].double()).view(L, H, dk))
        ref.append(O.gated_delta_rule(qq, kk, v[s].double().view(L, H, dv), gg, torch.sigmoid(b[s].double())).reshape(L, -1))
    for cuts in SCHEDULES:
        got = _recur(lambda bt, cat, st: ops.delta_rule(bt, cat("q"), cat("k"), cat("v"), cat("a"), cat("b"), a_log.to(DEV), st[0], heads=H,
                                                        kv_heads=G, dim=dk, vdim=dv, unit_eps=1e-6),
                     lengths, cuts, {"q": q, "k": k, "v": v, "a": a, "b": b}, [(H, dk, dv)])
        for s in range(3):
            assert rel_err(got[s], ref[s]) < 1e-4, (cuts, s)


def test_delta_rule_overwrites_a_key_it_has_seen():
    """With beta = 1 and no decay, writing (k, v2) after (k, v1) must leave v2 under k: the read-out with q = k returns v2 / sqrt(dk)
    (the update subtracts what the state already holds for k; a plain accumulation would return v1 + v2)."""
    ops = _ops()
    H, dk, dv = 1, 16, 8
    g = torch.Generator().manual_seed(10)
    kvec = torch.randn(dk, generator=g)
    k = torch.stack([kvec, torch.randn(dk, generator=g), kvec])
    v = torch.randn(3, dv, generator=g)
    a = torch.full((3, dk), -40.0)       # softplus -> 0: decay exactly 1
    b = torch.full((3, 1), 40.0)         # sigmoid -> 1
    batch = ops.PackedBatch(torch.tensor([0, 3], dtype=torch.int32, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
                            torch.zeros(1, dtype=torch.int32, device=DEV), 3)
    st = torch.zeros(1, H, dk, dv, device=DEV)
    out = ops.delta_rule(batch, k.to(DEV), k.to(DEV), v.to(DEV), a.to(DEV), b.to(DEV), torch.zeros(1, device=DEV), st, heads=1, kv_heads=1,
                         dim=dk, vdim=dv, unit_eps=1e-6).cpu()
    # token 2 reads with q = k_0 right after overwriting it
    kk = O.unit(k.double())
    S = torch.zeros(dk, dv, dtype=torch.float64)
    for t in range(3):
        S = S + torch.outer(kk[t], v[t].double() - S.T @ kk[t])
    assert rel_err(out[2], (S.T @ kk[2]) / math.sqrt(dk)) < 1e-4
    assert rel_err(out[2] * math.sqrt(dk), v[2]) < 0.2      # close to v2 alone (k_1 is nearly orthogonal), far from v1 + v2


# ---- the prompt-sized (tiled / chunked) forms against the token-serial ones: sizes at their switch-over points and tile edges ----
@pytest.mark.parametrize("dk,dv", [(128, 128), (10, 6), (64, 200)])
def test_window_attention_tile_edges_and_head_sizes(dk, dv):
    """Portions of 15 / 16 tokens sit on either side of the switch to the tiled kernel; 64 / 65 / 130 on either side of its query
    tile; window 70 makes the band start inside a key tile; head sizes with and without 16-byte rows."""
    ops = _ops()
    H, G, scale, window, keep, T = 4, 2, 0.2, 70, 3, 230
    spikes = [(0, 229, 2, 0), (0, 229, 3, 1), (0, 229, 229 - 69, 2), (0, 229, 229 - 70, 3), (0, 128, 128 - 69, 0), (0, 64, 0, 1)]
    q, k, v, gate = _attention_case([T, 37], H, G, dk, dv, 12, spikes)
    sink = torch.tensor([0.5, -2.0, 1.0, 0.0])
    ref = [O.window_sink_attention(q[s].double(), k[s].double(), v[s].double(), scale=scale, window=window, keep_first=keep, sink=sink.double(),
                                   gate_logits=gate[s].double()).reshape(len(q[s]), -1) for s in range(2)]
    for cuts in ([[230], [37]], [[15, 16, 64, 65, 70], [16, 15, 6]], [[130, 99, 1], [1, 36]]):
        got = _attend(ops, q, k, v, [T, 37], cuts, H=H, G=G, dk=dk, dv=dv, scale=scale, window=window, keep=keep, sink=sink, gate=gate, bs=16)
        for s in range(2):
            assert rel_err(got[s], ref[s]) < 1e-4, (cuts, s)


@pytest.mark.parametrize("H,dk,dv", [(2, 128, 128), (1, 20, 70)])
def test_linear_attention_chunk_edges(H, dk, dv):
    """Portions of 7 / 8 tokens on either side of the switch to the chunked kernel, 64 / 65 / 129 around its chunk, and value widths
    that need one, two and three column slices."""
    ops = _ops()
    lengths = [200, 9]
    g = torch.Generator().manual_seed(13)
    mk = lambda d: [torch.randn(L, H * d, generator=g) for L in lengths]  # noqa: E731
    q, k, v = mk(dk), mk(dk), mk(dv)
    decay = [0.8, 0.9991][:H]
    ref = [O.lightning_attention(O.silu(q[s].double()).view(-1, H, dk), O.silu(k[s].double()).view(-1, H, dk), O.silu(v[s].double()).view(-1, H, dv),
                                 decay).reshape(lengths[s], -1) for s in range(2)]
    dec = torch.tensor(decay, device=DEV)
    for cuts in ([[200], [9]], [[7, 8, 64, 65, 56], [8, 1]], [[129, 70, 1], [2, 7]]):
        got = _recur(lambda b, cat, st: ops.linear_attn(b, cat("q"), cat("k"), cat("v"), dec, st[0], heads=H, dim=dk, vdim=dv, in_act="silu"),
                     lengths, cuts, {"q": q, "k": k, "v": v}, [(H, dk, dv)])
        for s in range(2):
            assert rel_err(got[s], ref[s]) < 2e-4, (cuts, s)


@pytest.mark.parametrize("H,G,dk,dv", [(2, 1, 128, 128), (1, 1, 200, 40)])
def test_gated_delta_rule_wide_heads(H, G, dk, dv):
    ops = _ops()
    lengths = [50, 3]
    g = torch.Generator().manual_seed(14)
    mk = lambda d: [torch.randn(L, d, generator=g) for L in lengths]  # noqa: E731
    q, k, v, a, b = mk(G * dk), mk(G * dk), mk(H * dv), mk(H * dk), mk(H)
    a_log = torch.randn(H, generator=g) * 0.5 - 1.0
    ref = []
    for s in range(2):
        L = lengths[s]
        qq = O.unit(q[s].double().view(L, G, dk)) * dk ** -0.5
        kk = O.unit(k[s].double().view(L, G, dk))
        gg = torch.exp(-torch.exp(a_log.double())[None, :, None] * torch.nn.functional.softplus(a[s].double()).view(L, H, dk))
        ref.append(O.gated_delta_rule(qq, kk, v[s].double().view(L, H, dv), gg, torch.sigmoid(b[s].double())).reshape(L, -1))
    for cuts in ([[50], [3]], [[17, 16, 1, 15], [1, 2]]):
        got = _recur(lambda bt, cat, st: ops.delta_rule(bt, cat("q"), cat("k"), cat("v"), cat("a"), cat("b"), a_log.to(DEV), st[0], heads=H,
                                                        kv_heads=G, dim=dk, vdim=dv, unit_eps=1e-6),
                     lengths, cuts, {"q": q, "k": k, "v": v, "a": a, "b": b}, [(H, dk, dv)])
        for s in range(2):
            assert rel_err(got[s], ref[s]) < 1e-4, (cuts, s)


@pytest.mark.parametrize("rows,width", [(3, 1024), (70, 300), (5, 2048), (2, 2500)])
def test_rms_norm_row_widths(rows, width):
    """Widths served by each thread layout (a warp, 128 and 256 threads per row, and the re-reading kernel above 2048)."""
    ops = _ops()
    g = torch.Generator().manual_seed(15)
    x = torch.randn(rows, width, generator=g) * 2
    w = torch.randn(width, generator=g) * 0.2
    gate = torch.randn(rows, width, generator=g)
    ref = O.rms(x.double(), 1e-6) * (1 + w.double()) * torch.sigmoid(gate.double())
    got = ops.rms_norm(x.to(DEV), w.to(DEV), eps=1e-6, w_mode="one_plus", gate=gate.to(DEV), gate_act="sigmoid")
    assert rel_err(got.cpu(), ref) < 1e-5


def test_squared_relu_in_the_projection_epilogue():
    """bf16 inputs on the tensor-core path, prompt-sized and single-token-sized: the activation is applied to the fp32 accumulator."""
    from vyomai_b200.layers.mixers import Projection
    g = torch.Generator().manual_seed(16)
    w = (torch.randn(96, 64, generator=g) / 8).bfloat16()
    for rows in (3, 200):
        x = torch.randn(rows, 64, generator=g).bfloat16()
        got = Projection(w.to(DEV))(x.to(DEV), act="relu2", out_dtype=torch.float32)
        ref = torch.relu(x.double() @ w.double().T) ** 2
        assert rel_err(got.cpu(), ref) < 1e-5
