"""Each Zugunex mechanism alone on the GPU against its float64 statement in oracle/zugunex_oracle.py: pair rotation and the query
split, the latent page write, latent attention as a mixer (window, sink, gate, shared rows), the router, both forms of the
experts' sum, the batched per-head product and the tanh-GELU. Packed batches mix sequences that start, continue and advance by
one token, over shuffled pages."""
import math

import pytest
import torch

from oracle import zugunex_oracle as O
from tests import hybrid_util as HU
from tests import zugunex_util as U

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _inv_freq(base, dims):
    return torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64).float().to(DEV)


@pytest.mark.parametrize("rot_dims", [6, 4, 0])
def test_rope_split_rotates_pairs_by_position(rot_dims):
    from vyomai_b200 import ops
    H, keep, rd = 3, 5, 6
    lengths, pos0 = [7, 1, 4], [0, 130, 9]
    batch, *_ = HU.shuffled_batch(lengths, pos0, 4, DEV)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(sum(lengths), H * (keep + rd), generator=g)
    kept = torch.zeros(sum(lengths), H * keep, device=DEV)
    rot = torch.zeros(sum(lengths), H * 9 + 2, device=DEV)
    ops.rope_split(batch, x.to(DEV), _inv_freq(50.0, max(rot_dims, 2)), heads=H, keep=keep, rot_dim=rd, rot_dims=rot_dims, pass_out=kept,
                   rot_out=rot, rot_head=9, rot_col=2)
    xh = x.double().view(-1, H, keep + rd)
    at = 0
    for n, p in zip(lengths, pos0):
        want = O.rotate_pairs(xh[at:at + n, :, keep:], 50.0, rot_dims, pos0=p) if rot_dims else xh[at:at + n, :, keep:]
        got = rot[at:at + n, :H * 9].view(n, H, 9)[:, :, 2:2 + rd].cpu().double()
        assert float((got - want).abs().max()) < 2e-5
        at += n
    assert torch.equal(kept.cpu().view(-1, H, keep), x.view(-1, H, keep + rd)[:, :, :keep])


def test_angles_far_from_zero_are_fp32_accurate():
    """Position 100000 at frequency 1: the angle must be reduced exactly, not by a fast approximation."""
    from vyomai_b200 import ops
    batch, *_ = HU.shuffled_batch([1], [100000], 16, DEV)
    x = torch.tensor([[1.0, 0.0, 0.5, -0.25]], device=DEV)
    out = torch.zeros(1, 4, device=DEV)
    ops.rope_split(batch, x, _inv_freq(4.0, 4), heads=1, keep=0, rot_dim=4, rot_dims=4, pass_out=None, rot_out=out, rot_head=4, rot_col=0)
    want = O.rotate_pairs(x.cpu().double().view(1, 1, 4), 4.0, 4, pos0=100000).view(1, 4)
    assert float((out.cpu().double() - want).abs().max()) < 1e-2   # fp32 angle: 1e5 * 2^-24 ~ 6e-3 rad


def test_latent_page_write_norms_rotates_and_places_rows():
    from vyomai_b200 import ops
    R, rd, bs = 11, 6, 4
    lengths, pos0 = [9, 1, 5], [0, 6, 3]
    batch, table, _, n_blocks, _ = HU.shuffled_batch(lengths, pos0, bs, DEV)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(sum(lengths), R + rd + 3, generator=g)
    wn = 1.0 + 0.2 * torch.randn(R, generator=g)
    pool = torch.full((n_blocks, bs, 1, R + rd), 7.0, device=DEV)
    ops.latent_kv_write(batch, x.to(DEV)[:, :R + rd], wn.to(DEV), _inv_freq(30.0, rd), pool, rank=R, rot_dim=rd, rot_dims=rd, eps=1e-3)
    at = 0
    touched = set()
    for s, (n, p) in enumerate(zip(lengths, pos0)):
        xs = x[at:at + n].double()
        c = O.rms(xs[:, :R], 1e-3) * wn.double()
        kr = O.rotate_pairs(xs[:, R:R + rd], 30.0, rd, pos0=p)
        for i in range(n):
            blk, off = table[s][(p + i) // bs], (p + i) % bs
            touched.add((blk, off))
            row = pool[blk, off, 0].cpu().double()
            assert float((row[:R] - c[i]).abs().max()) < 1e-5 and float((row[R:] - kr[i]).abs().max()) < 1e-5
        at += n
    for blk in range(n_blocks):
        for off in range(bs):
            if (blk, off) not in touched:
                assert float(pool[blk, off].min()) == 7.0   # nothing else was written


def _mixer(cfg_m, seed, dtype=torch.float32, shared_from=None, width=40):
    from vyomai_b200.layers.mixers import LatentAttention
    g = torch.Generator().manual_seed(seed)
    H, dn, dr, dv, R = cfg_m["heads"], cfg_m["dim"], cfg_m["rot_dim"], cfg_m["vdim"], cfg_m["kv_rank"]
    shapes = {"q": (H * (dn + dr), width), "dkv": (R + dr, width), "uk": (H * dn, R), "uv": (H * dv, R), "g": (H, width), "o": (width, H * dv)}
    w = {k: (torch.randn(s, generator=g) / math.sqrt(s[1])).to(torch.bfloat16) for k, s in shapes.items()}
    w["dkv.norm"] = (1 + 0.1 * torch.randn(R, generator=g)).to(torch.bfloat16)
    w["sink"] = torch.randn(H, generator=g).to(torch.bfloat16)
    mix = LatentAttention(cfg_m, {k: v.to(DEV, dtype) for k, v in w.items()}, 1e-5, dtype, True, shared_from=shared_from)
    return mix, {k: v.double() for k, v in w.items()}


def _run_mixer(mix, W, h, lengths_by_step, bs=4, expanded=None):
    """Feeds h [T, width] (one sequence) to the mixer in portions through real pages; returns [T, width]."""
    from vyomai_b200 import ops
    from vyomai_b200.paged import LayerCacheView
    T = h.shape[0]
    n_blocks = (T + bs - 1) // bs + 2
    order = torch.randperm(n_blocks, generator=torch.Generator().manual_seed(5)).tolist()
    view = LayerCacheView()
    view.k_pool = torch.zeros((n_blocks, bs, 1, mix.row), device=DEV)
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)  # noqa: E731
    outs, at = [], 0
    for n in lengths_by_step:
        batch = ops.PackedBatch(t([0, n]), t([at]), t([0]), n, t(order).view(1, -1), bs)
        x = h[at:at + n].to(DEV)
        parts = [ops.linear_plain(x, wt.to(DEV).float()) for wt in mix.input_weights()]
        outs.append(mix.forward(parts, batch, view, expanded=expanded if at == 0 else False).float().cpu())
        at += n
    return torch.cat(outs)


@pytest.mark.parametrize("steps", [[37], [20, 1, 1, 1, 14], [2] * 18 + [1], [16, 21]])
def test_latent_attention_mixer(steps):
    m = U.attn(heads=3, dim=8, rot_dim=6, vdim=10, rank=20, window=7, scale=0.4)
    mix, W = _mixer(m, 2)
    h = torch.randn(37, 40, generator=torch.Generator().manual_seed(3))
    c, kr = O.latent_kv(h.double(), W, m, 1e-5)
    want = O.latent_attention(h.double(), W, m, c, kr)
    got = _run_mixer(mix, W, h, steps)
    assert HU.rel_err(got, want) < 1e-4


@pytest.mark.parametrize("window", [7, 16, 40])
def test_whole_prompt_form_equals_the_latent_form(window):
    """bf16 projections: a prompt from position 0 expands keys and values per head; portions and single tokens attend over latent
    rows. Same sum, against the oracle and against each other; the rows must also be in the pages for what follows."""
    m = U.attn(heads=4, dim=32, rot_dim=16, vdim=24, rank=48, window=window, scale=0.2)
    mix, W = _mixer(m, 8, dtype=torch.bfloat16, width=64)
    assert mix.expand is not None
    h = torch.randn(37, 64, generator=torch.Generator().manual_seed(9))
    c, kr = O.latent_kv(h.double(), W, m, 1e-5)
    want = O.latent_attention(h.double(), W, m, c, kr)
    latent = _run_mixer(mix, W, h, [37], expanded=False)
    whole = _run_mixer(mix, W, h, [37], expanded=True)
    then_decode = _run_mixer(mix, W, h, [30, 1, 1, 5], expanded=True)
    for got in (latent, whole, then_decode):
        assert HU.rel_err(got, want) < 2e-2
    assert HU.rel_err(whole, latent) < 2e-2 and HU.rel_err(then_decode[30:], latent[30:]) < 2e-2


def test_one_far_key_just_inside_the_window_dominates():
    """Scores are made so that exactly one key, window - 1 positions back, carries the softmax: an edge that is one off, or a
    key read from the wrong page row, changes the output completely."""
    window = 33
    m = U.attn(heads=2, dim=4, rot_dim=2, vdim=6, rank=12, window=window, scale=1.0)
    mix, W = _mixer(m, 6)
    T = 3 * window
    g = torch.Generator().manual_seed(7)
    h = 0.05 * torch.randn(T, 40, generator=g)
    for i in range(window - 1, T, 5):      # token i - (window - 1) gets a large latent, token i a query that finds it
        h[i - (window - 1)] = 3.0 * torch.randn(40, generator=g)
    c, kr = O.latent_kv(h.double(), W, m, 1e-5)
    want = O.latent_attention(h.double(), W, m, c, kr)
    for steps in ([T], [window + 3] + [1] * (T - window - 3), [7] * (T // 7) + [T % 7]):
        steps = [s for s in steps if s]
        assert HU.rel_err(_run_mixer(mix, W, h, steps, bs=16), want) < 1e-4, steps[:3]
    shifted = dict(m, mask={"size": window - 1})
    wrong = O.latent_attention(h.double(), W, shifted, c, kr)
    assert HU.rel_err(wrong, want) > 1e-2   # the construction does show an edge that is one off


@pytest.mark.parametrize("experts,top", [(5, 2), (16, 3), (1, 1), (40, 40), (70, 33)])
def test_router_matches_the_oracle(experts, top):
    from vyomai_b200 import ops
    g = torch.Generator().manual_seed(experts)
    z = 2.0 * torch.randn(19, experts + 1, generator=g)
    idx, wt, dense = ops.moe_route(z.to(DEV)[:, :experts], experts, top, 1.7)
    s = torch.sigmoid(z[:, :experts].double())
    val, ref_idx = torch.topk(s, top, dim=-1)
    ref_w = val / (val.sum(-1, keepdim=True) + 1e-20) * 1.7
    assert torch.equal(idx.cpu().long(), ref_idx)
    assert float((wt.cpu().double() - ref_w).abs().max()) < 1e-6
    want_dense = torch.zeros(19, experts, dtype=torch.float64).scatter_(1, ref_idx, ref_w)
    assert float((dense.cpu().double() - want_dense).abs().max()) < 1e-6


def test_router_ties_go_to_the_lowest_index():
    from vyomai_b200 import ops
    z = torch.zeros(2, 6, device=DEV)
    z[1, 4] = 1.0
    idx, wt, _ = ops.moe_route(z, 6, 3, 1.0)
    assert idx.cpu().tolist() == [[0, 1, 2], [4, 0, 1]]


@pytest.mark.parametrize("shared_ff", [None, 20])
@pytest.mark.parametrize("rows,sorted_min", [(1, 128), (7, 128), (20, 128), (40, 8), (300, 8)])
def test_both_forms_of_the_experts_sum(rows, sorted_min, shared_ff):
    from vyomai_b200 import ops
    from vyomai_b200.layers.mixers import MoEFeedForward
    E, top, ff, width = 5, 2, 12, 40
    g = torch.Generator().manual_seed(rows)
    w = {}
    for e in range(E):
        w[f"e{e}.up"] = (torch.randn(ff, width, generator=g) / math.sqrt(width)).to(torch.bfloat16)
        w[f"e{e}.down"] = (torch.randn(width, ff, generator=g) / math.sqrt(ff)).to(torch.bfloat16)
    w["router"] = (torch.randn(E, width, generator=g) / 2).to(torch.bfloat16)
    if shared_ff:
        w["shared.up"] = (torch.randn(shared_ff, width, generator=g) / math.sqrt(width)).to(torch.bfloat16)
        w["shared.down"] = (torch.randn(width, shared_ff, generator=g) / math.sqrt(shared_ff)).to(torch.bfloat16)
        w["shared.sg"] = torch.randn(1, width, generator=g).to(torch.bfloat16)
    mlp = MoEFeedForward({k: v.to(DEV).float() for k, v in w.items()}, E, top, 1.3, torch.float32, True, shared=bool(shared_ff), sorted_min_rows=sorted_min, force_sorted=True)
    h = torch.randn(rows, width, generator=g)
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)  # noqa: E731
    batch = ops.PackedBatch(t([0, rows]), t([0]), t([0]), rows, None, 0)
    got = mlp.forward(h.to(DEV), batch).cpu()
    spec = U.moe(experts=E, top=top, ff=ff, scale=1.3, shared_ff=shared_ff)
    want = O.moe_ff(h.double(), {k: v.double() for k, v in w.items()}, spec)
    assert HU.rel_err(got, want) < 1e-5


def test_the_form_is_chosen_by_estimated_time():
    """Narrow experts on the tensor cores: launches dominate, all experts at once; wide ones or fp32 FMA products: the sorted form."""
    from vyomai_b200.layers.mixers import MoEFeedForward

    def mlp(width, ff, dtype):
        w = {"router": torch.zeros(32, width, dtype=dtype, device=DEV)}
        for e in range(32):
            w[f"e{e}.up"], w[f"e{e}.down"] = torch.zeros(ff, width, dtype=dtype, device=DEV), torch.zeros(width, ff, dtype=dtype, device=DEV)
        return MoEFeedForward(w, 32, 4, 1.0, dtype, True)
    assert not mlp(1024, 256, torch.bfloat16)._sorted_is_faster(8192)
    assert mlp(2048, 1024, torch.bfloat16)._sorted_is_faster(8192)
    assert mlp(1024, 256, torch.float32)._sorted_is_faster(8192)


def test_sorted_pairs_are_grouped_by_expert_in_row_order():
    from vyomai_b200 import ops
    g = torch.Generator().manual_seed(9)
    idx = torch.stack([torch.randperm(7, generator=g)[:3] for _ in range(50)]).int()
    counts, offsets, perm, inv = (t.cpu() for t in ops.moe_sort(idx.to(DEV), 7))
    flat = idx.flatten()
    assert counts.tolist() == torch.bincount(flat, minlength=7).tolist()
    assert offsets.tolist() == [0] + torch.cumsum(counts, 0).tolist()
    for e in range(7):
        seg = perm[offsets[e]:offsets[e + 1]].tolist()
        assert seg == sorted(seg) and all(int(flat[i]) == e for i in seg)
    assert torch.equal(perm[inv.long()], torch.arange(150, dtype=torch.int32))


def test_batched_per_head_product():
    from vyomai_b200 import ops
    g = torch.Generator().manual_seed(10)
    for rows in (3, 20, 50):
        x = torch.randn(rows, 4 * 7 + 2, generator=g)
        w = torch.randn(4, 5, 6, generator=g)
        out = torch.zeros(rows, 4 * 9, device=DEV)
        ops.head_linear(x.to(DEV), w.to(DEV), out, x_head=7, out_head=9)
        for h in range(4):
            want = x[:, h * 7:h * 7 + 6].double() @ w[h].double().T
            assert float((out[:, h * 9:h * 9 + 5].cpu().double() - want).abs().max()) < 1e-5
            assert float(out[:, h * 9 + 5:h * 9 + 9].abs().max()) == 0.0


def test_gelu_tanh_in_both_projection_arms():
    from vyomai_b200.layers.mixers import Projection
    g = torch.Generator().manual_seed(11)
    x, w = torch.randn(40, 64, generator=g), torch.randn(48, 64, generator=g) / 8
    want = O.gelu_tanh(x.double() @ w.double().T)
    got32 = Projection(w.to(DEV))(x.to(DEV), act="gelu_tanh").cpu()
    assert HU.rel_err(got32, want) < 1e-5
    xb, wb = x.to(torch.bfloat16), w.to(torch.bfloat16)
    want_b = O.gelu_tanh(xb.double() @ wb.double().T)
    got16 = Projection(wb.to(DEV))(xb.to(DEV), act="gelu_tanh").cpu()
    assert HU.rel_err(got16, want_b) < 1e-3


@pytest.mark.parametrize("dim,vdim,kv_heads", [(24, 16, 2), (22, 10, 1)])
def test_single_token_attention_with_heads_grouped_per_cta(dim, vdim, kv_heads):
    """Large single-token batches put four heads of one key / value head into a CTA; small ones one head per CTA (the form the
    mixer tests hold against the oracle). Both must give the same numbers, through the 16-byte and the scalar loads."""
    from vyomai_b200 import ops
    H, n, bs = 8, 48, 4
    g = torch.Generator().manual_seed(dim)
    pos0 = torch.randint(0, 60, (n,), generator=g).tolist()
    batch, table, _, n_blocks, _ = HU.shuffled_batch([1] * n, pos0, bs, DEV)
    kp = torch.randn(n_blocks, bs, kv_heads, dim, generator=g).to(DEV)
    vp = torch.randn(n_blocks, bs, kv_heads, vdim, generator=g).to(DEV)
    q = torch.randn(n, H * dim, generator=g).to(DEV)
    sink, gate = torch.randn(H, generator=g).to(DEV), torch.randn(n, H, generator=g).to(DEV)
    kw = dict(heads=H, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=0.3, window=9, keep_first=0, sink=sink)
    whole = ops.window_attn(batch, q, kp, vp, gate=gate, **kw)
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)  # noqa: E731
    for a in range(0, n, 8):
        sub = ops.PackedBatch(t(list(range(9))), t(pos0[a:a + 8]), t([0] * 8), 1, batch.block_table[a:a + 8].contiguous(), bs)
        part = ops.window_attn(sub, q[a:a + 8], kp, vp, gate=gate[a:a + 8], **kw)
        assert float((part - whole[a:a + 8]).abs().max()) < 1e-5


@pytest.mark.parametrize("alias", [True, False])
@pytest.mark.parametrize("heads,dim,vdim,window", [(24, 40, 24, 300), (8, 22, 10, 0), (16, 224, 192, 130), (32, 64, 64, 64)])
def test_single_token_attention_with_heads_as_tile_rows(heads, dim, vdim, window, alias):
    """Eight or more query heads on one key / value head: the token's heads are the rows of a tile, a sequence's keys are split over
    CTAs and merged. Against a float64 softmax over the gathered pool rows: split edges, a partly filled head tile, the sink in
    one split only, values as the leading channels of the key rows (one pool) or in a pool of their own."""
    from vyomai_b200 import ops
    bs = 16
    g = torch.Generator().manual_seed(heads + dim)
    pos0 = [0, 63, 64, 700, 257]
    n = len(pos0)
    batch, table, _, n_blocks, _ = HU.shuffled_batch([1] * n, pos0, bs, DEV)
    kp = torch.randn(n_blocks, bs, 1, dim, generator=g)
    vp = kp[..., :vdim] if alias else torch.randn(n_blocks, bs, 1, vdim, generator=g)
    q = torch.randn(n, heads * dim, generator=g)
    sink, gate = torch.randn(heads, generator=g), torch.randn(n, heads, generator=g)
    kd = kp.to(DEV)
    vd = kd if alias else vp.to(DEV)
    got = ops.window_attn(batch, q.to(DEV), kd, vd, heads=heads, kv_heads=1, dim=dim, vdim=vdim, scale=0.2, window=window, keep_first=0,
                          sink=sink.to(DEV), gate=gate.to(DEV), k_row=dim, v_row=dim if alias else vdim).cpu().double()
    for s, p in enumerate(pos0):
        lo = 0 if window <= 0 else max(0, p - window + 1)
        rows = [(table[s][j // bs], j % bs) for j in range(lo, p + 1)]
        K = torch.stack([kp[b, o, 0] for b, o in rows]).double()
        V = torch.stack([vp[b, o, 0] for b, o in rows]).double()
        for h in range(heads):
            sc = K @ q[s, h * dim:(h + 1) * dim].double() * 0.2
            mx = torch.maximum(sc.max(), sink[h].double())
            e = torch.exp(sc - mx)
            o = (e[:, None] * V).sum(0) / (e.sum() + torch.exp(sink[h].double() - mx)) * torch.sigmoid(gate[s, h].double())
            assert float((got[s, h * vdim:(h + 1) * vdim] - o).abs().max()) < 1e-5, (s, h)
