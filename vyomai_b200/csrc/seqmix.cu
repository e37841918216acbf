// Sequence-mixer kernels over a packed (unpadded) batch: grouped / gated RMS norm, paged key / value write, windowed
// attention with kept first tokens and a softmax sink, causal depthwise convolution with carried taps, linear attention
// with a fixed decay, and the gated delta rule. Statistics, scores, decays and recurrent state are fp32; tensors are read
// and written as fp32 or bf16 according to their dtype arguments. Every kernel takes the batch as (cu_tokens, pos0, slot)
// device arrays, so one launch serves sequences that start, continue or advance by one token, and nothing depends on where
// a sequence sits in the batch.
#include <math.h>

#include "vy_common.cuh"

namespace vy {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float apply_uact(float x, int act) {
  switch (act) {
    case VY_UACT_RELU2: { const float r = fmaxf(x, 0.f); return r * r; }
    case VY_UACT_SILU: return siluf_(x);
    case VY_UACT_SIGMOID: return sigmoidf_(x);
    default: return x;
  }
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- RMS norm -------------------------------------------------------------------------------------------------------
struct NormDev {
  long long rows; int groups, width;
  const int* row_index;
  const void* x; long long ldx; int x_dt;
  const void* w; int w_dt, w_mode;
  const void* gate; long long ld_gate; int gate_dt, gate_act;
  float eps, coef; int accumulate;
  void* out; long long ld_out; int out_dt;
};

__global__ void __launch_bounds__(128) rms_norm_kernel(NormDev d) {
  pdl_trigger();
  pdl_wait();
  const long long r = blockIdx.x * 4LL + (threadIdx.x >> 5);
  if (r >= d.rows) return;
  const int lane = threadIdx.x & 31;
  const long long tok = r / d.groups;
  const int grp = static_cast<int>(r - tok * d.groups);
  const long long st = d.row_index ? d.row_index[tok] : tok;
  const long long xo = st * d.ldx + static_cast<long long>(grp) * d.width;
  float ss = 0.f;
  for (int c = lane; c < d.width; c += 32) {
    const float v = ld_as_float(d.x, d.x_dt, xo + c);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  const float inv = d.coef / sqrtf(ss / static_cast<float>(d.width) + d.eps);
  const long long go = st * d.ld_gate + static_cast<long long>(grp) * d.width;
  const long long oo = tok * d.ld_out + static_cast<long long>(grp) * d.width;
  for (int c = lane; c < d.width; c += 32) {
    float y = ld_as_float(d.x, d.x_dt, xo + c) * inv;
    if (d.w_mode == 1) y *= ld_as_float(d.w, d.w_dt, c);
    else if (d.w_mode == 2) y *= 1.f + ld_as_float(d.w, d.w_dt, c);
    if (d.gate) {
      const float g = ld_as_float(d.gate, d.gate_dt, go + c);
      y *= d.gate_act == VY_UACT_SIGMOID ? sigmoidf_(g) : g;
    }
    if (d.accumulate) y += ld_as_float(d.out, d.out_dt, oo + c);
    st_from_float(d.out, d.out_dt, oo + c, y);
  }
}

// ---- paged key / value write ------------------------------------------------------------------------------------------
struct KvwDev {
  const int* cu; const int* pos0; const int* table; int tw, bs;
  const void* k; long long ldk; const void* v; long long ldv; int in_dt;
  int kw, vw;
  void* kp; void* vp; int pool_dt;
};

__global__ void __launch_bounds__(128) kv_page_write_kernel(KvwDev d) {
  pdl_trigger();
  pdl_wait();
  const int s = blockIdx.y;
  const int base = d.cu[s], n = d.cu[s + 1] - base;
  for (int i = blockIdx.x; i < n; i += gridDim.x) {
    const int pos = d.pos0[s] + i;
    const long long row = static_cast<long long>(d.table[static_cast<long long>(s) * d.tw + pos / d.bs]) * d.bs + pos % d.bs;
    const long long src = base + i;
    for (int c = threadIdx.x; c < d.kw + d.vw; c += blockDim.x) {
      if (c < d.kw) st_from_float(d.kp, d.pool_dt, row * d.kw + c, ld_as_float(d.k, d.in_dt, src * d.ldk + c));
      else st_from_float(d.vp, d.pool_dt, row * d.vw + (c - d.kw), ld_as_float(d.v, d.in_dt, src * d.ldv + (c - d.kw)));
    }
  }
}

// ---- windowed attention with kept first tokens and a sink ---------------------------------------------------------------
struct WinDev {
  const int* cu; const int* pos0; const int* table; int tw, bs;
  const void* q; long long ldq; int q_dt;
  const void* kp; const void* vp; int pool_dt;
  int heads, kv_heads, dim, vdim;
  float scale; int window, keep;
  const void* sink; int sink_dt;
  const void* gate; long long ld_gate; int gate_dt;
  void* out; long long ld_out; int out_dt;
};

constexpr int WA_WARPS = 4;
constexpr int WA_VR = 8;  // value columns per lane: vdim <= 256

__device__ __forceinline__ float dot_row(const void* base, int dt, long long off, int n, const float* __restrict__ qs) {
  float acc = 0.f;
  if (dt == VY_F32 && (n & 3) == 0 && (off & 3) == 0) {
    const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + off);
    for (int i = 0; i < (n >> 2); ++i) {
      const float4 k = p[i];
      acc = fmaf(qs[4 * i], k.x, acc);
      acc = fmaf(qs[4 * i + 1], k.y, acc);
      acc = fmaf(qs[4 * i + 2], k.z, acc);
      acc = fmaf(qs[4 * i + 3], k.w, acc);
    }
  } else if (dt == VY_BF16 && (n & 7) == 0 && (off & 7) == 0) {
    for (int i = 0; i < n; i += 8) {
      float k[8];
      ld8_as_float(base, dt, off + i, k);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc = fmaf(qs[i + j], k[j], acc);
    }
  } else {
    for (int i = 0; i < n; ++i) acc = fmaf(qs[i], ld_as_float(base, dt, off + i), acc);
  }
  return acc;
}

template <bool SPLIT>
__global__ void __launch_bounds__(WA_WARPS * 32) window_attn_kernel(WinDev d) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float wa_smem[];
  const int s = blockIdx.z, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int base = d.cu[s], n = d.cu[s + 1] - base;
  const int qi = SPLIT ? static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x) * WA_WARPS + warp;
  if (qi >= n) return;  // SPLIT: uniform over the CTA; otherwise the warps never meet at a CTA barrier
  const int g = h / (d.heads / d.kv_heads);
  float* qs = wa_smem + warp * d.dim;
  const long long qrow = base + qi;
  for (int i = lane; i < d.dim; i += 32) qs[i] = ld_as_float(d.q, d.q_dt, qrow * d.ldq + static_cast<long long>(h) * d.dim + i);
  __syncwarp();
  const int pos = d.pos0[s] + qi;
  // visible keys: [0, nA) (kept first tokens) and [lowB, pos] (the window), disjoint by construction
  const int nA = d.window <= 0 ? pos + 1 : min(d.keep, pos + 1);
  const int lowB = d.window <= 0 ? pos + 1 : max(pos - d.window + 1, nA);
  const int count = nA + (pos + 1 - lowB);
  float m = -INFINITY, l = 0.f;
  if (d.sink && (!SPLIT || warp == 0)) {
    m = ld_as_float(d.sink, d.sink_dt, h);
    l = 1.f;
  }
  float acc[WA_VR];
#pragma unroll
  for (int r = 0; r < WA_VR; ++r) acc[r] = 0.f;
  const int* tab = d.table + static_cast<long long>(s) * d.tw;
  const int kstride = d.kv_heads * d.dim, vstride = d.kv_heads * d.vdim;
  const int tiles = (count + 31) >> 5;
  for (int tt = SPLIT ? warp : 0; tt < tiles; tt += SPLIT ? WA_WARPS : 1) {
    const int c = tt * 32 + lane;
    const bool valid = c < count;
    long long row = 0;
    float sc = -INFINITY;
    if (valid) {
      const int kp = c < nA ? c : lowB + (c - nA);
      row = static_cast<long long>(tab[kp / d.bs]) * d.bs + kp % d.bs;
      sc = dot_row(d.kp, d.pool_dt, row * kstride + static_cast<long long>(g) * d.dim, d.dim, qs) * d.scale;
    }
    const float m_new = fmaxf(m, warp_max(sc));
    const float p = valid ? expf(sc - m_new) : 0.f;
    const float corr = m == -INFINITY ? 0.f : expf(m - m_new);
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int r = 0; r < WA_VR; ++r) acc[r] *= corr;
    const int nv = min(32, count - tt * 32);
    for (int jj = 0; jj < nv; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const long long rj = __shfl_sync(0xffffffffu, row, jj);
      const long long vo = rj * vstride + static_cast<long long>(g) * d.vdim;
#pragma unroll
      for (int r = 0; r < WA_VR; ++r) {
        const int col = lane + 32 * r;
        if (col < d.vdim) acc[r] = fmaf(pj, ld_as_float(d.vp, d.pool_dt, vo + col), acc[r]);
      }
    }
  }
  if (SPLIT) {
    // merge the four partial softmaxes in warp order
    float* ms = wa_smem + WA_WARPS * d.dim;       // [WA_WARPS]
    float* ls = ms + WA_WARPS;                    // [WA_WARPS]
    float* as = ls + WA_WARPS;                    // [WA_WARPS][vdim]
    if (lane == 0) { ms[warp] = m; ls[warp] = l; }
#pragma unroll
    for (int r = 0; r < WA_VR; ++r) {
      const int col = lane + 32 * r;
      if (col < d.vdim) as[warp * d.vdim + col] = acc[r];
    }
    __syncthreads();
    if (warp != 0) return;
    float M = ms[0];
    for (int w = 1; w < WA_WARPS; ++w) M = fmaxf(M, ms[w]);
    l = 0.f;
    float wgt[WA_WARPS];
    for (int w = 0; w < WA_WARPS; ++w) {
      wgt[w] = ms[w] == -INFINITY ? 0.f : expf(ms[w] - M);
      l += ls[w] * wgt[w];
    }
#pragma unroll
    for (int r = 0; r < WA_VR; ++r) {
      const int col = lane + 32 * r;
      float a = 0.f;
      if (col < d.vdim)
        for (int w = 0; w < WA_WARPS; ++w) a += as[w * d.vdim + col] * wgt[w];
      acc[r] = a;
    }
  }
  float og = 1.f / l;
  if (d.gate) og *= sigmoidf_(ld_as_float(d.gate, d.gate_dt, qrow * d.ld_gate + h));
#pragma unroll
  for (int r = 0; r < WA_VR; ++r) {
    const int col = lane + 32 * r;
    if (col < d.vdim) st_from_float(d.out, d.out_dt, qrow * d.ld_out + static_cast<long long>(h) * d.vdim + col, acc[r] * og);
  }
}

// ---- causal depthwise convolution with carried taps ------------------------------------------------------------------
struct ConvDev {
  const int* cu; const int* pos0; const int* slot;
  int channels, taps;
  const void* x; long long ldx; int x_dt;
  const void* w; int w_dt;
  float* state;
  int act;
  void* out; long long ld_out; int out_dt;
};
constexpr int CONV_MAX_TAPS = 16;
constexpr int CONV_TOK = 32;

__global__ void __launch_bounds__(128) causal_conv_kernel(ConvDev d) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int s = blockIdx.z;
  const int base = d.cu[s], n = d.cu[s + 1] - base;
  if (c >= d.channels) return;
  float w[CONV_MAX_TAPS];
#pragma unroll
  for (int t = 0; t < CONV_MAX_TAPS; ++t) w[t] = t < d.taps ? ld_as_float(d.w, d.w_dt, static_cast<long long>(c) * d.taps + t) : 0.f;
  const bool carried = d.pos0[s] > 0;
  const float* stp = d.state + (static_cast<long long>(d.slot[s]) * d.channels + c) * (d.taps - 1);
  for (int i = blockIdx.y * CONV_TOK; i < n && i < (blockIdx.y + 1) * CONV_TOK; ++i) {
    float y = 0.f;
#pragma unroll
    for (int dd = 0; dd < CONV_MAX_TAPS; ++dd) {
      if (dd < d.taps) {
        const int j = i - dd;
        float xv = 0.f;
        if (j >= 0) xv = ld_as_float(d.x, d.x_dt, static_cast<long long>(base + j) * d.ldx + c);
        else if (carried) xv = stp[d.taps - 1 + j];
        y = fmaf(w[d.taps - 1 - dd], xv, y);
      }
    }
    st_from_float(d.out, d.out_dt, static_cast<long long>(base + i) * d.ld_out + c, apply_uact(y, d.act));
  }
}

__global__ void __launch_bounds__(128) causal_conv_state_kernel(ConvDev d) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int s = blockIdx.y;
  const int base = d.cu[s], n = d.cu[s + 1] - base;
  if (c >= d.channels || n <= 0) return;
  const bool carried = d.pos0[s] > 0;
  float* stp = d.state + (static_cast<long long>(d.slot[s]) * d.channels + c) * (d.taps - 1);
  float tmp[CONV_MAX_TAPS];
#pragma unroll
  for (int t = 0; t < CONV_MAX_TAPS - 1; ++t) {
    if (t < d.taps - 1) {
      const int j = n - (d.taps - 1) + t;
      tmp[t] = j >= 0 ? ld_as_float(d.x, d.x_dt, static_cast<long long>(base + j) * d.ldx + c) : (carried ? stp[d.taps - 1 + j] : 0.f);
    }
  }
#pragma unroll
  for (int t = 0; t < CONV_MAX_TAPS - 1; ++t)
    if (t < d.taps - 1) stp[t] = tmp[t];
}

// ---- recurrences: one thread owns one column of the dim x vdim state in registers ---------------------------------------
struct RecDev {
  const int* cu; const int* pos0; const int* slot;
  const void* q; long long ldq; const void* k; long long ldk; const void* v; long long ldv; int in_dt; int in_act;
  const void* a; long long ld_a; int a_dt;
  const void* b; long long ld_b; int b_dt;
  const void* a_log; int a_log_dt;
  const float* decay;
  int heads, kv_heads, dim, vdim;
  float unit_eps;
  float* state;
  void* out; long long ld_out; int out_dt;
};

template <int DP>
struct RecChunk { static constexpr int CT = DP >= 256 ? 8 : 16; };

// linear attention with a fixed decay: S = decay S + k v^T, o = S^T q
template <int DP>
__global__ void __launch_bounds__(128) linear_attn_kernel(RecDev d) {
  pdl_trigger();
  pdl_wait();
  constexpr int CT = RecChunk<DP>::CT;
  __shared__ float qs[CT][DP];
  __shared__ float ks[CT][DP];
  const int s = blockIdx.z, h = blockIdx.y;
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int base = d.cu[s], n = d.cu[s + 1] - base;
  if (n <= 0) return;
  const bool active = j < d.vdim;
  const float decay = d.decay[h];
  float S[DP];
  float* sp = d.state + ((static_cast<long long>(d.slot[s]) * d.heads + h) * d.dim) * d.vdim + j;
  const bool carried = d.pos0[s] > 0;
#pragma unroll
  for (int i = 0; i < DP; ++i) S[i] = (carried && active && i < d.dim) ? sp[static_cast<long long>(i) * d.vdim] : 0.f;
  for (int t0 = 0; t0 < n; t0 += CT) {
    const int nt = min(CT, n - t0);
    __syncthreads();
    for (int e = threadIdx.x; e < nt * DP; e += blockDim.x) {
      const int tt = e / DP, i = e - tt * DP;
      const long long row = base + t0 + tt;
      float qv = 0.f, kv = 0.f;
      if (i < d.dim) {
        qv = apply_uact(ld_as_float(d.q, d.in_dt, row * d.ldq + static_cast<long long>(h) * d.dim + i), d.in_act);
        kv = apply_uact(ld_as_float(d.k, d.in_dt, row * d.ldk + static_cast<long long>(h) * d.dim + i), d.in_act);
      }
      qs[tt][i] = qv;
      ks[tt][i] = kv;
    }
    __syncthreads();
    if (active) {
      for (int tt = 0; tt < nt; ++tt) {
        const long long row = base + t0 + tt;
        const float vj = apply_uact(ld_as_float(d.v, d.in_dt, row * d.ldv + static_cast<long long>(h) * d.vdim + j), d.in_act);
        float o = 0.f;
#pragma unroll
        for (int i = 0; i < DP; ++i) {
          S[i] = fmaf(decay, S[i], ks[tt][i] * vj);
          o = fmaf(S[i], qs[tt][i], o);
        }
        st_from_float(d.out, d.out_dt, row * d.ld_out + static_cast<long long>(h) * d.vdim + j, o);
      }
    }
  }
  if (active) {
#pragma unroll
    for (int i = 0; i < DP; ++i)
      if (i < d.dim) sp[static_cast<long long>(i) * d.vdim] = S[i];
  }
}

// gated delta rule
template <int DP>
__global__ void __launch_bounds__(128) delta_rule_kernel(RecDev d) {
  pdl_trigger();
  pdl_wait();
  constexpr int CT = RecChunk<DP>::CT;
  extern __shared__ float dr_smem[];
  float (*qs)[DP] = reinterpret_cast<float (*)[DP]>(dr_smem);
  float (*ks)[DP] = reinterpret_cast<float (*)[DP]>(dr_smem + CT * DP);
  float (*gs)[DP] = reinterpret_cast<float (*)[DP]>(dr_smem + 2 * CT * DP);
  float* betas = dr_smem + 3 * CT * DP;
  const int s = blockIdx.z, h = blockIdx.y;
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int base = d.cu[s], n = d.cu[s + 1] - base;
  if (n <= 0) return;
  const bool active = j < d.vdim;
  const int gq = h / (d.heads / d.kv_heads);
  const float neg_rate = -expf(ld_as_float(d.a_log, d.a_log_dt, h));
  const float qscale = 1.f / sqrtf(static_cast<float>(d.dim));
  float S[DP];
  float* sp = d.state + ((static_cast<long long>(d.slot[s]) * d.heads + h) * d.dim) * d.vdim + j;
  const bool carried = d.pos0[s] > 0;
#pragma unroll
  for (int i = 0; i < DP; ++i) S[i] = (carried && active && i < d.dim) ? sp[static_cast<long long>(i) * d.vdim] : 0.f;
  for (int t0 = 0; t0 < n; t0 += CT) {
    const int nt = min(CT, n - t0);
    __syncthreads();
    for (int tt = warp; tt < nt; tt += nwarps) {
      const long long row = base + t0 + tt;
      float sq = 0.f, sk = 0.f;
      for (int i = lane; i < DP; i += 32) {
        float qv = 0.f, kv = 0.f, gv = 1.f;
        if (i < d.dim) {
          qv = ld_as_float(d.q, d.in_dt, row * d.ldq + static_cast<long long>(gq) * d.dim + i);
          kv = ld_as_float(d.k, d.in_dt, row * d.ldk + static_cast<long long>(gq) * d.dim + i);
          gv = expf(neg_rate * softplusf_(ld_as_float(d.a, d.a_dt, row * d.ld_a + static_cast<long long>(h) * d.dim + i)));
        }
        sq = fmaf(qv, qv, sq);
        sk = fmaf(kv, kv, sk);
        qs[tt][i] = qv;
        ks[tt][i] = kv;
        gs[tt][i] = gv;
      }
      sq = warp_sum(sq);
      sk = warp_sum(sk);
      const float qn = qscale / sqrtf(sq + d.unit_eps), kn = 1.f / sqrtf(sk + d.unit_eps);
      for (int i = lane; i < DP; i += 32) {
        qs[tt][i] *= qn;
        ks[tt][i] *= kn;
      }
      if (lane == 0) betas[tt] = sigmoidf_(ld_as_float(d.b, d.b_dt, row * d.ld_b + h));
    }
    __syncthreads();
    if (active) {
      for (int tt = 0; tt < nt; ++tt) {
        const long long row = base + t0 + tt;
        const float vj = ld_as_float(d.v, d.in_dt, row * d.ldv + static_cast<long long>(h) * d.vdim + j);
        float r = 0.f;
#pragma unroll
        for (int i = 0; i < DP; ++i) {
          S[i] *= gs[tt][i];
          r = fmaf(S[i], ks[tt][i], r);
        }
        const float u = betas[tt] * (vj - r);
        float o = 0.f;
#pragma unroll
        for (int i = 0; i < DP; ++i) {
          S[i] = fmaf(ks[tt][i], u, S[i]);
          o = fmaf(S[i], qs[tt][i], o);
        }
        st_from_float(d.out, d.out_dt, row * d.ld_out + static_cast<long long>(h) * d.vdim + j, o);
      }
    }
  }
  if (active) {
#pragma unroll
    for (int i = 0; i < DP; ++i)
      if (i < d.dim) sp[static_cast<long long>(i) * d.vdim] = S[i];
  }
}

static int pad_dim(int dim) { return dim <= 16 ? 16 : dim <= 32 ? 32 : dim <= 64 ? 64 : dim <= 128 ? 128 : 256; }
static int col_threads(int vdim) { return vdim <= 32 ? 32 : vdim <= 64 ? 64 : 128; }

}  // namespace vy

#define VY_NEED_DEVICE(name)                                                   \
  if (!vy_device_ok()) {                                                       \
    ::vy::set_error(name ": no sm_100 device (there is no CPU fallback)");     \
    return VY_ERR_NO_DEVICE;                                                   \
  }

extern "C" int vy_rms_norm(const VyRmsNorm* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_rms_norm: null params");
  VY_NEED_DEVICE("vy_rms_norm");
  VY_CHECK_ARG(p->tokens > 0 && p->groups > 0 && p->width > 0 && p->x && p->out, "vy_rms_norm: bad arguments");
  VY_CHECK_ARG(dtype_ok(p->x_dtype) && dtype_ok(p->out_dtype), "vy_rms_norm: bad dtype");
  VY_CHECK_ARG(p->w_mode >= 0 && p->w_mode <= 2 && (p->w_mode == 0 || (p->weight && dtype_ok(p->w_dtype))), "vy_rms_norm: bad weight");
  if (p->gate) VY_CHECK_ARG(dtype_ok(p->gate_dtype), "vy_rms_norm: bad gate dtype");
  NormDev d;
  d.rows = static_cast<long long>(p->tokens) * p->groups; d.groups = p->groups; d.width = p->width;
  d.row_index = p->row_index;
  d.x = p->x; d.ldx = p->ldx; d.x_dt = p->x_dtype;
  d.w = p->weight; d.w_dt = p->w_dtype; d.w_mode = p->w_mode;
  d.gate = p->gate; d.ld_gate = p->ld_gate; d.gate_dt = p->gate_dtype; d.gate_act = p->gate_act;
  d.eps = p->eps; d.coef = p->coef == 0.f ? 1.f : p->coef; d.accumulate = p->accumulate;
  d.out = p->out; d.ld_out = p->ld_out; d.out_dt = p->out_dtype;
  const long long blocks = (d.rows + 3) / 4;
  VY_CHECK_ARG(blocks <= 2147483647LL, "vy_rms_norm: too many rows");
  VY_CUDA_OK(launch_kernel(rms_norm_kernel, dim3(static_cast<unsigned>(blocks)), dim3(128), 0, static_cast<cudaStream_t>(p->stream), d));
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}

extern "C" int vy_kv_page_write(const VyKvWrite* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_kv_page_write: null params");
  VY_NEED_DEVICE("vy_kv_page_write");
  VY_CHECK_ARG(p->n_seqs > 0 && p->n_seqs <= 65535 && p->max_new > 0 && p->cu_tokens && p->pos0 && p->block_table && p->block_size > 0 &&
                   p->table_width > 0, "vy_kv_page_write: bad batch");
  VY_CHECK_ARG(p->k && p->v && p->k_pool && p->v_pool && p->k_width > 0 && p->v_width > 0 && dtype_ok(p->in_dtype) && dtype_ok(p->pool_dtype),
               "vy_kv_page_write: bad tensors");
  KvwDev d;
  d.cu = p->cu_tokens; d.pos0 = p->pos0; d.table = p->block_table; d.tw = p->table_width; d.bs = p->block_size;
  d.k = p->k; d.ldk = p->ldk; d.v = p->v; d.ldv = p->ldv; d.in_dt = p->in_dtype;
  d.kw = p->k_width; d.vw = p->v_width;
  d.kp = p->k_pool; d.vp = p->v_pool; d.pool_dt = p->pool_dtype;
  const int gx = p->max_new < 4096 ? p->max_new : 4096;
  VY_CUDA_OK(launch_kernel(kv_page_write_kernel, dim3(gx, p->n_seqs), dim3(128), 0, static_cast<cudaStream_t>(p->stream), d));
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}

extern "C" int vy_window_attn(const VyWinAttn* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_window_attn: null params");
  VY_NEED_DEVICE("vy_window_attn");
  VY_CHECK_ARG(p->n_seqs > 0 && p->n_seqs <= 65535 && p->max_new > 0 && p->cu_tokens && p->pos0 && p->block_table && p->block_size > 0 &&
                   p->table_width > 0, "vy_window_attn: bad batch");
  VY_CHECK_ARG(p->heads > 0 && p->kv_heads > 0 && p->heads % p->kv_heads == 0 && p->heads <= 65535 && p->dim > 0 && p->vdim > 0 &&
                   p->vdim <= 32 * WA_VR, "vy_window_attn: bad head geometry (heads %d, kv_heads %d, dim %d, vdim %d <= %d)", p->heads,
               p->kv_heads, p->dim, p->vdim, 32 * WA_VR);
  VY_CHECK_ARG(p->q && p->k_pool && p->v_pool && p->out && dtype_ok(p->q_dtype) && dtype_ok(p->pool_dtype) && dtype_ok(p->out_dtype),
               "vy_window_attn: bad tensors");
  VY_CHECK_ARG(p->keep_first >= 0, "vy_window_attn: negative keep_first");
  if (p->sink) VY_CHECK_ARG(dtype_ok(p->sink_dtype), "vy_window_attn: bad sink dtype");
  if (p->gate) VY_CHECK_ARG(dtype_ok(p->gate_dtype), "vy_window_attn: bad gate dtype");
  WinDev d;
  d.cu = p->cu_tokens; d.pos0 = p->pos0; d.table = p->block_table; d.tw = p->table_width; d.bs = p->block_size;
  d.q = p->q; d.ldq = p->ldq; d.q_dt = p->q_dtype;
  d.kp = p->k_pool; d.vp = p->v_pool; d.pool_dt = p->pool_dtype;
  d.heads = p->heads; d.kv_heads = p->kv_heads; d.dim = p->dim; d.vdim = p->vdim;
  d.scale = p->scale; d.window = p->window; d.keep = p->keep_first;
  d.sink = p->sink; d.sink_dt = p->sink_dtype;
  d.gate = p->gate; d.ld_gate = p->ld_gate; d.gate_dt = p->gate_dtype;
  d.out = p->out; d.ld_out = p->ld_out; d.out_dt = p->out_dtype;
  cudaStream_t st = static_cast<cudaStream_t>(p->stream);
  const size_t smem = sizeof(float) * (static_cast<size_t>(WA_WARPS) * p->dim + 2 * WA_WARPS + static_cast<size_t>(WA_WARPS) * p->vdim);
  VY_CHECK_ARG(smem <= 48 * 1024, "vy_window_attn: dim %d too large", p->dim);
  if (p->max_new == 1) {
    VY_CUDA_OK(launch_kernel(window_attn_kernel<true>, dim3(1, p->heads, p->n_seqs), dim3(WA_WARPS * 32), smem, st, d));
  } else {
    VY_CUDA_OK(launch_kernel(window_attn_kernel<false>, dim3((p->max_new + WA_WARPS - 1) / WA_WARPS, p->heads, p->n_seqs),
                             dim3(WA_WARPS * 32), smem, st, d));
  }
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}

extern "C" int vy_causal_conv(const VyCausalConv* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_causal_conv: null params");
  VY_NEED_DEVICE("vy_causal_conv");
  VY_CHECK_ARG(p->n_seqs > 0 && p->n_seqs <= 65535 && p->max_new > 0 && p->cu_tokens && p->pos0 && p->slot, "vy_causal_conv: bad batch");
  VY_CHECK_ARG(p->channels > 0 && p->taps >= 1 && p->taps <= CONV_MAX_TAPS, "vy_causal_conv: channels %d, taps %d (1..%d)", p->channels,
               p->taps, CONV_MAX_TAPS);
  VY_CHECK_ARG(p->x && p->w && p->out && p->x != p->out && (p->state || p->taps == 1) && dtype_ok(p->x_dtype) && dtype_ok(p->w_dtype) &&
                   dtype_ok(p->out_dtype), "vy_causal_conv: bad tensors");
  VY_CHECK_ARG((p->max_new + CONV_TOK - 1) / CONV_TOK <= 65535, "vy_causal_conv: too many tokens per sequence");
  ConvDev d;
  d.cu = p->cu_tokens; d.pos0 = p->pos0; d.slot = p->slot;
  d.channels = p->channels; d.taps = p->taps;
  d.x = p->x; d.ldx = p->ldx; d.x_dt = p->x_dtype;
  d.w = p->w; d.w_dt = p->w_dtype;
  d.state = p->state; d.act = p->act;
  d.out = p->out; d.ld_out = p->ld_out; d.out_dt = p->out_dtype;
  cudaStream_t st = static_cast<cudaStream_t>(p->stream);
  const int cb = (p->channels + 127) / 128;
  VY_CUDA_OK(launch_kernel(causal_conv_kernel, dim3(cb, (p->max_new + CONV_TOK - 1) / CONV_TOK, p->n_seqs), dim3(128), 0, st, d));
  VY_LAUNCH_OK();
  count_launch();
  if (p->taps > 1) {
    VY_CUDA_OK(launch_kernel(causal_conv_state_kernel, dim3(cb, p->n_seqs), dim3(128), 0, st, d));
    VY_LAUNCH_OK();
    count_launch();
  }
  return VY_OK;
}

namespace vy {
template <int DP>
static cudaError_t launch_linear_attn(const RecDev& d, int n_seqs, cudaStream_t st) {
  const int threads = col_threads(d.vdim);
  return launch_kernel(linear_attn_kernel<DP>, dim3((d.vdim + threads - 1) / threads, d.heads, n_seqs), dim3(threads), 0, st, d);
}
template <int DP>
static cudaError_t launch_delta_rule(const RecDev& d, int n_seqs, cudaStream_t st) {
  const int threads = col_threads(d.vdim);
  constexpr int CT = RecChunk<DP>::CT;
  const size_t smem = sizeof(float) * (3 * CT * DP + CT);
  return launch_kernel(delta_rule_kernel<DP>, dim3((d.vdim + threads - 1) / threads, d.heads, n_seqs), dim3(threads), smem, st, d);
}
}  // namespace vy

extern "C" int vy_linear_attn(const VyLinAttn* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_linear_attn: null params");
  VY_NEED_DEVICE("vy_linear_attn");
  VY_CHECK_ARG(p->n_seqs > 0 && p->n_seqs <= 65535 && p->cu_tokens && p->pos0 && p->slot, "vy_linear_attn: bad batch");
  VY_CHECK_ARG(p->heads > 0 && p->heads <= 65535 && p->dim > 0 && p->dim <= 256 && p->vdim > 0, "vy_linear_attn: heads %d, dim %d (<= 256), vdim %d",
               p->heads, p->dim, p->vdim);
  VY_CHECK_ARG(p->q && p->k && p->v && p->decay && p->state && p->out && dtype_ok(p->in_dtype) && dtype_ok(p->out_dtype),
               "vy_linear_attn: bad tensors");
  RecDev d;
  memset(&d, 0, sizeof(d));
  d.cu = p->cu_tokens; d.pos0 = p->pos0; d.slot = p->slot;
  d.q = p->q; d.ldq = p->ldq; d.k = p->k; d.ldk = p->ldk; d.v = p->v; d.ldv = p->ldv; d.in_dt = p->in_dtype; d.in_act = p->in_act;
  d.decay = p->decay;
  d.heads = p->heads; d.kv_heads = p->heads; d.dim = p->dim; d.vdim = p->vdim;
  d.state = p->state;
  d.out = p->out; d.ld_out = p->ld_out; d.out_dt = p->out_dtype;
  cudaStream_t st = static_cast<cudaStream_t>(p->stream);
  cudaError_t e;
  switch (pad_dim(p->dim)) {
    case 16: e = launch_linear_attn<16>(d, p->n_seqs, st); break;
    case 32: e = launch_linear_attn<32>(d, p->n_seqs, st); break;
    case 64: e = launch_linear_attn<64>(d, p->n_seqs, st); break;
    case 128: e = launch_linear_attn<128>(d, p->n_seqs, st); break;
    default: e = launch_linear_attn<256>(d, p->n_seqs, st); break;
  }
  VY_CUDA_OK(e);
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}

extern "C" int vy_delta_rule(const VyDeltaRule* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_delta_rule: null params");
  VY_NEED_DEVICE("vy_delta_rule");
  VY_CHECK_ARG(p->n_seqs > 0 && p->n_seqs <= 65535 && p->cu_tokens && p->pos0 && p->slot, "vy_delta_rule: bad batch");
  VY_CHECK_ARG(p->heads > 0 && p->heads <= 65535 && p->kv_heads > 0 && p->heads % p->kv_heads == 0 && p->dim > 0 && p->dim <= 256 && p->vdim > 0,
               "vy_delta_rule: heads %d, kv_heads %d, dim %d (<= 256), vdim %d", p->heads, p->kv_heads, p->dim, p->vdim);
  VY_CHECK_ARG(p->q && p->k && p->v && p->a && p->b && p->a_log && p->state && p->out && dtype_ok(p->in_dtype) && dtype_ok(p->a_dtype) &&
                   dtype_ok(p->b_dtype) && dtype_ok(p->a_log_dtype) && dtype_ok(p->out_dtype), "vy_delta_rule: bad tensors");
  RecDev d;
  memset(&d, 0, sizeof(d));
  d.cu = p->cu_tokens; d.pos0 = p->pos0; d.slot = p->slot;
  d.q = p->q; d.ldq = p->ldq; d.k = p->k; d.ldk = p->ldk; d.v = p->v; d.ldv = p->ldv; d.in_dt = p->in_dtype;
  d.a = p->a; d.ld_a = p->ld_a; d.a_dt = p->a_dtype;
  d.b = p->b; d.ld_b = p->ld_b; d.b_dt = p->b_dtype;
  d.a_log = p->a_log; d.a_log_dt = p->a_log_dtype;
  d.heads = p->heads; d.kv_heads = p->kv_heads; d.dim = p->dim; d.vdim = p->vdim;
  d.unit_eps = p->unit_eps;
  d.state = p->state;
  d.out = p->out; d.ld_out = p->ld_out; d.out_dt = p->out_dtype;
  cudaStream_t st = static_cast<cudaStream_t>(p->stream);
  cudaError_t e;
  switch (pad_dim(p->dim)) {
    case 16: e = launch_delta_rule<16>(d, p->n_seqs, st); break;
    case 32: e = launch_delta_rule<32>(d, p->n_seqs, st); break;
    case 64: e = launch_delta_rule<64>(d, p->n_seqs, st); break;
    case 128: e = launch_delta_rule<128>(d, p->n_seqs, st); break;
    default: {
      static bool once = false;
      if (!once) {
        cudaFuncSetAttribute(delta_rule_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
        once = true;
      }
      e = launch_delta_rule<256>(d, p->n_seqs, st);
      break;
    }
  }
  VY_CUDA_OK(e);
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}
