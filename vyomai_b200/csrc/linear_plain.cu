// vy_linear_plain: out = act(A W^T + bias) * scale + addend for any M, N, K and any alignment, fp32 FMA accumulation.
// Three kernels: 64 x 64 x 16 shared-memory tiles (4 x 4 outputs per thread) for many rows, a weight-streaming kernel
// (one warp per output feature, lanes over K) for at most 8 rows, and a 32-feature tile for 9 .. 32 rows. A call may hold a batch
// of independent products of one shape (blockIdx z / y picks the product). This is the exact-fp32 arm of every projection of the
// sequence-mixer models and the bf16 arm of the shapes the tensor-core GEMM does not take (a contraction over a
// low rank, a handful of output features, strides that are not 16-byte multiples). vy_unary and vy_embed_rows live
// here as well.
#include "vy_common.cuh"

namespace vy {

__device__ __forceinline__ float uact(float x, int act) {
  switch (act) {
    case VY_UACT_RELU2: { const float r = fmaxf(x, 0.f); return r * r; }
    case VY_UACT_SILU: return x / (1.f + expf(-x));
    case VY_UACT_SIGMOID: return 1.f / (1.f + expf(-x));
    case VY_UACT_GELU_TANH: return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
    default: return x;
  }
}

struct LinDev {
  int M, N, K;
  const void* A; long long lda; int a_dt;
  const void* W; long long ldw; int w_dt;
  const void* bias; int bias_dt;
  const void* addend; long long ld_addend; int addend_dt;
  int act; float scale;
  void* out; long long ld_out; int out_dt;
  long long a_batch, w_batch, out_batch;   // element strides between the independent products of a batched call
};

// product b of a batched call: the same shapes at shifted base pointers
__device__ __forceinline__ void lin_select(LinDev& d, int b) {
  if (b == 0) return;
  d.A = static_cast<const char*>(d.A) + d.a_batch * b * (d.a_dt == VY_F32 ? 4 : 2);
  d.W = static_cast<const char*>(d.W) + d.w_batch * b * (d.w_dt == VY_F32 ? 4 : 2);
  d.out = static_cast<char*>(d.out) + d.out_batch * b * (d.out_dt == VY_F32 ? 4 : 2);
}

__device__ __forceinline__ void lin_store(const LinDev& d, int m, int n, float acc) {
  if (d.bias) acc += ld_as_float(d.bias, d.bias_dt, n);
  acc = uact(acc, d.act) * d.scale;
  if (d.addend) acc += ld_as_float(d.addend, d.addend_dt, static_cast<long long>(m) * d.ld_addend + n);
  st_from_float(d.out, d.out_dt, static_cast<long long>(m) * d.ld_out + n, acc);
}

constexpr int LT = 64, LK = 16;

__global__ void __launch_bounds__(256) linear_tile_kernel(LinDev d) {
  pdl_trigger();
  pdl_wait();
  lin_select(d, blockIdx.z);
  __shared__ float As[LK][LT + 4];
  __shared__ float Ws[LK][LT + 4];
  const int m0 = blockIdx.y * LT, n0 = blockIdx.x * LT;
  const int tid = threadIdx.x;
  const int lr = tid >> 2, lk = (tid & 3) * 4;  // loader: row 0..63, 4 consecutive k
  const int tm = (tid >> 4) * 4, tn = (tid & 15) * 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < d.K; k0 += LK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      const int am = m0 + lr, wn = n0 + lr;
      As[lk + i][lr] = (am < d.M && k < d.K) ? ld_as_float(d.A, d.a_dt, static_cast<long long>(am) * d.lda + k) : 0.f;
      Ws[lk + i][lr] = (wn < d.N && k < d.K) ? ld_as_float(d.W, d.w_dt, static_cast<long long>(wn) * d.ldw + k) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < LK; ++k) {
      const float4 a = *reinterpret_cast<const float4*>(&As[k][tm]);
      const float4 w = *reinterpret_cast<const float4*>(&Ws[k][tn]);
      const float av[4] = {a.x, a.y, a.z, a.w}, wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (m0 + tm + i < d.M && n0 + tn + j < d.N) lin_store(d, m0 + tm + i, n0 + tn + j, acc[i][j]);
}

// at most 8 rows: one warp per output feature, lanes stride over K (coalesced weight rows), shuffle reduction
__global__ void __launch_bounds__(256) linear_rows_kernel(LinDev d) {
  pdl_trigger();
  pdl_wait();
  lin_select(d, blockIdx.y);
  const int n = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (n >= d.N) return;
  float acc[8];
#pragma unroll
  for (int m = 0; m < 8; ++m) acc[m] = 0.f;
  for (int k = lane; k < d.K; k += 32) {
    const float w = ld_as_float(d.W, d.w_dt, static_cast<long long>(n) * d.ldw + k);
#pragma unroll
    for (int m = 0; m < 8; ++m)
      if (m < d.M) acc[m] = fmaf(ld_as_float(d.A, d.a_dt, static_cast<long long>(m) * d.lda + k), w, acc[m]);
  }
#pragma unroll
  for (int m = 0; m < 8; ++m) {
    float v = acc[m];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0 && m < d.M) lin_store(d, m, n, v);
  }
}

// 9 .. 32 rows (a decode batch; the per-head products of latent attention): a CTA takes 32 output features of one product, thread
// (feature, group of 4 rows); A and W pass through shared memory 64 k at a time, W transposed so that a warp's features are adjacent
constexpr int LS_N = 32, LS_K = 64, LS_M = 32;
__global__ void __launch_bounds__(256) linear_small_kernel(LinDev d) {
  pdl_trigger();
  pdl_wait();
  lin_select(d, blockIdx.y);
  __shared__ __align__(16) float xs[LS_M][LS_K + 4];
  __shared__ float ws[LS_K][LS_N + 1];
  const int t = threadIdx.x, n = t & 31, mg = t >> 5;
  const int n0 = blockIdx.x * LS_N;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k0 = 0; k0 < d.K; k0 += LS_K) {
    {
      const int r = t >> 3, kk = (t & 7) * 8;   // 32 rows x 8 threads x 8 k
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int k = k0 + kk + j;
        xs[r][kk + j] = (r < d.M && k < d.K) ? ld_as_float(d.A, d.a_dt, static_cast<long long>(r) * d.lda + k) : 0.f;
        ws[kk + j][r] = (n0 + r < d.N && k < d.K) ? ld_as_float(d.W, d.w_dt, static_cast<long long>(n0 + r) * d.ldw + k) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll 4
    for (int k = 0; k < LS_K; k += 4) {
      const float w0 = ws[k][n], w1 = ws[k + 1][n], w2 = ws[k + 2][n], w3 = ws[k + 3][n];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 x = *reinterpret_cast<const float4*>(&xs[4 * mg + i][k]);
        acc[i] = fmaf(x.x, w0, acc[i]);
        acc[i] = fmaf(x.y, w1, acc[i]);
        acc[i] = fmaf(x.z, w2, acc[i]);
        acc[i] = fmaf(x.w, w3, acc[i]);
      }
    }
    __syncthreads();
  }
  if (n0 + n < d.N)
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (4 * mg + i < d.M) lin_store(d, 4 * mg + i, n0 + n, acc[i]);
}

__global__ void __launch_bounds__(256) unary_kernel(long long rows, int cols, const void* x, long long ldx, int x_dt, int act,
                                                     void* out, long long ld_out, int out_dt) {
  pdl_trigger();
  pdl_wait();
  const long long n = rows * cols;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / cols;
    const int c = static_cast<int>(i - r * cols);
    st_from_float(out, out_dt, r * ld_out + c, uact(ld_as_float(x, x_dt, r * ldx + c), act));
  }
}

__global__ void __launch_bounds__(128) embed_rows_kernel(int rows, int width, int vocab, const int* __restrict__ ids,
                                                         const void* table, long long ld_table, int table_dt, float scale, void* out,
                                                         long long ld_out, int out_dt) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int id = ids[r];
  const bool ok = id >= 0 && id < vocab;
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    st_from_float(out, out_dt, static_cast<long long>(r) * ld_out + c,
                  ok ? scale * ld_as_float(table, table_dt, static_cast<long long>(id) * ld_table + c) : 0.f);
}

}  // namespace vy

extern "C" int vy_linear_plain(const VyLinear* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_linear_plain: null params");
  if (!vy_device_ok()) {
    set_error("vy_linear_plain: no sm_100 device (there is no CPU fallback)");
    return VY_ERR_NO_DEVICE;
  }
  VY_CHECK_ARG(p->M > 0 && p->N > 0 && p->K > 0, "vy_linear_plain: bad shape M=%d N=%d K=%d", p->M, p->N, p->K);
  VY_CHECK_ARG(p->A && p->W && p->out, "vy_linear_plain: null operand");
  VY_CHECK_ARG(dtype_ok(p->a_dtype) && dtype_ok(p->w_dtype) && dtype_ok(p->out_dtype), "vy_linear_plain: bad dtype");
  VY_CHECK_ARG(p->lda >= p->K && p->ldw >= p->K && p->ld_out >= p->N, "vy_linear_plain: leading dimension smaller than the row");
  VY_CHECK_ARG(p->act >= VY_UACT_NONE && p->act <= VY_UACT_GELU_TANH, "vy_linear_plain: bad act %d", p->act);
  const int batch = p->batch > 1 ? p->batch : 1;
  VY_CHECK_ARG(batch <= 65535 && (batch == 1 || (!p->bias && !p->addend)), "vy_linear_plain: a batched call takes no bias / addend (batch %d)", batch);
  if (p->bias) VY_CHECK_ARG(dtype_ok(p->bias_dtype), "vy_linear_plain: bad bias_dtype");
  if (p->addend) VY_CHECK_ARG(dtype_ok(p->addend_dtype) && p->ld_addend >= p->N, "vy_linear_plain: bad addend");
  LinDev d;
  d.M = p->M; d.N = p->N; d.K = p->K;
  d.A = p->A; d.lda = p->lda; d.a_dt = p->a_dtype;
  d.W = p->W; d.ldw = p->ldw; d.w_dt = p->w_dtype;
  d.bias = p->bias; d.bias_dt = p->bias_dtype;
  d.addend = p->addend; d.ld_addend = p->ld_addend; d.addend_dt = p->addend_dtype;
  d.act = p->act; d.scale = p->scale == 0.f ? 1.f : p->scale;
  d.out = p->out; d.ld_out = p->ld_out; d.out_dt = p->out_dtype;
  d.a_batch = p->a_batch; d.w_batch = p->w_batch; d.out_batch = p->out_batch;
  cudaStream_t st = static_cast<cudaStream_t>(p->stream);
  if (p->M <= 8) {
    VY_CUDA_OK(launch_kernel(linear_rows_kernel, dim3((p->N + 7) / 8, batch), dim3(256), 0, st, d));
  } else if (p->M <= LS_M) {
    VY_CUDA_OK(launch_kernel(linear_small_kernel, dim3((p->N + LS_N - 1) / LS_N, batch), dim3(256), 0, st, d));
  } else {
    VY_CHECK_ARG((p->M + LT - 1) / LT <= 65535, "vy_linear_plain: too many rows (%d)", p->M);
    VY_CUDA_OK(launch_kernel(linear_tile_kernel, dim3((p->N + LT - 1) / LT, (p->M + LT - 1) / LT, batch), dim3(256), 0, st, d));
  }
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}

extern "C" int vy_unary(int64_t rows, int32_t cols, const void* x, int64_t ldx, int32_t x_dtype, int32_t act, void* out,
                        int64_t ld_out, int32_t out_dtype, void* stream) {
  using namespace vy;
  if (!vy_device_ok()) {
    set_error("vy_unary: no sm_100 device (there is no CPU fallback)");
    return VY_ERR_NO_DEVICE;
  }
  VY_CHECK_ARG(rows > 0 && cols > 0 && x && out, "vy_unary: bad arguments");
  VY_CHECK_ARG(dtype_ok(x_dtype) && dtype_ok(out_dtype) && act >= VY_UACT_NONE && act <= VY_UACT_GELU_TANH, "vy_unary: bad dtype / act");
  long long blocks = (rows * cols + 255) / 256;
  if (blocks > 16LL * num_sms()) blocks = 16LL * num_sms();
  VY_CUDA_OK(launch_kernel(unary_kernel, dim3(static_cast<int>(blocks)), dim3(256), 0, static_cast<cudaStream_t>(stream),
                           static_cast<long long>(rows), cols, x, static_cast<long long>(ldx), x_dtype, act, out,
                           static_cast<long long>(ld_out), out_dtype));
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}

extern "C" int vy_embed_rows(int32_t rows, int32_t width, int32_t vocab, const int32_t* ids, const void* table, int64_t ld_table,
                             int32_t table_dtype, float scale, void* out, int64_t ld_out, int32_t out_dtype, void* stream) {
  using namespace vy;
  if (!vy_device_ok()) {
    set_error("vy_embed_rows: no sm_100 device (there is no CPU fallback)");
    return VY_ERR_NO_DEVICE;
  }
  VY_CHECK_ARG(rows > 0 && width > 0 && vocab > 0 && ids && table && out, "vy_embed_rows: bad arguments");
  VY_CHECK_ARG(dtype_ok(table_dtype) && dtype_ok(out_dtype), "vy_embed_rows: bad dtype");
  VY_CUDA_OK(launch_kernel(embed_rows_kernel, dim3(rows), dim3(128), 0, static_cast<cudaStream_t>(stream), rows, width, vocab, ids,
                           table, static_cast<long long>(ld_table), table_dtype, scale, out, static_cast<long long>(ld_out), out_dtype));
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}
