// Shared by the sequence-mixer kernels (seqmix.cu: token-serial forms used for single tokens and short portions;
// seqmix_tiled.cu: tiled forms used for prompts): activation helpers, the kernels' argument blocks and the tiled launchers.
#pragma once
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
    case VY_UACT_GELU_TANH: return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
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

// windowed attention with kept first tokens and a sink, over pages
struct WinDev {
  const int* cu; const int* pos0; const int* table; int tw, bs;
  const void* q; long long ldq; int q_dt;
  const void* kp; const void* vp; int pool_dt;
  long long k_row, v_row;   // row strides of the pools in elements (kv_heads * dim and kv_heads * vdim unless the caller views one pool twice)
  int heads, kv_heads, dim, vdim;
  float scale; int window, keep;
  const void* sink; int sink_dt;
  const void* gate; long long ld_gate; int gate_dt;
  void* out; long long ld_out; int out_dt;
};

// recurrences (linear attention with a fixed decay, gated delta rule): state [slots, heads, dim, vdim] fp32
struct RecDev {
  const int* cu; const int* pos0; const int* slot;
  const void* q; long long ldq; const void* k; long long ldk; const void* v; long long ldv; int in_dt; int in_act;
  const void* a; long long ld_a; int a_dt;
  const void* b; long long ld_b; int b_dt;
  const void* a_log; int a_log_dt;
  const float* decay;
  int heads, kv_heads, dim, vdim;
  float unit_eps;
  int prepared;   // delta rule: q / k are unit vectors already (q scaled), `a` holds the decays and `b` the write strengths
  float* state;
  void* out; long long ld_out; int out_dt;
};

// Prompt-sized steps: defined in seqmix_tiled.cu.
cudaError_t launch_linear_attn_chunked(const RecDev& d, int n_seqs, cudaStream_t st);
cudaError_t launch_window_attn_tiled(const WinDev& d, int n_seqs, int max_new, cudaStream_t st);
// Single tokens whose query heads share key / value rows in groups of 8 or more (latent rows): heads as the rows of a tile.
bool window_attn_heads_applies(const WinDev& d);
long long window_attn_heads_workspace_floats(int n_seqs, int heads, int kv_heads, int vdim);
cudaError_t launch_window_attn_heads(const WinDev& d, int n_seqs, float* ws, long long ws_floats, cudaStream_t st, int* launches);

}  // namespace vy
