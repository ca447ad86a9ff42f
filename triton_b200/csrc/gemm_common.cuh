// Pieces shared by the SIMT and the tcgen05 grouped-GEMM kernels: the device-side argument block, the
// tile -> (expert, row block) mapping through the ragged block schedule, and the fused epilogue
// (bias * beta, out_alpha, SwiGLU, gamma, cast, scatter) in the order of triton_kernels
// matmul_details/_p_matmul.py:610-628.
#pragma once
#include "common.cuh"

struct GemmParams {
  const void* x; int64_t ld_x; int64_t rows_x;
  const void* w; int64_t w_stride_e, w_stride_k, w_stride_n;
  const uint8_t* w_scale; int64_t ws_stride_e, ws_stride_k, ws_stride_n;
  int E, K, N;
  const int32_t* slice_sizes; const int32_t* slice_offs;
  const int32_t* block_offs; const int32_t* block_sched;   // rows for this kernel's BLOCK_M
  int64_t M;
  const void* bias; int bias_dtype; int64_t ld_bias;
  const int32_t* gather_indx; const int32_t* scatter_indx;
  const float* betas; const float* gammas;
  float out_alpha; int has_out_alpha;
  int activation; float act_alpha, act_limit; int act_has_limit;
  void* y; int64_t ld_y;
  int32_t* status;
  void* y_peers[MOE_MAX_PEERS]; int n_y_peers; int64_t y_rows_per_peer;   // output rows spread over peer buffers
};

// first element of output row `dst`: in y, or in the peer buffer that holds that row
template <typename TY> __device__ __forceinline__ TY* gemm_out_row(const GemmParams& p, int64_t dst) {
  if (p.n_y_peers == 0) return (TY*)p.y + dst * p.ld_y;
  const int64_t peer = dst / p.y_rows_per_peer;
  return (TY*)p.y_peers[peer] + (dst - peer * p.y_rows_per_peer) * p.ld_y;
}

__device__ __forceinline__ float load_bias(const void* bias, int dtype, int64_t off) {
  switch (dtype) {
    case MOE_F32: return ((const float*)bias)[off];
    case MOE_F16: return __half2float(((const __half*)bias)[off]);
    default: return __bfloat162float(((const __nv_bfloat16*)bias)[off]);
  }
}

__device__ __forceinline__ float gemm_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// SwiGLU on one (gate, linear) pair of fp32 accumulators (triton_kernels swiglu_details/_swiglu.py:55-64)
__device__ __forceinline__ float gemm_swiglu(float g, float l, float alpha, float limit, int has_limit) {
  if (has_limit) {
    g = fminf(g, limit);
    l = fminf(fmaxf(l, -limit), limit);
  }
  // approximate reciprocal: an IEEE division would take its slow path whenever the exponential overflows
  const float s = __fdividef(g, 1.0f + gemm_ex2(-alpha * g * 1.4426950408889634f));
  return fmaf(s, l, s);
}

// Row block -> (expert, first row, valid rows).  Returns false when the block is padding.
template <int BLOCK_M>
__device__ __forceinline__ bool gemm_map_block(const GemmParams& p, int64_t pid_m, int& e, int64_t& row0, int& rows) {
  if (p.slice_sizes == nullptr) {
    e = 0;
    row0 = pid_m * BLOCK_M;
    if (row0 >= p.M) return false;
    rows = (int)min((int64_t)BLOCK_M, p.M - row0);
    return true;
  }
  const uint32_t ent = (uint32_t)p.block_sched[pid_m];
  if (ent == 0xFFFFFFFFu) return false;
  e = (int)(ent & 0xFFFFu);
  const int blk = (int)(ent >> 16);
  const int size = p.slice_sizes[e];
  row0 = (int64_t)p.slice_offs[e] + (int64_t)blk * BLOCK_M;
  rows = min(BLOCK_M, size - blk * BLOCK_M);
  return rows > 0;
}
