// General ragged grouped GEMM on CUDA cores: any of fp32/fp16/bf16 activations against dense weights of
// the same type or MXFP4 weights in the canonical (K-packed) layout.  It is the path for shapes and
// layouts the tensor-core kernel does not take (small or odd problems, canonical weights, the dense
// router GEMM) and the differential check for that kernel.  Role of triton_kernels
// matmul_details/_matmul.py:43 (the non-persistent pointer kernel).
//
// Block tile 64 x 64 x 32 (one MX scale group per k step), 256 threads, 4 x 4 outputs per thread,
// fp32 accumulation.
#include "gemm_common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 32;

__device__ __forceinline__ float e2m1_val(uint32_t code) {
  const uint32_t mag = code & 7u;
  uint32_t bits = (mag == 0) ? 0u : (mag == 1) ? 0x3F000000u : (((mag >> 1) + 126u) << 23) | ((mag & 1u) << 22);
  return __uint_as_float(bits | ((code & 8u) << 28));
}

template <typename TX, typename TY, int WKIND>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const GemmParams p) {
  __shared__ float Xs[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  __shared__ int64_t s_src_row[BM];

  int e; int64_t row0; int rows;
  if (!gemm_map_block<BM>(p, blockIdx.y, e, row0, rows)) return;
  const int n0 = blockIdx.x * BN;
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;

  if (tid < BM) {
    int64_t src = -1;
    if (tid < rows) {
      const int64_t m = row0 + tid;
      src = p.gather_indx ? (int64_t)p.gather_indx[m] : m;
      if (src >= p.rows_x) src = -1;
    }
    s_src_row[tid] = src;
  }
  __syncthreads();

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  const TX* X = (const TX*)p.x;
  for (int k0 = 0; k0 < p.K; k0 += BK) {
    // activations: 64 rows x 32 k, 8 elements per thread
    {
      const int r = tid >> 2, kc = (tid & 3) * 8;
      const int64_t src = s_src_row[r];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int k = k0 + kc + j;
        float v = 0.0f;
        if (src >= 0 && k < p.K) v = to_f32<TX>(X[src * p.ld_x + k]);
        Xs[kc + j][r] = v;
      }
    }
    // weights: 32 k x 64 n
    if constexpr (WKIND == MOE_W_MX4_CANONICAL) {
      const int n = tid >> 2, part = tid & 3;   // 8 k values = 4 bytes
      const int gn = n0 + n;
      float w8[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) w8[j] = 0.0f;
      if (gn < p.N && k0 + part * 8 < p.K) {
        const uint8_t* qrow = (const uint8_t*)p.w + (int64_t)e * p.w_stride_e + (int64_t)gn * p.w_stride_n;
        const uint32_t word = *reinterpret_cast<const uint32_t*>(qrow + (k0 >> 1) + part * 4);
        const uint32_t sb = p.w_scale[(int64_t)e * p.ws_stride_e + (int64_t)(k0 >> 5) * p.ws_stride_k +
                                      (int64_t)gn * p.ws_stride_n];
        // scale as the reference's bf16 upcast sees it: bits (byte << 7) in bf16, i.e. byte 0 -> 0.0
        const float s = __uint_as_float(sb << 23);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          // e2m1 value times a power of two, rounded to bf16 exactly as upcast_from_mxfp(..., bf16) would
          w8[j] = __bfloat162float(__float2bfloat16_rn(e2m1_val((word >> (4 * j)) & 0xFu) * s));
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) Ws[part * 8 + j][n] = w8[j];
    } else {
      const int k = tid >> 3, nc = (tid & 7) * 8;
      const TX* W = (const TX*)p.w + (int64_t)e * p.w_stride_e;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int gn = n0 + nc + j;
        float v = 0.0f;
        if (gn < p.N && k0 + k < p.K) v = to_f32<TX>(W[(int64_t)(k0 + k) * p.w_stride_k + (int64_t)gn * p.w_stride_n]);
        Ws[k][nc + j] = v;
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = Xs[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }

  // epilogue
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty * 4 + i;
    if (r >= rows) continue;
    const int64_t m = row0 + r;
    int64_t dst = m;
    if (p.scatter_indx) {
      dst = p.scatter_indx[m];
      if (dst < 0) continue;
    }
    TY* yrow = gemm_out_row<TY>(p, dst);
    const float beta = p.betas ? p.betas[m] : 1.0f;
    const float gamma = p.gammas ? p.gammas[m] : 1.0f;
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      float t = acc[i][j];
      if (p.bias && gn < p.N) t += load_bias(p.bias, p.bias_dtype, (int64_t)e * p.ld_bias + gn) * beta;
      if (p.has_out_alpha) t *= p.out_alpha;
      v[j] = t;
    }
    if (p.activation == MOE_ACT_SWIGLU) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int gn = n0 + tx * 4 + 2 * j;
        if (gn + 1 < p.N)
          yrow[gn >> 1] =
              from_f32<TY>(gemm_swiglu(v[2 * j], v[2 * j + 1], p.act_alpha, p.act_limit, p.act_has_limit) * gamma);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int gn = n0 + tx * 4 + j;
        if (gn < p.N) yrow[gn] = from_f32<TY>(v[j] * gamma);
      }
    }
  }
}

template <typename TX, typename TY>
int launch_simt(const GemmParams& p, int w_kind, int64_t grid_m, cudaStream_t st) {
  dim3 grid((unsigned)cdiv64(p.N, BN), (unsigned)grid_m);
  if (w_kind == MOE_W_MX4_CANONICAL)
    gemm_simt_kernel<TX, TY, MOE_W_MX4_CANONICAL><<<grid, 256, 0, st>>>(p);
  else
    gemm_simt_kernel<TX, TY, MOE_W_DENSE><<<grid, 256, 0, st>>>(p);
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}

}  // namespace

int moe_gemm_simt_launch(const GemmParams& p, int x_dtype, int y_dtype, int w_kind, int64_t grid_m, cudaStream_t st) {
  MOE_CHECK_ARG(grid_m <= 65535, "moe_grouped_gemm: too many row blocks for the SIMT kernel (%lld)", (long long)grid_m);
#define MOE_SIMT_CASE(DX, TX, DY, TY) \
  if (x_dtype == DX && y_dtype == DY) return launch_simt<TX, TY>(p, w_kind, grid_m, st);
  MOE_SIMT_CASE(MOE_BF16, __nv_bfloat16, MOE_BF16, __nv_bfloat16)
  MOE_SIMT_CASE(MOE_BF16, __nv_bfloat16, MOE_F32, float)
  MOE_SIMT_CASE(MOE_F16, __half, MOE_F16, __half)
  MOE_SIMT_CASE(MOE_F16, __half, MOE_F32, float)
  MOE_SIMT_CASE(MOE_F32, float, MOE_F32, float)
  MOE_SIMT_CASE(MOE_F32, float, MOE_BF16, __nv_bfloat16)
#undef MOE_SIMT_CASE
  moe_set_error("moe_grouped_gemm: dtype combination (x %d -> y %d) unsupported", x_dtype, y_dtype);
  return MOE_ERR_UNSUPPORTED;
}
