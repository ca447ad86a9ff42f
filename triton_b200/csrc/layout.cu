// One-time re-layout of canonical MXFP4 weights into the tile-contiguous form the tcgen05 kernel streams.
//
// Canonical (what moe_downcast_mxfp4 writes for w[E,K,N] quantised along K): values [E][N][K/2] bytes,
// byte b of a row holding k = 2b (low nibble) and 2b+1 (high nibble); scales [E][N][K/32] (any strides).
// Tiled: tiles of 128 n x 128 k ordered [E][n_tile][k_tile].
//   value tile: 8 KB = [4 scale groups][128 rows][16 bytes]: the 16 bytes of (group g, row r) are the 32 k values
//               k = 32g .. 32g+31 of that row, so that 8 consecutive lanes reading 8 consecutive rows of one
//               group touch 128 contiguous bytes.  Inside, 32-bit word q covers k = 32g + 8q .. +7 with nibble p
//               holding k + {0,2,4,6,1,3,5,7}[p], so that (word >> 4i) & 0x000F000F yields the pair (2i, 2i+1) in
//               the low and high half-word.
//   scale tile: 128 rows x 4 bytes (the four 32-groups of the k tile).
// Out-of-range n or k is zero (value 0, scale byte 0).
#include "common.cuh"

namespace {

constexpr int TN = 128, TK = 128;

__device__ __forceinline__ uint32_t nibble_interleave(uint32_t w) {   // natural -> (evens | odds << 16)
  uint32_t r = 0;
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    r |= ((w >> (8 * a)) & 0xFu) << (4 * a);             // k = 2a
    r |= ((w >> (8 * a + 4)) & 0xFu) << (16 + 4 * a);    // k = 2a + 1
  }
  return r;
}
__device__ __forceinline__ uint32_t nibble_deinterleave(uint32_t r) {
  uint32_t w = 0;
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    w |= ((r >> (4 * a)) & 0xFu) << (8 * a);
    w |= ((r >> (16 + 4 * a)) & 0xFu) << (8 * a + 4);
  }
  return w;
}

__global__ void __launch_bounds__(256) to_b200_values(const uint8_t* __restrict__ q, int64_t q_stride_e,
                                                      int64_t q_stride_n, int E, int K, int N, int NT, int KT,
                                                      uint32_t* __restrict__ out) {
  const int64_t total = (int64_t)E * NT * KT * TN * 16;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int qw = (int)(i & 3);                       // word inside the 16-byte group chunk
    const int r = (int)((i >> 2) & (TN - 1));
    const int g = (int)((i >> 9) & 3);
    const int j = g * 4 + qw;                          // word of the row: k = 8 j .. 8 j + 7
    int64_t t = i >> 11;
    const int kt = (int)(t % KT); t /= KT;
    const int nt = (int)(t % NT);
    const int e = (int)(t / NT);
    const int n = nt * TN + r, k = kt * TK + j * 8;
    uint32_t w = 0;
    if (n < N && k < K) {
      const uint8_t* src = q + (int64_t)e * q_stride_e + (int64_t)n * q_stride_n + (k >> 1);
      // K is a multiple of 32, so the four bytes are all in range
      w = (uint32_t)src[0] | ((uint32_t)src[1] << 8) | ((uint32_t)src[2] << 16) | ((uint32_t)src[3] << 24);
    }
    out[i] = nibble_interleave(w);
  }
}

__global__ void __launch_bounds__(256) to_b200_scales(const uint8_t* __restrict__ s, int64_t s_stride_e,
                                                      int64_t s_stride_k, int64_t s_stride_n, int E, int K, int N,
                                                      int NT, int KT, uint32_t* __restrict__ out) {
  const int64_t total = (int64_t)E * NT * KT * TN;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int r = (int)(i & (TN - 1));
    int64_t t = i >> 7;
    const int kt = (int)(t % KT); t /= KT;
    const int nt = (int)(t % NT);
    const int e = (int)(t / NT);
    const int n = nt * TN + r;
    uint32_t w = 0;
    if (n < N) {
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const int kg = kt * 4 + g;
        if (kg * 32 < K)
          w |= (uint32_t)s[(int64_t)e * s_stride_e + (int64_t)kg * s_stride_k + (int64_t)n * s_stride_n] << (8 * g);
      }
    }
    out[i] = w;
  }
}

__global__ void __launch_bounds__(256) from_b200_kernel(const uint32_t* __restrict__ values,
                                                        const uint8_t* __restrict__ scales, int E, int K, int N, int NT,
                                                        int KT, uint8_t* __restrict__ q, uint8_t* __restrict__ s) {
  const int64_t words_per_row = K >> 3;
  const int64_t total = (int64_t)E * N * words_per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t wj = i % words_per_row;
    int64_t t = i / words_per_row;
    const int n = (int)(t % N);
    const int e = (int)(t / N);
    const int k = (int)(wj * 8);
    const int nt = n / TN, r = n % TN, kt = k / TK, j = (k % TK) / 8;
    const int64_t tile = ((int64_t)e * NT + nt) * KT + kt;
    if (q) {
      const uint32_t w = nibble_deinterleave(values[tile * (TN * 16) + (j >> 2) * (TN * 4) + r * 4 + (j & 3)]);
      uint8_t* dst = q + ((int64_t)e * N + n) * (K >> 1) + (k >> 1);
      dst[0] = (uint8_t)w; dst[1] = (uint8_t)(w >> 8); dst[2] = (uint8_t)(w >> 16); dst[3] = (uint8_t)(w >> 24);
    }
    if (s && (k & 31) == 0)
      s[((int64_t)e * N + n) * (K >> 5) + (k >> 5)] = scales[tile * (TN * 4) + r * 4 + ((k % TK) >> 5)];
  }
}

int grid_for(int64_t total) {
  int64_t blocks = cdiv64(total, 256);
  int64_t cap = (int64_t)moe_sm_count() * 16;
  if (blocks > cap) blocks = cap;
  return (int)(blocks < 1 ? 1 : blocks);
}

}  // namespace

extern "C" __attribute__((visibility("default"))) size_t moe_weight_b200_value_bytes(int E, int K, int N) {
  return (size_t)E * (size_t)cdiv64(N, TN) * (size_t)cdiv64(K, TK) * (size_t)(TN * TK / 2);
}
extern "C" __attribute__((visibility("default"))) size_t moe_weight_b200_scale_bytes(int E, int K, int N) {
  return (size_t)E * (size_t)cdiv64(N, TN) * (size_t)cdiv64(K, TK) * (size_t)(TN * 4);
}

extern "C" __attribute__((visibility("default"))) int moe_weight_layout_to_b200(const uint8_t* q, int64_t q_stride_e, int64_t q_stride_n, const uint8_t* scale,
                                         int64_t s_stride_e, int64_t s_stride_k, int64_t s_stride_n, int E, int K, int N,
                                         uint8_t* out_values, uint8_t* out_scales, void* stream) {
  MOE_CHECK_ARG(E > 0 && K > 0 && N > 0 && K % 32 == 0, "moe_weight_layout_to_b200: need K %% 32 == 0 (K=%d)", K);
  MOE_CHECK_ARG((q != nullptr) == (out_values != nullptr) && (scale != nullptr) == (out_scales != nullptr) &&
                    (q || scale),
                "moe_weight_layout_to_b200: pass (q, out_values) and/or (scale, out_scales)");
  MOE_CHECK_ARG((uintptr_t)out_values % 16 == 0 && (uintptr_t)out_scales % 16 == 0,
                "moe_weight_layout_to_b200: outputs must be 16-byte aligned");
  const int NT = (int)cdiv64(N, TN), KT = (int)cdiv64(K, TK);
  cudaStream_t st = (cudaStream_t)stream;
  if (q) {
    to_b200_values<<<grid_for((int64_t)E * NT * KT * TN * 16), 256, 0, st>>>(q, q_stride_e, q_stride_n, E, K, N, NT, KT,
                                                                            (uint32_t*)out_values);
    MOE_CHECK_LAUNCH();
  }
  if (scale) {
    to_b200_scales<<<grid_for((int64_t)E * NT * KT * TN), 256, 0, st>>>(scale, s_stride_e, s_stride_k, s_stride_n, E, K,
                                                                       N, NT, KT, (uint32_t*)out_scales);
    MOE_CHECK_LAUNCH();
  }
  return MOE_OK;
}

extern "C" __attribute__((visibility("default"))) int moe_weight_layout_from_b200(const uint8_t* values, const uint8_t* scales, int E, int K, int N,
                                           uint8_t* q, uint8_t* scale, void* stream) {
  MOE_CHECK_ARG(E > 0 && K > 0 && N > 0 && K % 32 == 0, "moe_weight_layout_from_b200: need K %% 32 == 0 (K=%d)", K);
  MOE_CHECK_ARG((values != nullptr) == (q != nullptr) && (scales != nullptr) == (scale != nullptr) && (q || scale),
                "moe_weight_layout_from_b200: pass (values, q) and/or (scales, scale)");
  const int NT = (int)cdiv64(N, TN), KT = (int)cdiv64(K, TK);
  from_b200_kernel<<<grid_for((int64_t)E * N * (K >> 3)), 256, 0, (cudaStream_t)stream>>>(
      (const uint32_t*)values, scales, E, K, N, NT, KT, q, scale);
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}

// ---- block-scaled layout (what the kind::mxf8f6f4 kernel streams) --------------------------------------------------
// Tiles of 128 n x 128 k ordered [E][k_tile][n_block]: the blocks a CTA tile needs in one k step are neighbours.
//   value tile: 128 rows x 64 bytes, byte b of a row holding k = 2b (low nibble) and 2b + 1 (high nibble) -- plain
//               packed e2m1, which the TMA unit expands to one byte per element on its way into shared memory;
//   scale tile: 512 bytes, the scale of (row r, group g) at (r % 32) * 16 + (r / 32) * 4 + g: the order tcgen05.cp
//               (32x128b.warpx4) moves into tensor memory, the same 128 x 4 packed block as BlackwellMXScaleLayout of
//               the reference (tensor_details/layout_details/blackwell_scale.py:165-175).
// Out-of-range n or k is zero (value 0, scale byte 0 = 2^-127).
namespace {

__global__ void __launch_bounds__(256) to_b200mx_values(const uint8_t* __restrict__ q, int64_t q_stride_e,
                                                        int64_t q_stride_n, int E, int K, int N, int NB, int KT,
                                                        uint32_t* __restrict__ out) {
  const int64_t total = (int64_t)E * KT * NB * TN * 16;             // 32-bit words
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int j = (int)(i & 15);                       // word of the row: k = 8 j .. 8 j + 7
    const int r = (int)((i >> 4) & (TN - 1));
    int64_t t = i >> 11;
    const int nb = (int)(t % NB); t /= NB;
    const int kt = (int)(t % KT);
    const int e = (int)(t / KT);
    const int n = nb * TN + r, k = kt * TK + j * 8;
    uint32_t w = 0;
    if (n < N && k < K) {
      const uint8_t* src = q + (int64_t)e * q_stride_e + (int64_t)n * q_stride_n + (k >> 1);
      w = (uint32_t)src[0] | ((uint32_t)src[1] << 8) | ((uint32_t)src[2] << 16) | ((uint32_t)src[3] << 24);
    }
    out[i] = w;
  }
}

__global__ void __launch_bounds__(256) to_b200mx_scales(const uint8_t* __restrict__ s, int64_t s_stride_e,
                                                        int64_t s_stride_k, int64_t s_stride_n, int E, int K, int N,
                                                        int NB, int KT, uint32_t* __restrict__ out) {
  const int64_t total = (int64_t)E * KT * NB * TN;                  // one 32-bit word = the 4 groups of a row
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i & (TN - 1));                 // word inside the tile: (r % 32) * 4 + r / 32
    const int r = (c >> 2) + 32 * (c & 3);
    int64_t t = i >> 7;
    const int nb = (int)(t % NB); t /= NB;
    const int kt = (int)(t % KT);
    const int e = (int)(t / KT);
    const int n = nb * TN + r;
    uint32_t w = 0;
    if (n < N) {
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const int kg = kt * 4 + g;
        if (kg * 32 < K)
          w |= (uint32_t)s[(int64_t)e * s_stride_e + (int64_t)kg * s_stride_k + (int64_t)n * s_stride_n] << (8 * g);
      }
    }
    out[i] = w;
  }
}

__global__ void __launch_bounds__(256) from_b200mx_kernel(const uint32_t* __restrict__ values,
                                                          const uint8_t* __restrict__ scales, int E, int K, int N, int NB,
                                                          int KT, uint8_t* __restrict__ q, uint8_t* __restrict__ s) {
  const int64_t words_per_row = K >> 3;
  const int64_t total = (int64_t)E * N * words_per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t wj = i % words_per_row;
    int64_t t = i / words_per_row;
    const int n = (int)(t % N);
    const int e = (int)(t / N);
    const int k = (int)(wj * 8);
    const int nb = n / TN, r = n % TN, kt = k / TK, j = (k % TK) / 8;
    const int64_t tile = ((int64_t)e * KT + kt) * NB + nb;
    if (q) {
      const uint32_t w = values[tile * (TN * 16) + r * 16 + j];
      uint8_t* dst = q + ((int64_t)e * N + n) * (K >> 1) + (k >> 1);
      dst[0] = (uint8_t)w; dst[1] = (uint8_t)(w >> 8); dst[2] = (uint8_t)(w >> 16); dst[3] = (uint8_t)(w >> 24);
    }
    if (s && (k & 31) == 0)
      s[((int64_t)e * N + n) * (K >> 5) + (k >> 5)] = scales[tile * 512 + (r & 31) * 16 + (r >> 5) * 4 + ((k % TK) >> 5)];
  }
}

}  // namespace

extern "C" __attribute__((visibility("default"))) int moe_weight_layout_to_b200mx(const uint8_t* q, int64_t q_stride_e, int64_t q_stride_n, const uint8_t* scale,
                                         int64_t s_stride_e, int64_t s_stride_k, int64_t s_stride_n, int E, int K, int N,
                                         uint8_t* out_values, uint8_t* out_scales, void* stream) {
  MOE_CHECK_ARG(E > 0 && K > 0 && N > 0 && K % 32 == 0, "moe_weight_layout_to_b200mx: need K %% 32 == 0 (K=%d)", K);
  MOE_CHECK_ARG((q != nullptr) == (out_values != nullptr) && (scale != nullptr) == (out_scales != nullptr) &&
                    (q || scale),
                "moe_weight_layout_to_b200mx: pass (q, out_values) and/or (scale, out_scales)");
  MOE_CHECK_ARG((uintptr_t)out_values % 32 == 0 && (uintptr_t)out_scales % 16 == 0,
                "moe_weight_layout_to_b200mx: values must be 32-byte and scales 16-byte aligned");
  const int NB = (int)cdiv64(N, TN), KT = (int)cdiv64(K, TK);
  cudaStream_t st = (cudaStream_t)stream;
  if (q) {
    to_b200mx_values<<<grid_for((int64_t)E * NB * KT * TN * 16), 256, 0, st>>>(q, q_stride_e, q_stride_n, E, K, N, NB, KT,
                                                                              (uint32_t*)out_values);
    MOE_CHECK_LAUNCH();
  }
  if (scale) {
    to_b200mx_scales<<<grid_for((int64_t)E * NB * KT * TN), 256, 0, st>>>(scale, s_stride_e, s_stride_k, s_stride_n, E, K,
                                                                         N, NB, KT, (uint32_t*)out_scales);
    MOE_CHECK_LAUNCH();
  }
  return MOE_OK;
}

extern "C" __attribute__((visibility("default"))) int moe_weight_layout_from_b200mx(const uint8_t* values, const uint8_t* scales, int E, int K, int N,
                                           uint8_t* q, uint8_t* scale, void* stream) {
  MOE_CHECK_ARG(E > 0 && K > 0 && N > 0 && K % 32 == 0, "moe_weight_layout_from_b200mx: need K %% 32 == 0 (K=%d)", K);
  MOE_CHECK_ARG((values != nullptr) == (q != nullptr) && (scales != nullptr) == (scale != nullptr) && (q || scale),
                "moe_weight_layout_from_b200mx: pass (values, q) and/or (scales, scale)");
  const int NB = (int)cdiv64(N, TN), KT = (int)cdiv64(K, TK);
  from_b200mx_kernel<<<grid_for((int64_t)E * N * (K >> 3)), 256, 0, (cudaStream_t)stream>>>(
      (const uint32_t*)values, scales, E, K, N, NB, KT, q, scale);
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}
