// MXFP4 quantiser / dequantiser for sm_100a: e2m1 values packed two per byte (element 2i in the low
// nibble) with one e8m0 scale byte per 32 elements along the quantised axis.
//
// Arithmetic (bit-exact with triton_kernels numerics_details/mxfp_details/_downcast_to_mxfp.py:33-147
// and _upcast_from_mxfp.py:8-53, 109-220):
//   m      = max |x| over the 32-group, in fp32
//   ds     = m / 6 (ROUND_UP) or m / 4 (ROUND_DOWN), IEEE round-to-nearest division
//   u      = (bits(ds) + 0x007FFFFF) & 0x7F800000  (ROUND_UP: next power of two)
//            bits(ds) & 0x7F800000                  (ROUND_DOWN)
//   scale  = u >> 23 ;  inv = (u == 0) ? 0 : 1 / float(u)
//   code   = RTNE_e2m1(x * inv), saturating at +-6
// Both kernels are HBM-bound: 16-byte loads/stores, one thread per 32-group on the contiguous path (one division and
// one scale per group, 16 bytes of codes per store).
#include "common.cuh"
#include <cuda_fp4.h>
#include <type_traits>

namespace {

__device__ __forceinline__ uint32_t scale_bits(float m, int mode) {
  if (mode == MOE_ROUND_UP) {
    float ds = __fdiv_rn(m, 6.0f);
    return (__float_as_uint(ds) + 0x007FFFFFu) & 0x7F800000u;
  }
  float ds = __fdiv_rn(m, 4.0f);
  return __float_as_uint(ds) & 0x7F800000u;
}

// 1 / u for u = 2^(e - 127) stored as e << 23: the exponent mirrored around the bias, exactly what an IEEE division
// returns.  e = 0 (group of zeros) gives 0 as in the reference; e <= 253 always holds because max|x| / 4 < 2^127.
__device__ __forceinline__ float inv_scale(uint32_t u) {
  return (u == 0u) ? 0.0f : __uint_as_float(0x7F000000u - u);
}

// Position of a grid-stride loop over [rows][chunks per row] without a division per iteration.
template <typename I> struct RowCursorT {
  I row, c, step_row, step_c, per_row;
  __device__ __forceinline__ RowCursorT(int64_t first, int64_t stride, int64_t chunks_per_row) {
    per_row = (I)chunks_per_row;
    row = (I)(first / chunks_per_row); c = (I)(first - (int64_t)row * chunks_per_row);
    step_row = (I)(stride / chunks_per_row); step_c = (I)(stride - (int64_t)step_row * chunks_per_row);
  }
  __device__ __forceinline__ void next() {
    row += step_row; c += step_c;
    if (c >= per_row) { c -= per_row; ++row; }
  }
};
using RowCursor = RowCursorT<int64_t>;

// two fp32 -> one byte: `lo` in bits 0..3, `hi` in bits 4..7 (round-to-nearest-even, saturating)
__device__ __forceinline__ uint32_t e2m1x2(float lo, float hi) {
  return (uint32_t)__nv_cvt_float2_to_fp4x2(make_float2(lo, hi), __NV_E2M1, cudaRoundNearest);
}

template <typename T> struct Vec16;  // 16-byte vector of T
template <> struct Vec16<__nv_bfloat16> { static constexpr int N = 8; };
template <> struct Vec16<__half> { static constexpr int N = 8; };
template <> struct Vec16<float> { static constexpr int N = 4; };

// ---- contiguous path: quant axis has unit stride, rows 16-byte aligned ------------------------------
// One thread owns whole 32-groups: 64 (or 128) contiguous input bytes as 16-byte loads, one division and one scale
// per group, one 16-byte store of the 32 codes and one byte of scale.  GROUPS_UNROLL groups are loaded before the first
// is converted, so that enough bytes are in flight per SM to cover the HBM latency.
constexpr int GROUPS_UNROLL = 2;

template <typename T> __device__ __forceinline__ void unpack16(const uint4& r, float* v);
template <> __device__ __forceinline__ void unpack16<__nv_bfloat16>(const uint4& r, float* v) {
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[2 * j] = __uint_as_float(w[j] << 16);
    v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
  }
}
template <> __device__ __forceinline__ void unpack16<__half>(const uint4& r, float* v) {
  const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __half22float2(h[j]);
    v[2 * j] = f.x;
    v[2 * j + 1] = f.y;
  }
}
template <> __device__ __forceinline__ void unpack16<float>(const uint4& r, float* v) {
  v[0] = __uint_as_float(r.x); v[1] = __uint_as_float(r.y); v[2] = __uint_as_float(r.z); v[3] = __uint_as_float(r.w);
}

// the 32 values of a group as VPG raw 16-byte vectors -> scale bits and 16 bytes of codes.  The vectors are unpacked
// twice (once for the maximum, once for the codes) instead of holding 32 floats across the division.
template <typename T, int VPG>
__device__ __forceinline__ uint4 quantise_raw(const uint4 (&raw)[VPG], int mode, uint32_t& sc) {
  constexpr int EPV = 32 / VPG;
  float m = 0.0f;
#pragma unroll
  for (int k = 0; k < VPG; ++k) {
    float v[EPV];
    unpack16<T>(raw[k], v);
#pragma unroll
    for (int j = 0; j < EPV; ++j) m = fmaxf(m, fabsf(v[j]));
  }
  sc = scale_bits(m, mode);
  const float inv = inv_scale(sc);
  uint32_t w[4];
  if constexpr (EPV == 8) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float v[8];
      unpack16<T>(raw[k], v);
      const uint32_t b0 = e2m1x2(v[0] * inv, v[1] * inv), b1 = e2m1x2(v[2] * inv, v[3] * inv);
      const uint32_t b2 = e2m1x2(v[4] * inv, v[5] * inv), b3 = e2m1x2(v[6] * inv, v[7] * inv);
      w[k] = __byte_perm(b0 | (b1 << 8), b2 | (b3 << 8), 0x5410);
    }
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float v[8];
      unpack16<T>(raw[2 * k], v);
      unpack16<T>(raw[2 * k + 1], v + 4);
      const uint32_t b0 = e2m1x2(v[0] * inv, v[1] * inv), b1 = e2m1x2(v[2] * inv, v[3] * inv);
      const uint32_t b2 = e2m1x2(v[4] * inv, v[5] * inv), b3 = e2m1x2(v[6] * inv, v[7] * inv);
      w[k] = __byte_perm(b0 | (b1 << 8), b2 | (b3 << 8), 0x5410);
    }
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// 32 fp32 values -> scale bits and 16 bytes of codes
__device__ __forceinline__ uint4 quantise_group(const float (&v)[32], int mode, uint32_t& sc) {
  float m = 0.0f;
#pragma unroll
  for (int j = 0; j < 32; ++j) m = fmaxf(m, fabsf(v[j]));
  sc = scale_bits(m, mode);
  const float inv = inv_scale(sc);
  uint32_t w[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const uint32_t b0 = e2m1x2(v[8 * k] * inv, v[8 * k + 1] * inv), b1 = e2m1x2(v[8 * k + 2] * inv, v[8 * k + 3] * inv);
    const uint32_t b2 = e2m1x2(v[8 * k + 4] * inv, v[8 * k + 5] * inv), b3 = e2m1x2(v[8 * k + 6] * inv, v[8 * k + 7] * inv);
    w[k] = __byte_perm(b0 | (b1 << 8), b2 | (b3 << 8), 0x5410);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

template <typename T, typename I>
__global__ void __launch_bounds__(256, sizeof(T) == 2 ? 3 : 2) downcast_rows_kernel(const T* __restrict__ x, int64_t n_rows, int64_t quant,
                                                            int64_t outer, int64_t sx_batch, int64_t sx_outer,
                                                            uint8_t* __restrict__ q, uint8_t* __restrict__ scale,
                                                            int mode) {
  constexpr int EPV = 16 / (int)sizeof(T);               // elements per 16-byte vector
  constexpr int VPG = 32 / EPV;                          // vectors per group
  const int64_t groups_per_row = quant >> 5;
  const int64_t total = n_rows * groups_per_row;
  const int64_t stride = (int64_t)gridDim.x * (GROUPS_UNROLL * 256);
  const int64_t tile0 = (int64_t)blockIdx.x * (GROUPS_UNROLL * 256);
  RowCursorT<I> cur[GROUPS_UNROLL] = {RowCursorT<I>(tile0 + threadIdx.x, stride, groups_per_row),
                                      RowCursorT<I>(tile0 + 256 + threadIdx.x, stride, groups_per_row)};
  const bool one_batch = outer == n_rows;
  for (int64_t tile = tile0; tile < total; tile += stride) {
    uint4 raw[GROUPS_UNROLL][VPG];
    bool live[GROUPS_UNROLL];
#pragma unroll
    for (int u = 0; u < GROUPS_UNROLL; ++u) {
      live[u] = tile + u * 256 + threadIdx.x < total;
      if (live[u]) {
        const int64_t row = cur[u].row, c = cur[u].c;
        int64_t b = 0, o = row;
        if (!one_batch) { b = row / outer; o = row - b * outer; }
        const uint4* src = reinterpret_cast<const uint4*>(x + b * sx_batch + o * sx_outer + c * 32);
#pragma unroll
        for (int k = 0; k < VPG; ++k) raw[u][k] = src[k];
      }
    }
#pragma unroll
    for (int u = 0; u < GROUPS_UNROLL; ++u) {
      if (live[u]) {
        uint32_t sc;
        const uint4 codes = quantise_raw<T, VPG>(raw[u], mode, sc);
        const int64_t row = cur[u].row, c = cur[u].c;
        *reinterpret_cast<uint4*>(q + row * (quant >> 1) + c * 16) = codes;
        scale[row * groups_per_row + c] = (uint8_t)(sc >> 23);
      }
      cur[u].next();
    }
  }
}

// ---- quantised axis strided, the other axis contiguous (axis 0 of a row-major matrix): a thread owns the 32-groups of
// two neighbouring columns, so that a warp load covers 128 (bf16 / fp16) contiguous bytes; each column's codes are 16
// contiguous bytes of the output.
template <typename T>
__global__ void __launch_bounds__(128) downcast_cols2_kernel(const T* __restrict__ x, int64_t batch, int64_t outer,
                                                             int64_t quant, int64_t sx_batch, int64_t sx_quant,
                                                             uint8_t* __restrict__ q, uint8_t* __restrict__ scale, int mode) {
  const int64_t groups = quant >> 5;
  const int64_t pairs = outer >> 1;
  const int64_t total = batch * groups * pairs;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t op = i % pairs;
    const int64_t t = i / pairs;
    const int64_t g = t % groups;
    const int64_t b = t / groups;
    const T* src = x + b * sx_batch + g * 32 * sx_quant + op * 2;
    float v0[32], v1[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if constexpr (sizeof(T) == 2) {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(src + j * sx_quant);
        if constexpr (std::is_same<T, __nv_bfloat16>::value) {
          v0[j] = __uint_as_float(w << 16);
          v1[j] = __uint_as_float(w & 0xFFFF0000u);
        } else {
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
          v0[j] = f.x;
          v1[j] = f.y;
        }
      } else {
        const float2 f = *reinterpret_cast<const float2*>(src + j * sx_quant);
        v0[j] = f.x;
        v1[j] = f.y;
      }
    }
    uint32_t s0, s1;
    const uint4 c0 = quantise_group(v0, mode, s0), c1 = quantise_group(v1, mode, s1);
    const int64_t row = b * outer + op * 2;
    *reinterpret_cast<uint4*>(q + row * (quant >> 1) + g * 16) = c0;
    *reinterpret_cast<uint4*>(q + (row + 1) * (quant >> 1) + g * 16) = c1;
    scale[row * groups + g] = (uint8_t)(s0 >> 23);
    scale[(row + 1) * groups + g] = (uint8_t)(s1 >> 23);
  }
}

// ---- strided path: any strides; consecutive threads walk the `outer` axis ---------------------------
template <typename T>
__global__ void __launch_bounds__(256) downcast_strided_kernel(const T* __restrict__ x, int64_t batch, int64_t outer,
                                                               int64_t quant, int64_t sx_batch, int64_t sx_outer,
                                                               int64_t sx_quant, uint8_t* __restrict__ q,
                                                               uint8_t* __restrict__ scale, int mode) {
  const int64_t groups = quant >> 5;
  const int64_t total = batch * outer * groups;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t o = i % outer;
    const int64_t t = i / outer;
    const int64_t g = t % groups;
    const int64_t b = t / groups;
    const T* src = x + b * sx_batch + o * sx_outer + g * 32 * sx_quant;
    float v[32];
    float m = 0.0f;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      v[j] = to_f32<T>(src[j * sx_quant]);
      m = fmaxf(m, fabsf(v[j]));
    }
    const uint32_t u = scale_bits(m, mode);
    const float inv = inv_scale(u);
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      uint32_t p = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) p |= e2m1x2(v[8 * k + 2 * j] * inv, v[8 * k + 2 * j + 1] * inv) << (8 * j);
      w[k] = p;
    }
    const int64_t row = b * outer + o;
    *reinterpret_cast<uint4*>(q + row * (quant >> 1) + g * 16) = make_uint4(w[0], w[1], w[2], w[3]);
    scale[row * groups + g] = (uint8_t)(u >> 23);
  }
}

__device__ __forceinline__ float e2m1_to_f32(uint32_t code) {
  // magnitude bits e1 e0 m: 0, .5, 1, 1.5, 2, 3, 4, 6
  const uint32_t mag = code & 7u;
  uint32_t bits = (mag == 0) ? 0u : (mag == 1) ? 0x3F000000u : (((mag >> 1) + 126u) << 23) | ((mag & 1u) << 22);
  return __uint_as_float(bits | ((code & 8u) << 28));
}

template <typename T> __device__ __forceinline__ float finite_max();
template <> __device__ __forceinline__ float finite_max<float>() { return 3.4028234663852886e+38f; }
template <> __device__ __forceinline__ float finite_max<__nv_bfloat16>() { return 3.3895313892515355e+38f; }
template <> __device__ __forceinline__ float finite_max<__half>() { return 65504.0f; }

template <typename T>
__device__ __forceinline__ T dequant_one(uint32_t code, float s, bool nan_scale) {
  float r = e2m1_to_f32(code) * s;
  const float mx = finite_max<T>();
  r = fminf(fmaxf(r, -mx), mx);
  if (nan_scale) r = __uint_as_float(0x7FC00000u);
  return from_f32<T>(r);
}

// bf16 fast path: the three magnitude bits of a code placed at bf16 bits 8:6 are value * 2^-126, and one
// bf16x2 multiply by 2^(sb - 1) gives value * 2^(sb - 127) exactly (every product is representable; sb = 0 multiplies
// by zero as the reference's scale bits 0 << 23 do).  Scale bytes from 253 up can overflow and take the general path.
__device__ __forceinline__ uint32_t bf16x2_mul_rn(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// codes k and k + 4 of word w (nibble p holds element p) -> bf16x2 (low half: element k) of value * 2^-126
template <int K> __device__ __forceinline__ uint32_t e2m1_pair_k(uint32_t w) {
  const uint32_t mag = (K < 2 ? (w << (6 - 4 * K)) : (w >> (4 * K - 6))) & 0x01C001C0u;
  const uint32_t sgn = (w << (12 - 4 * K)) & 0x80008000u;
  return mag | sgn;
}
__device__ __forceinline__ uint4 upcast8_bf16(uint32_t w, uint32_t sb) {
  uint32_t c2, r[4];
  if (sb <= 128u) {
    c2 = (sb ? ((sb + 126u) << 7) : 0u) * 0x10001u;
    r[0] = bf16x2_mul_rn(e2m1_pair_k<0>(w), c2); r[1] = bf16x2_mul_rn(e2m1_pair_k<1>(w), c2);
    r[2] = bf16x2_mul_rn(e2m1_pair_k<2>(w), c2); r[3] = bf16x2_mul_rn(e2m1_pair_k<3>(w), c2);
  } else {                                           // 2^(sb - 1) is not a bf16: multiply by 2^126, then by 2^(sb - 127)
    const uint32_t k2 = 0x7E807E80u, s2 = (sb << 7) * 0x10001u;
    r[0] = bf16x2_mul_rn(bf16x2_mul_rn(e2m1_pair_k<0>(w), k2), s2); r[1] = bf16x2_mul_rn(bf16x2_mul_rn(e2m1_pair_k<1>(w), k2), s2);
    r[2] = bf16x2_mul_rn(bf16x2_mul_rn(e2m1_pair_k<2>(w), k2), s2); r[3] = bf16x2_mul_rn(bf16x2_mul_rn(e2m1_pair_k<3>(w), k2), s2);
  }
  // r[k] = (element k, element k + 4): back to element order
  return make_uint4(__byte_perm(r[0], r[1], 0x5410), __byte_perm(r[2], r[3], 0x5410), __byte_perm(r[0], r[1], 0x7632),
                    __byte_perm(r[2], r[3], 0x7632));
}

constexpr int ROWS_UNROLL = 4;
// contiguous output: thread owns 8 elements (4 input bytes) of each of ROWS_UNROLL chunks per iteration
template <typename T>
__global__ void __launch_bounds__(256) upcast_rows_kernel(const uint8_t* __restrict__ q,
                                                          const uint8_t* __restrict__ scale, T* __restrict__ out,
                                                          int64_t n_rows, int64_t quant, int64_t outer,
                                                          int64_t so_batch, int64_t so_outer) {
  const int64_t chunks_per_row = quant >> 3;
  const int64_t total = n_rows * chunks_per_row;
  const int64_t stride = (int64_t)gridDim.x * (ROWS_UNROLL * 256);
  const int64_t tile0 = (int64_t)blockIdx.x * (ROWS_UNROLL * 256);
  RowCursor cur[ROWS_UNROLL] = {RowCursor(tile0 + threadIdx.x, stride, chunks_per_row),
                                RowCursor(tile0 + 256 + threadIdx.x, stride, chunks_per_row),
                                RowCursor(tile0 + 512 + threadIdx.x, stride, chunks_per_row),
                                RowCursor(tile0 + 768 + threadIdx.x, stride, chunks_per_row)};
  const bool one_batch = outer == n_rows;
  for (int64_t tile = tile0; tile < total; tile += stride) {
    uint32_t w[ROWS_UNROLL], sb[ROWS_UNROLL];
#pragma unroll
    for (int u = 0; u < ROWS_UNROLL; ++u) {
      const bool live = tile + u * 256 + threadIdx.x < total;
      const int64_t row = live ? cur[u].row : 0, c = live ? cur[u].c : 0;
      w[u] = *reinterpret_cast<const uint32_t*>(q + row * (quant >> 1) + c * 4);
      sb[u] = scale[row * (quant >> 5) + (c >> 2)];
    }
#pragma unroll
    for (int u = 0; u < ROWS_UNROLL; ++u) {
      const bool live = tile + u * 256 + threadIdx.x < total;
      const int64_t row = cur[u].row, c = cur[u].c;
      cur[u].next();
      if (!live) continue;
      int64_t b = 0, o = row;
      if (!one_batch) { b = row / outer; o = row - b * outer; }
      T* dst = out + b * so_batch + o * so_outer + c * 8;
      if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        if (sb[u] < 253u) {
          *reinterpret_cast<uint4*>(dst) = upcast8_bf16(w[u], sb[u]);
          continue;
        }
      }
      const float s = __uint_as_float(sb[u] << 23);
      const bool nan_scale = sb[u] == 0xFFu;
      T e[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) e[j] = dequant_one<T>((w[u] >> (4 * j)) & 0xFu, s, nan_scale);
      if constexpr (sizeof(T) == 2) {
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(e);
      } else {
        *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(e);
        *reinterpret_cast<float4*>(dst + 4) = *reinterpret_cast<const float4*>(e + 4);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) upcast_strided_kernel(const uint8_t* __restrict__ q,
                                                             const uint8_t* __restrict__ scale, T* __restrict__ out,
                                                             int64_t batch, int64_t outer, int64_t quant,
                                                             int64_t so_batch, int64_t so_outer, int64_t so_quant) {
  const int64_t groups = quant >> 5;
  const int64_t total = batch * outer * groups;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t o = i % outer;
    const int64_t t = i / outer;
    const int64_t g = t % groups;
    const int64_t b = t / groups;
    const int64_t row = b * outer + o;
    const uint4 raw = *reinterpret_cast<const uint4*>(q + row * (quant >> 1) + g * 16);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    const uint32_t sb = scale[row * groups + g];
    const float s = __uint_as_float(sb << 23);
    const bool nan_scale = sb == 0xFFu;
    T* dst = out + b * so_batch + o * so_outer + g * 32 * so_quant;
#pragma unroll
    for (int j = 0; j < 32; ++j) dst[j * so_quant] = dequant_one<T>((w[j >> 3] >> (4 * (j & 7))) & 0xFu, s, nan_scale);
  }
}

int grid_for(int64_t total, int threads) {
  int64_t blocks = cdiv64(total, threads);
  int64_t cap = (int64_t)moe_sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) int moe_downcast_mxfp4(const void* x, int src_dtype, int64_t batch, int64_t outer, int64_t quant,
                                  int64_t sx_batch, int64_t sx_outer, int64_t sx_quant, uint8_t* q, uint8_t* scale,
                                  int rounding_mode, void* stream) {
  MOE_CHECK_ARG(batch >= 0 && outer >= 0 && quant >= 0, "moe_downcast_mxfp4: negative extent");
  MOE_CHECK_ARG(quant % 32 == 0, "moe_downcast_mxfp4: quantised axis (%lld) must be a multiple of 32", (long long)quant);
  MOE_CHECK_ARG(rounding_mode == MOE_ROUND_UP || rounding_mode == MOE_ROUND_DOWN, "moe_downcast_mxfp4: bad rounding mode");
  if (batch * outer * quant == 0) return MOE_OK;
  MOE_CHECK_ARG(x && q && scale, "moe_downcast_mxfp4: NULL pointer");
  cudaStream_t st = (cudaStream_t)stream;
  MOE_DISPATCH_FLOAT(src_dtype, T, {
    const int64_t align = 16 / (int64_t)sizeof(T);
    const bool rows_ok = sx_quant == 1 && ((uintptr_t)x % 16 == 0) && (sx_outer % align == 0) &&
                         (sx_batch % align == 0) && ((uintptr_t)q % 4 == 0);
    const int64_t align2 = 2;                                         // two columns per thread: 4- or 8-byte loads
    const bool cols2_ok = sx_outer == 1 && sx_quant != 1 && outer % 2 == 0 && ((uintptr_t)x % (2 * sizeof(T)) == 0) &&
                          (sx_quant % align2 == 0) && (sx_batch % align2 == 0) && ((uintptr_t)q % 16 == 0);
    if (rows_ok && (uintptr_t)q % 16 == 0) {
      const int64_t total = batch * outer * (quant >> 5);
      if (total + (int64_t)GROUPS_UNROLL * 256 * moe_sm_count() * 16 < 2147483647LL)       // 32-bit row / group counters
        downcast_rows_kernel<T, int32_t><<<grid_for(total, GROUPS_UNROLL * 256), 256, 0, st>>>(
            (const T*)x, batch * outer, quant, outer, sx_batch, sx_outer, q, scale, rounding_mode);
      else
        downcast_rows_kernel<T, int64_t><<<grid_for(total, GROUPS_UNROLL * 256), 256, 0, st>>>(
            (const T*)x, batch * outer, quant, outer, sx_batch, sx_outer, q, scale, rounding_mode);
    } else if (cols2_ok) {
      const int64_t total = batch * (outer >> 1) * (quant >> 5);
      downcast_cols2_kernel<T><<<grid_for(total, 128), 128, 0, st>>>((const T*)x, batch, outer, quant, sx_batch, sx_quant, q,
                                                                     scale, rounding_mode);
    } else {
      MOE_CHECK_ARG((uintptr_t)q % 16 == 0, "moe_downcast_mxfp4: q must be 16-byte aligned");
      const int64_t total = batch * outer * (quant >> 5);
      downcast_strided_kernel<T><<<grid_for(total, 256), 256, 0, st>>>((const T*)x, batch, outer, quant, sx_batch,
                                                                       sx_outer, sx_quant, q, scale, rounding_mode);
    }
  });
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}

extern "C" __attribute__((visibility("default"))) int moe_upcast_mxfp4(const uint8_t* q, const uint8_t* scale, void* out, int dst_dtype, int64_t batch,
                                int64_t outer, int64_t quant, int64_t so_batch, int64_t so_outer, int64_t so_quant,
                                void* stream) {
  MOE_CHECK_ARG(batch >= 0 && outer >= 0 && quant >= 0, "moe_upcast_mxfp4: negative extent");
  MOE_CHECK_ARG(quant % 32 == 0, "moe_upcast_mxfp4: quantised axis (%lld) must be a multiple of 32", (long long)quant);
  if (batch * outer * quant == 0) return MOE_OK;
  MOE_CHECK_ARG(q && scale && out, "moe_upcast_mxfp4: NULL pointer");
  cudaStream_t st = (cudaStream_t)stream;
  MOE_DISPATCH_FLOAT(dst_dtype, T, {
    const int64_t align = 16 / (int64_t)sizeof(T);
    const bool rows_ok = so_quant == 1 && ((uintptr_t)out % 16 == 0) && (so_outer % align == 0) &&
                         (so_batch % align == 0) && ((uintptr_t)q % 4 == 0);
    if (rows_ok) {
      const int64_t total = batch * outer * (quant >> 3);
      upcast_rows_kernel<T><<<grid_for(total, ROWS_UNROLL * 256), 256, 0, st>>>(q, scale, (T*)out, batch * outer, quant, outer,
                                                                  so_batch, so_outer);
    } else {
      MOE_CHECK_ARG((uintptr_t)q % 16 == 0, "moe_upcast_mxfp4: q must be 16-byte aligned");
      const int64_t total = batch * outer * (quant >> 5);
      upcast_strided_kernel<T><<<grid_for(total, 256), 256, 0, st>>>(q, scale, (T*)out, batch, outer, quant, so_batch,
                                                                     so_outer, so_quant);
    }
  });
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}
