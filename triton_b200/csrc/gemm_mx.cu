// Ragged grouped GEMM on the block-scaled tensor-core path of sm_100a:
//   tcgen05.mma.kind::mxf8f6f4.block_scale -- e2m1 weights with their e8m0 scales go into the MMA as they are
//   stored (no software dequantisation), activations are e4m3 with e8m0 scales per 32 k.
//
// What the reference reaches through `PrecisionConfig(a_mx_scale=..., b_mx_scale=...)` and fp8 activations
// (triton_kernels matmul.py:130-132, 311-336; matmul_details/_p_matmul.py:399-407): its MXFP4 weights feed
// tl.dot_scaled, which lowers to this instruction kind.
//
// Operand roles are swapped with respect to the bf16 kernel: the WEIGHTS are the M = 128 operand (a tile is 128
// weight rows x 128 k) and the TOKENS are the N operand (16 .. 128 columns), so that a handful of tokens costs a
// handful of accumulator columns.  A CTA tile is MB (1 or 3) weight blocks x one block of tokens; the token block
// stays in shared memory per k step and is shared by the MB weight blocks.
//
// bf16 activations are split into two e4m3 terms, hi = mxfp8(x) and lo = mxfp8(x - hi), each with its own e8m0
// scale per 32 k (error about 2^-8 of the group maximum, inside the tolerance of the bf16 path).  Both terms sit
// side by side as N columns of ONE MMA ([hi tokens | lo tokens], every column has its own scale), the epilogue adds the
// two accumulator columns of a token.  e4m3 / MXFP8 activations enter as they are (one term).
//
// With at most 16 token rows per block (decode) bf16 activations take a second form: FOUR e2m1 terms, each the MXFP4
// quantisation of what the terms before it left over (about 2^-14 of the group maximum after four), and the MMA is
//   tcgen05.mma.kind::mxf4.block_scale.scale_vec::2X -- K = 64 per instruction and both operands packed, so a
// weight tile stays 8 KB in shared memory (plain TMA copy, 64-byte swizzle) instead of the 16 KB of the byte-per-
// element form, and a k step costs half the MMA instructions.  Twice the bytes in flight per SM and half the
// instruction count are what a weight-streaming step is short of; the four terms are four groups of N columns.
//
// Data flow of one k step (128 k):
//   weights     one TMA tensor copy: MB x (128 rows x 64 packed bytes) from the tile-contiguous layout of
//               moe_weight_layout_to_b200mx, unpacked by the TMA unit (CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B) into the
//               byte-per-element, 128-byte-swizzled operand the MMA reads;
//   w scales    one bulk copy of MB x 512 B, already in the [32 lanes][4 quarters][4 k groups] order;
//   tokens      one bulk copy of a chunk the pack kernel below prepared per (token block, k step): the e4m3 rows in
//               the swizzled operand layout followed by their 512 B of scales;
//   scales -> tensor memory through registers (tcgen05.st by four loader warps), then MB x 4 MMAs of K = 32.
// Warps: 0 producer (one thread), 1 MMA issue + tensor-memory owner, 2-5 epilogue, 6-9 scale loaders.  Every mbarrier
// wait is bounded.
#include "gemm_tc_common.cuh"
#include <cuda_fp8.h>
#include <utility>

// e4m3 output (the next GEMM's activations): round to nearest, saturating at +-448 like the MMA's own conversions
template <> __device__ __forceinline__ __nv_fp8_e4m3 from_f32<__nv_fp8_e4m3>(float v) {
  __nv_fp8_e4m3 r;
  r.__x = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
  return r;
}

namespace {

constexpr int MX_THREADS = 320;               // warp 0 producer, 1 MMA, 2-5 epilogue, 6-9 scale loaders
constexpr int MX_MAX_STAGES = 8;
constexpr int MX_W_TILE = 128 * 128;           // one weight block of a stage in shared memory (byte per element)
constexpr int MX_W_TILE_TX = 128 * 64;         // what its copy reports to the mbarrier: the packed bytes read; also the
                                               // size of a weight block that stays packed (four-term form)
constexpr int MX_WS_TILE = 512;                // its scales
constexpr int MX_SF_COLS = 16;                 // tensor-memory columns of scales per stage (MB x 4 + 4)
constexpr int MX_SF_BASE = 512 - MX_MAX_STAGES * MX_SF_COLS;    // 384: accumulators live below
constexpr int MX_SMEM_LIMIT = 227 * 1024;
constexpr int MX_CTL_BARS = 3 * MX_MAX_STAGES + 5;          // full, empty, scales-ready rings; 2 + 2 accumulator; drain
constexpr int MX_CTL_BYTES = MX_CTL_BARS * 8 + 16;          // + tensor-memory base, abort flag

struct MxParams {
  const uint8_t* xq;            // packed token chunks: [slot][k step][n_mma rows x 128 B | 1024 B scale area]
  int64_t chunk_bytes;
  int n_mma;                    // MMA N: token columns (hi and lo when split)
  int tb;                       // token rows per block (16, 32, 64 or 128)
  int split;                    // terms of a token: 1, 2 (bf16 as hi + lo e4m3) or 4 (bf16 as e2m1 terms); term t of
                                // token j is column t * tb + j
  int KT, NB;                   // 128-k steps, 128-row weight blocks
  int stages, stage_bytes;
  int acc_bufs;
  int n_groups;                 // ceil(NB / MB)
  int64_t grid_m;               // static bound on token blocks (dense problems: exact)
};

struct MxMaps {
  CUtensorMap m[3];             // boxes of 1, 2 and 3 weight blocks
};

// The tiles of one CTA, in the order every role walks them.  A tile is one token block x up to MB consecutive weight
// blocks; tile = (weight group, token block) with token blocks varying fastest, dealt out round robin, so that CTAs
// running at the same time share a weight group (large problems: the group is read from HBM once).  (Equal contiguous
// ranges of weight blocks per CTA, which leave no partly filled last wave, were measured 5-12 % slower at 16 and 64
// tokens: they cut more tiles short of MB blocks, and a k step costs about the same whatever it carries.  Slices of K per
// tile with fp32 partial sums in global memory -- red.global.add, the slice that arrives last runs the epilogue -- were
// correct and 20-35 % slower at 4 to 64 tokens: 48 scalar reductions per thread and slice, their fence and the counter
// round trip take longer than a slice of a few k steps, and the epilogue warps become the bottleneck.)
struct MxSched {
  int64_t useful_m, cur, end;
  int NB, MB;
  __device__ __forceinline__ MxSched(int64_t useful_m_, int NB_, int NG, int MB_)
      : useful_m(useful_m_), cur(blockIdx.x), end(useful_m_ * NG), NB(NB_), MB(MB_) {}
  __device__ __forceinline__ bool next(int64_t& pid_m, int& nb0, int& mb_live) {
    if (cur >= end) return false;
    pid_m = cur % useful_m;
    nb0 = (int)(cur / useful_m) * MB;
    mb_live = min(MB, NB - nb0);
    cur += gridDim.x;
    return true;
  }
};

// ---- token block -> (expert, first row, rows) through the block schedule of the block size in use -----------
__device__ __forceinline__ bool mx_map_block(const GemmParams& p, int tb, int64_t pid_m, int& e, int64_t& row0, int& rows) {
  if (p.slice_sizes == nullptr) {
    e = 0;
    row0 = pid_m * tb;
    if (row0 >= p.M) return false;
    rows = (int)min((int64_t)tb, p.M - row0);
    return true;
  }
  const uint32_t ent = (uint32_t)p.block_sched[pid_m];
  if (ent == 0xFFFFFFFFu) return false;
  e = (int)(ent & 0xFFFFu);
  const int blk = (int)(ent >> 16);
  row0 = (int64_t)p.slice_offs[e] + (int64_t)blk * tb;
  rows = min(tb, p.slice_sizes[e] - blk * tb);
  return rows > 0;
}

// ---- programmatic dependent launch ---------------------------------------------------------------------------
// The pack kernel and the GEMM are launched with the programmatic-stream-serialization attribute: the next kernel of the
// stream may start while this one still runs, and whatever it reads from a predecessor comes after its own
// griddepcontrol.wait, which returns once the predecessors have completed and their writes are visible.  A decode step is
// short launches back to back; this way a kernel's launch and prologue overlap the tail of its predecessor.  (Inside a
// replayed CUDA graph the gain is within the noise: launches are back to back there anyway.  Requesting the first weight
// tiles ahead of the wait changed nothing either.)
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ============================================================================================================
// Pack kernel: token rows -> per (token block, k step) chunks in the operand layout of the MMA.
//   row r of the chunk (r < n_mma) is 128 bytes = 128 e4m3 values of k = 128 kt .. +127, its 16-byte pieces XOR-
//   swizzled with (r & 7) like a 128-byte-swizzled TMA tile; the scale of (row r, group g) is byte
//   (r % 32) * 16 + (r / 32) * 4 + g of the 512 bytes that follow the rows.
// grid = (token blocks, k steps); a warp takes a row at a time, a lane 4 consecutive k.
// ============================================================================================================
struct PackParams {
  const void* x; int64_t ld_x; int64_t rows_x;        // source rows; ld in elements
  const uint8_t* x_scale; int64_t ld_xs;              // e8m0 [rows_x, K / 32] for MXFP8 sources, else NULL
  const int32_t* gather;
  int K, KT, tb, n_mma;
  int64_t chunk_bytes;
  uint8_t* out;
};

__device__ __forceinline__ uint32_t f32x2_to_e4m3x2(float lo, float hi) {       // low byte <- lo, high byte <- hi
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float2 e4m3x2_to_f32x2(uint32_t v) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((uint16_t)v));
  return __half22float2(*reinterpret_cast<__half2*>(&h2));
}
// e8m0 byte s with 2^(s-127) >= amax / 448 (smallest such power of two), and the exact factors 2^(s-127), 2^(127-s)
__device__ __forceinline__ void mx8_scale(float amax, uint32_t& sb, float& scale, float& inv) {
  const float ds = amax * (1.0f / 448.0f);
  uint32_t u = (__float_as_uint(ds) + 0x007FFFFFu) & 0x7F800000u;
  sb = u >> 23;
  if (amax == 0.0f) sb = 127u;
  sb = min(max(sb, 1u), 253u);
  scale = __uint_as_float(sb << 23);
  inv = __uint_as_float((254u - sb) << 23);
}

template <bool SPLIT>
__global__ void __launch_bounds__(256) mx_pack_x_kernel(const GemmParams p, const PackParams a) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t slot = blockIdx.x;
  const int kt = blockIdx.y;
  int e; int64_t row0; int rows;
  if (!mx_map_block(p, a.tb, slot, e, row0, rows)) return;
  uint8_t* chunk = a.out + (slot * a.KT + kt) * a.chunk_bytes;
  uint8_t* sc = chunk + (int64_t)a.n_mma * 128;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k = kt * 128 + lane * 4;
  const int g = lane >> 3;
  const uint32_t piece = (uint32_t)(lane >> 2), within = (uint32_t)(lane & 3) * 4u;
  for (int r = warp; r < rows; r += 8) {
    const int64_t m = row0 + r;
    int64_t src = a.gather ? (int64_t)a.gather[m] : m;
    if (src >= a.rows_x) src = -1;
    const bool live = src >= 0 && k < a.K;        // K % 32 == 0: a lane's four values are in or out together
    if constexpr (SPLIT) {
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (live) {
        const uint2 raw = *reinterpret_cast<const uint2*>((const __nv_bfloat16*)a.x + src * a.ld_x + k);
        v[0] = __uint_as_float(raw.x << 16); v[1] = __uint_as_float(raw.x & 0xFFFF0000u);
        v[2] = __uint_as_float(raw.y << 16); v[3] = __uint_as_float(raw.y & 0xFFFF0000u);
      }
      float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
      for (int o = 1; o <= 4; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
      if (!(amax < 3.0e38f)) amax = 3.0e38f;      // Inf / NaN in the group: keep the scale finite
      uint32_t sb_hi; float s_hi, i_hi;
      mx8_scale(amax, sb_hi, s_hi, i_hi);
      const uint32_t h01 = f32x2_to_e4m3x2(v[0] * i_hi, v[1] * i_hi), h23 = f32x2_to_e4m3x2(v[2] * i_hi, v[3] * i_hi);
      const float2 f01 = e4m3x2_to_f32x2(h01), f23 = e4m3x2_to_f32x2(h23);
      float rs[4] = {v[0] - f01.x * s_hi, v[1] - f01.y * s_hi, v[2] - f23.x * s_hi, v[3] - f23.y * s_hi};
      float rmax = fmaxf(fmaxf(fabsf(rs[0]), fabsf(rs[1])), fmaxf(fabsf(rs[2]), fabsf(rs[3])));
#pragma unroll
      for (int o = 1; o <= 4; o <<= 1) rmax = fmaxf(rmax, __shfl_xor_sync(0xFFFFFFFFu, rmax, o));
      if (!(rmax < 3.0e38f)) rmax = 0.0f;
      uint32_t sb_lo; float s_lo, i_lo;
      mx8_scale(rmax, sb_lo, s_lo, i_lo);
      const uint32_t l01 = f32x2_to_e4m3x2(rs[0] * i_lo, rs[1] * i_lo), l23 = f32x2_to_e4m3x2(rs[2] * i_lo, rs[3] * i_lo);
      const int r_lo = a.tb + r;
      *reinterpret_cast<uint32_t*>(chunk + r * 128 + ((piece ^ (uint32_t)(r & 7)) << 4) + within) = h01 | (h23 << 16);
      *reinterpret_cast<uint32_t*>(chunk + r_lo * 128 + ((piece ^ (uint32_t)(r_lo & 7)) << 4) + within) = l01 | (l23 << 16);
      if ((lane & 7) == 0) {
        sc[(r & 31) * 16 + (r >> 5) * 4 + g] = (uint8_t)sb_hi;
        sc[(r_lo & 31) * 16 + (r_lo >> 5) * 4 + g] = (uint8_t)sb_lo;
      }
    } else {
      uint32_t w = 0;
      if (live) w = *reinterpret_cast<const uint32_t*>((const uint8_t*)a.x + src * a.ld_x + k);
      *reinterpret_cast<uint32_t*>(chunk + r * 128 + ((piece ^ (uint32_t)(r & 7)) << 4) + within) = w;
      if ((lane & 7) == 0) {
        uint8_t s = 127;
        if (live && a.x_scale) s = a.x_scale[src * a.ld_xs + (k >> 5)];
        sc[(r & 31) * 16 + (r >> 5) * 4 + g] = s;
      }
    }
  }
}

// ---- four e2m1 terms -----------------------------------------------------------------------------------------
// Chunk of the four-term form: row r (r < 4 tb; term t of token j is row t * tb + j) is 64 bytes = 128 e2m1 values, low
// nibble first, its 16-byte pieces XOR-swizzled with ((r >> 1) & 3) like a 64-byte-swizzled TMA tile; scales as above.
__device__ __forceinline__ uint32_t f32_to_e2m1(float q) {           // round to nearest, ties to the even code; |q| <= 6
  const float a = fabsf(q);
  const uint32_t c = (uint32_t)(a > 0.25f) + (uint32_t)(a >= 0.75f) + (uint32_t)(a > 1.25f) + (uint32_t)(a >= 1.75f) +
                     (uint32_t)(a > 2.5f) + (uint32_t)(a >= 3.5f) + (uint32_t)(a > 5.0f);
  return c | ((__float_as_uint(q) >> 28) & 8u);
}
__device__ __forceinline__ float e2m1_to_f32(uint32_t c) {
  const uint32_t m = c & 7u;
  // 0, 0.5 | (1 + 0.5 (m & 1)) * 2^((m >> 1) - 1)
  float v = m < 2u ? 0.5f * (float)m : __uint_as_float(((126u + (m >> 1)) << 23) | ((m & 1u) << 22));
  return (c & 8u) ? -v : v;
}
// e8m0 byte s with 2^(s-127) >= amax / 6, and the exact factors 2^(s-127), 2^(127-s)
__device__ __forceinline__ void mx4_scale(float amax, uint32_t& sb, float& scale, float& inv) {
  // amax / 6 rounded UP to a power of two; the product with a constant just above 1/6 is never below the quotient, so
  // every value of the group still fits (it doubles the scale where amax is within an ulp of 6 * 2^e, which costs nothing
  // that matters here) and the division is off the chain
  const float ds = amax * 0.16666668f;
  uint32_t u = (__float_as_uint(ds) + 0x007FFFFFu) & 0x7F800000u;
  sb = u >> 23;
  if (amax == 0.0f) sb = 127u;
  sb = min(max(sb, 1u), 253u);
  scale = __uint_as_float(sb << 23);
  inv = __uint_as_float((254u - sb) << 23);
}

// (A warp per (token block, k step, four rows) with the rows' chains side by side, and dead warps grouped into whole
// CTAs, was tried in place of the loop over rows below: 2.3 x slower.  A row's four-term chain is latency, and four of
// them in one warp add up where eight warps of a CTA overlap them.)
__global__ void __launch_bounds__(256) mx_pack_x4_kernel(const GemmParams p, const PackParams a) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t slot = blockIdx.x;
  const int kt = blockIdx.y;
  int e; int64_t row0; int rows;
  if (!mx_map_block(p, a.tb, slot, e, row0, rows)) return;
  uint8_t* chunk = a.out + (slot * a.KT + kt) * a.chunk_bytes;
  uint8_t* sc = chunk + (int64_t)a.n_mma * 64;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k = kt * 128 + lane * 4;
  const uint32_t g = (uint32_t)(lane >> 3), within = (uint32_t)(lane & 7) * 2u;     // a 32-group is one 16-byte piece
  for (int r = warp; r < rows; r += 8) {
    const int64_t m = row0 + r;
    int64_t src = a.gather ? (int64_t)a.gather[m] : m;
    if (src >= a.rows_x) src = -1;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (src >= 0 && k < a.K) {
      const uint2 raw = *reinterpret_cast<const uint2*>((const __nv_bfloat16*)a.x + src * a.ld_x + k);
      v[0] = __uint_as_float(raw.x << 16); v[1] = __uint_as_float(raw.x & 0xFFFF0000u);
      v[2] = __uint_as_float(raw.y << 16); v[3] = __uint_as_float(raw.y & 0xFFFF0000u);
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      // maximum of the 32-group: the 8 lanes that hold it reduce the bit patterns of their |values| (non-negative floats
      // order like unsigned integers; NaN patterns rank above Inf and are caught below)
      float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
      amax = __uint_as_float(__reduce_max_sync(0xFFu << (lane & 24), __float_as_uint(amax)));
      if (!(amax < 3.0e38f)) amax = t == 0 ? 3.0e38f : 0.0f;       // Inf / NaN in the group: keep the scales finite
      uint32_t sb; float s, inv;
      mx4_scale(amax, sb, s, inv);
      uint32_t codes = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t c = f32_to_e2m1(v[i] * inv);
        codes |= c << (4 * i);
        v[i] -= e2m1_to_f32(c) * s;
      }
      const int rt = t * a.tb + r;
      *reinterpret_cast<uint16_t*>(chunk + rt * 64 + ((g ^ (uint32_t)((rt >> 1) & 3)) << 4) + within) = (uint16_t)codes;
      if ((lane & 7) == 0) sc[(rt & 31) * 16 + (rt >> 5) * 4 + (int)g] = (uint8_t)sb;
    }
  }
}

// ============================================================================================================
// PTX pieces of the block-scaled path
// ============================================================================================================
// 3-D tile copy: box (128 elements, 128 rows, MB tiles) of the weight tensor map, starting at tile `z`
__device__ __forceinline__ void tma_tile_3d(uint32_t dst, const CUtensorMap* tmap, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
      "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}
// instruction descriptor of kind::mxf8f6f4: A = e2m1 (code 5), B = e4m3 (code 0), both K-major, e8m0 scales,
// M = 128, N = n; sf selects the byte (k group) of the scale words for A and B
__device__ __forceinline__ uint32_t mx_idesc(int n, uint32_t sf) {
  return (sf << 4) | (5u << 7) | (0u << 10) | ((uint32_t)(n >> 3) << 17) | (1u << 23) | (1u << 27) | (sf << 29);
}
// kind::mxf4: A and B e2m1 (code 1), packed, K-major, K = 64; sf selects the byte PAIR (0 or 2) of the scale words
__device__ __forceinline__ uint32_t mx4_idesc(int n, uint32_t sf) {
  return (sf << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | (1u << 23) | (1u << 27) | (sf << 29);
}
// shared-memory descriptor of a K-major operand with 64-byte rows and 64-byte swizzle (8-row groups 512 B apart)
__device__ __forceinline__ uint64_t make_desc_sw64(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(512 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)4 << 61;
  return d;
}
__device__ __forceinline__ void mma_mxf4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%4], [%5], p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_mxf8f6f4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                             uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
      : "memory");
}

// ============================================================================================================
// The GEMM kernel
// ============================================================================================================
// F4: the four-term form (packed operands, kind::mxf4); otherwise byte-per-element operands, kind::mxf8f6f4
// KM (four-term form, MB = 3): the three weight tiles of a stage are three consecutive K STEPS of ONE weight block instead of
// one k step of three blocks -- for steps with so few tiles that a CTA gets single weight blocks (one to four tokens: 60
// to 165 three-block tiles for 148 SMs).  A stage of one 8 KB tile cannot keep a per-SM copy pipeline busy (a ring of
// 8 KB stages streams 3.3 TB/s over the GPU however many are in flight, 24 KB stages 7.1 TB/s).
template <typename TY, int MB, bool F4, bool KM = false>
__global__ void __launch_bounds__(MX_THREADS, 1)
gemm_mx_kernel(const GemmParams p, const MxParams q, const __grid_constant__ MxMaps w_maps) {
  static_assert(!KM || (F4 && MB == 3), "the k-step form is built for the four-term kernel with three tiles per stage");
  constexpr uint32_t W_TILE = F4 ? MX_W_TILE_TX : MX_W_TILE;       // bytes of a weight block in shared memory
  constexpr uint32_t X_ROW = F4 ? 64u : 128u;                      // bytes of a token row of a k step
  constexpr int NACC = KM ? 1 : MB;                                // accumulators (weight blocks) of a tile
  constexpr int SF_COLS = KM ? 24 : MX_SF_COLS;                    // scale columns of a stage: KM has three token chunks
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int STAGES = q.stages;
  // per stage: [MB weight tiles][token rows + 1024 B scale area (KM: three such chunks)][MB x 512 B weight scales]
  const uint32_t OFF_X = MB * W_TILE;
  const uint32_t OFF_XS = OFF_X + (uint32_t)q.n_mma * X_ROW;
  const uint32_t OFF_WS = KM ? OFF_X + 3u * (uint32_t)q.chunk_bytes : OFF_XS + 1024u;
  const uint32_t SF_BASE = KM ? 512u - (uint32_t)(MX_MAX_STAGES > 5 ? 5 : MX_MAX_STAGES) * 24u : (uint32_t)MX_SF_BASE;
  const uint32_t ctl0 = sbase + (uint32_t)STAGES * (uint32_t)q.stage_bytes;
  auto BAR_FULL = [&](int s) { return ctl0 + 8u * (uint32_t)s; };
  auto BAR_EMPTY = [&](int s) { return ctl0 + 8u * (uint32_t)(MX_MAX_STAGES + s); };
  auto BAR_SF = [&](int s) { return ctl0 + 8u * (uint32_t)(2 * MX_MAX_STAGES + s); };      // scales are in tensor memory
  auto BAR_ACC_FULL = [&](int a) { return ctl0 + 8u * (uint32_t)(3 * MX_MAX_STAGES + a); };
  auto BAR_ACC_EMPTY = [&](int a) { return ctl0 + 8u * (uint32_t)(3 * MX_MAX_STAGES + 2 + a); };
  const uint32_t BAR_DRAIN = ctl0 + 8u * (uint32_t)(3 * MX_MAX_STAGES + 4);
  uint8_t* ctl_ptr = smem + (size_t)STAGES * (size_t)q.stage_bytes;
  volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(ctl_ptr + MX_CTL_BARS * 8);
  volatile int* s_abort = reinterpret_cast<volatile int*>(ctl_ptr + MX_CTL_BARS * 8 + 4);
  Ctl ctl{s_abort, p.status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < MX_MAX_STAGES; ++s) {
      mbar_init(BAR_FULL(s), 1);
      mbar_init(BAR_EMPTY(s), 1);
      mbar_init(BAR_SF(s), 4);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(BAR_ACC_FULL(a), 1);
      mbar_init(BAR_ACC_EMPTY(a), 4);
    }
    mbar_init(BAR_DRAIN, 1);
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)s_tmem)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;
  pdl_launch_dependents();
  pdl_wait();

  const int KT = q.KT, NB = q.NB, NG = q.n_groups;
  int64_t useful_m = q.grid_m;
  if (p.slice_sizes) useful_m = (int64_t)p.block_offs[p.E];
  const int acc_stride = NACC * q.n_mma;            // accumulator columns of one buffer
  MxSched sched(useful_m, NB, NG, NACC);
  const int KS = KM ? (KT + 2) / 3 : KT;            // stages of a tile
  int64_t pid_m;
  int nb0, mb_live;

  if (warp == 0) {
    // ================================= producer =======================================================
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      while (ok && sched.next(pid_m, nb0, mb_live)) {
        int e; int64_t row0; int rows;
        mx_map_block(p, q.tb, pid_m, e, row0, rows);
        const uint8_t* xsrc = q.xq + pid_m * KT * q.chunk_bytes;
        const CUtensorMap* w_map = &w_maps.m[mb_live - 1];
        for (int kt = 0; kt < KS; ++kt, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(BAR_EMPTY(s), ((it / STAGES) & 1u) ^ 1u, ctl, 601);
          if (!ok) break;
          const uint32_t st = sbase + (uint32_t)s * (uint32_t)q.stage_bytes;
          if constexpr (KM) {
            const int k_live = min(3, KT - 3 * kt);
            mbar_expect_tx(BAR_FULL(s), (uint32_t)k_live * ((uint32_t)(MX_W_TILE_TX + MX_WS_TILE) + (uint32_t)q.chunk_bytes));
            for (int i = 0; i < k_live; ++i) {
              const int64_t tile = ((int64_t)e * KT + 3 * kt + i) * NB + nb0;
              tma_tile_3d(st + (uint32_t)i * W_TILE, &w_maps.m[0], 0, 0, (int)tile, BAR_FULL(s));
              bulk_g2s(st + OFF_WS + (uint32_t)i * MX_WS_TILE, p.w_scale + tile * MX_WS_TILE, (uint32_t)MX_WS_TILE, BAR_FULL(s));
            }
            bulk_g2s(st + OFF_X, xsrc + (int64_t)(3 * kt) * q.chunk_bytes, (uint32_t)k_live * (uint32_t)q.chunk_bytes, BAR_FULL(s));
          } else {
            const int64_t tile = ((int64_t)e * KT + kt) * NB + nb0;
            mbar_expect_tx(BAR_FULL(s), (uint32_t)(mb_live * (MX_W_TILE_TX + MX_WS_TILE)) + (uint32_t)q.chunk_bytes);
            tma_tile_3d(st, w_map, 0, 0, (int)tile, BAR_FULL(s));
            bulk_g2s(st + OFF_WS, p.w_scale + tile * MX_WS_TILE, (uint32_t)(mb_live * MX_WS_TILE), BAR_FULL(s));
            bulk_g2s(st + OFF_X, xsrc + (int64_t)kt * q.chunk_bytes, (uint32_t)q.chunk_bytes, BAR_FULL(s));
          }
        }
      }
      if (!ok) {
        // aborting: let the copies that were already issued land before the CTA leaves
        const uint32_t lo = it > (uint32_t)STAGES ? it - STAGES : 0;
        for (uint32_t j = lo; j < it; ++j)
          for (uint32_t i = 0; i < (1u << 16) && !mbar_test(BAR_FULL(j % STAGES), (j / STAGES) & 1u); ++i) __nanosleep(64);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ================================= MMA issuer =====================================================
    if (lane == 0) {
      uint32_t it = 0, tc = 0;
      bool ok = true;
      for (; ok && sched.next(pid_m, nb0, mb_live); ++tc) {
        const uint32_t ab = tc % (uint32_t)q.acc_bufs;
        ok = mbar_wait(BAR_ACC_EMPTY(ab), ((tc / (uint32_t)q.acc_bufs) & 1u) ^ 1u, ctl, 603);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + ab * (uint32_t)acc_stride;
        for (int kt = 0; kt < KS; ++kt, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(BAR_FULL(s), (it / STAGES) & 1u, ctl, 602);
          ok = ok && mbar_wait(BAR_SF(s), (it / STAGES) & 1u, ctl, 606);
          if (!ok) break;
          tc_fence_after();
          const uint32_t st = sbase + (uint32_t)s * (uint32_t)q.stage_bytes;
          const uint32_t sf = tmem_base + SF_BASE + (uint32_t)(s * SF_COLS);
          // k group outermost: consecutive MMAs go to different accumulators
          if constexpr (KM) {
            const int k_live = min(3, KT - 3 * kt);
#pragma unroll
            for (int i = 0; i < 3; ++i) {
              if (i < k_live) {
                const uint64_t adesc = make_desc_sw64(st + (uint32_t)i * W_TILE);
                const uint64_t bdesc = make_desc_sw64(st + OFF_X + (uint32_t)i * (uint32_t)q.chunk_bytes);
#pragma unroll
                for (int kk = 0; kk < 2; ++kk)
                  mma_mxf4(d_tmem, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), mx4_idesc(q.n_mma, (uint32_t)(kk * 2)),
                           sf + 4u * (uint32_t)i, sf + 12u + 4u * (uint32_t)i, (kt | i | kk) ? 1u : 0u);
              }
            }
          } else if constexpr (F4) {
            const uint64_t bdesc = make_desc_sw64(st + OFF_X);
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
              for (int mb = 0; mb < MB; ++mb) {
                if (mb < mb_live)
                  mma_mxf4(d_tmem + (uint32_t)(mb * q.n_mma), make_desc_sw64(st + (uint32_t)mb * W_TILE) + (uint64_t)(kk * 2),
                           bdesc + (uint64_t)(kk * 2), mx4_idesc(q.n_mma, (uint32_t)(kk * 2)), sf + 4u * (uint32_t)mb, sf + 4u * MB,
                           (kt | kk) ? 1u : 0u);
              }
            }
          } else {
            const uint64_t bdesc = make_desc(st + OFF_X);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
              for (int mb = 0; mb < MB; ++mb) {
                if (mb < mb_live)
                  mma_mxf8f6f4(d_tmem + (uint32_t)(mb * q.n_mma), make_desc(st + (uint32_t)mb * W_TILE) + (uint64_t)(kk * 2),
                               bdesc + (uint64_t)(kk * 2), mx_idesc(q.n_mma, (uint32_t)kk), sf + 4u * (uint32_t)mb, sf + 4u * MB,
                               (kt | kk) ? 1u : 0u);
              }
            }
          }
          mma_commit(BAR_EMPTY(s));
        }
        if (ok) mma_commit(BAR_ACC_FULL(ab));
      }
      // every MMA issued by this thread has retired before tensor memory is freed
      mma_commit(BAR_DRAIN);
      mbar_wait(BAR_DRAIN, 0, ctl, 605);
    }
    __syncwarp();
  } else if (warp >= 6) {
    // ================================= scale loaders ==================================================
    // The scales of a stage go from shared to tensor memory through registers (tcgen05.st), one warp per lane quarter:
    // lane l of every quarter holds the 16 bytes of row l of each 512-byte scale block (the MB weight blocks, then the
    // tokens), i.e. the four columns the MMA reads for rows l, l + 32, l + 64, l + 96.  This keeps the copies out of
    // the in-order queue of the tensor pipe, where a tcgen05.cp ahead of every k step cost about a third of the step.
    const int qd = warp & 3;
    uint32_t it = 0;
    bool ok = true;
    while (ok && sched.next(pid_m, nb0, mb_live)) {
      for (int kt = 0; kt < KS; ++kt, ++it) {
        const int s = it % STAGES;
        ok = __all_sync(0xFFFFFFFFu, mbar_wait(BAR_FULL(s), (it / STAGES) & 1u, ctl, 607));
        if (!ok) break;
        const uint32_t st = sbase + (uint32_t)s * (uint32_t)q.stage_bytes;
        const uint32_t taddr = tmem_base + ((uint32_t)(qd * 32) << 16) + SF_BASE + (uint32_t)(s * SF_COLS);
        if constexpr (KM) {
          // columns 0..11: the weight scales of the three k steps, 12..23: the token scales of the three chunks
          const int k_live = min(3, KT - 3 * kt);
          uint4 w[3], x[3];
#pragma unroll
          for (int i = 0; i < 3; ++i) {
            w[i] = i < k_live ? lds128(st + OFF_WS + (uint32_t)i * MX_WS_TILE + (uint32_t)lane * 16u) : make_uint4(0, 0, 0, 0);
            x[i] = i < k_live ? lds128(st + OFF_X + (uint32_t)i * (uint32_t)q.chunk_bytes + (uint32_t)q.n_mma * X_ROW + (uint32_t)lane * 16u)
                              : make_uint4(0, 0, 0, 0);
          }
          asm volatile(
              "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
              "r"(w[0].x), "r"(w[0].y), "r"(w[0].z), "r"(w[0].w), "r"(w[1].x), "r"(w[1].y), "r"(w[1].z), "r"(w[1].w),
              "r"(w[2].x), "r"(w[2].y), "r"(w[2].z), "r"(w[2].w), "r"(x[0].x), "r"(x[0].y), "r"(x[0].z), "r"(x[0].w)
              : "memory");
          asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr + 16u), "r"(x[1].x),
                       "r"(x[1].y), "r"(x[1].z), "r"(x[1].w), "r"(x[2].x), "r"(x[2].y), "r"(x[2].z), "r"(x[2].w)
                       : "memory");
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(BAR_SF(s));
          continue;
        }
        uint4 v[MB + 1];
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
          v[mb] = mb < mb_live ? lds128(st + OFF_WS + (uint32_t)mb * MX_WS_TILE + (uint32_t)lane * 16u) : make_uint4(0, 0, 0, 0);
        v[MB] = lds128(st + OFF_XS + (uint32_t)lane * 16u);
        if constexpr (MB == 3) {
          asm volatile(
              "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
              "r"(v[0].x), "r"(v[0].y), "r"(v[0].z), "r"(v[0].w), "r"(v[1].x), "r"(v[1].y), "r"(v[1].z), "r"(v[1].w),
              "r"(v[2].x), "r"(v[2].y), "r"(v[2].z), "r"(v[2].w), "r"(v[3].x), "r"(v[3].y), "r"(v[3].z), "r"(v[3].w)
              : "memory");
        } else {
          asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(v[0].x),
                       "r"(v[0].y), "r"(v[0].z), "r"(v[0].w), "r"(v[1].x), "r"(v[1].y), "r"(v[1].z), "r"(v[1].w)
                       : "memory");
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(BAR_SF(s));
      }
    }
  } else {
    // ================================= epilogue =======================================================
    // Accumulator [weight row = lane][token = column]: lane l of the warp that owns lane quarter qd holds output
    // column n = n0 + 128 mb + 32 qd + l.  Token parameters sit one token per lane and are broadcast by shuffle; for
    // SwiGLU the even lane holds the gate and the odd lane the linear half of a pair.
    const int qd = warp & 3;
    const bool swiglu = p.activation == MOE_ACT_SWIGLU;
    uint32_t tc = 0;
    bool ok = true;
    for (; ok && sched.next(pid_m, nb0, mb_live); ++tc) {
      int e; int64_t row0; int rows;
      mx_map_block(p, q.tb, pid_m, e, row0, rows);
      const uint32_t ab = tc % (uint32_t)q.acc_bufs;
      float bias_n[NACC];
#pragma unroll
      for (int mb = 0; mb < NACC; ++mb) {
        const int n = (nb0 + mb) * 128 + qd * 32 + lane;
        bias_n[mb] = (p.bias && n < p.N) ? load_bias(p.bias, p.bias_dtype, (int64_t)e * p.ld_bias + n) : 0.0f;
      }
      ok = __all_sync(0xFFFFFFFFu, mbar_wait(BAR_ACC_FULL(ab), (tc / (uint32_t)q.acc_bufs) & 1u, ctl, 604));
      if (!ok) break;
      tc_fence_after();
      for (int c0 = 0; c0 < rows; c0 += 16) {
        // parameters of token c0 + lane (lanes 0..15)
        const int tj = c0 + (lane & 15);
        TY* dst_l = nullptr;
        float beta_l = 1.0f, gamma_l = 1.0f;
        if (tj < rows) {
          const int64_t m = row0 + tj;
          const int64_t d = p.scatter_indx ? (int64_t)p.scatter_indx[m] : m;
          if (d >= 0) dst_l = gemm_out_row<TY>(p, d);
          if (p.betas) beta_l = p.betas[m];
          if (p.gammas) gamma_l = p.gammas[m];
        }
        const int jmax = min(16, rows - c0);
#pragma unroll
        for (int mb = 0; mb < NACC; ++mb) {
          if (mb < mb_live) {
            const int n = (nb0 + mb) * 128 + qd * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(qd * 32) << 16) + ab * (uint32_t)acc_stride +
                                   (uint32_t)(mb * q.n_mma + c0);
            uint32_t hi[16], lo[16];
            tmem_ld16(taddr, hi);
            if (q.split > 1) tmem_ld16(taddr + (uint32_t)q.tb, lo);
            tmem_ld_wait();
            if constexpr (F4) {                                   // terms 2 and 3
              uint32_t t2[16], t3[16];
              tmem_ld16(taddr + 2u * (uint32_t)q.tb, t2);
              tmem_ld16(taddr + 3u * (uint32_t)q.tb, t3);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                hi[j] = __float_as_uint(__uint_as_float(hi[j]) + __uint_as_float(t3[j]));      // smallest terms first
                lo[j] = __float_as_uint(__uint_as_float(lo[j]) + __uint_as_float(t2[j]));
              }
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (j < jmax) {                                   // warp-uniform
                TY* yrow = (TY*)__shfl_sync(0xFFFFFFFFu, (unsigned long long)dst_l, j);
                const float beta = __shfl_sync(0xFFFFFFFFu, beta_l, j);
                const float gamma = __shfl_sync(0xFFFFFFFFu, gamma_l, j);
                float a = __uint_as_float(hi[j]);
                if (q.split > 1) a += __uint_as_float(lo[j]);
                a += bias_n[mb] * beta;
                if (p.has_out_alpha) a *= p.out_alpha;
                if (swiglu) {
                  const float other = __shfl_xor_sync(0xFFFFFFFFu, a, 1);
                  if (!(lane & 1) && yrow != nullptr && n + 1 < p.N)
                    yrow[n >> 1] = from_f32<TY>(gemm_swiglu(a, other, p.act_alpha, p.act_limit, p.act_has_limit) * gamma);
                } else if (yrow != nullptr && n < p.N) {
                  yrow[n] = from_f32<TY>(a * gamma);
                }
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(BAR_ACC_EMPTY(ab));
    }
  }

  // ---- teardown ----------------------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

// ---- host side -----------------------------------------------------------------------------------------------
struct MxPlan {
  int tb, n_mma, split, f4, km, mb, KT, NB, n_groups, stages, stage_bytes, acc_bufs;
  int64_t grid_m, chunk_bytes, ws_bytes;
};

int64_t blocks_bound(int64_t n_slices, int64_t n_rows, int64_t block) {
  if (n_rows <= n_slices) return n_rows;
  const int64_t a = n_rows + 1 - n_slices;
  return n_slices - 1 + (a + block - 1) / block;
}

MxPlan mx_plan(const MoeGemmArgs& a) {
  MxPlan pl;
  const bool bf16 = a.x_dtype == MOE_BF16;
  const bool pin_f4 = bf16 && a.kernel == MOE_GEMM_MX_F4, pin_f8 = a.kernel == MOE_GEMM_MX_F8;
  const int tb_max = bf16 ? (pin_f4 ? 32 : 64) : 128;
  int tb = 16;
  if (a.tile_m == 16 || a.tile_m == 32 || a.tile_m == 64 || a.tile_m == 128) {
    tb = a.tile_m;
  } else {
    // bf16 tokens: 16 rows up to 8 rows per expert on average, 32 beyond (64-row blocks were slower than two 32-row
    // blocks at every size measured: 32 rows per expert 294 against 226 us on a 32-expert layer, 911 against 698 us on
    // a 128-expert one); fp8 tokens grow to 128
    const int64_t per = a.slice_sizes ? (a.M + a.E - 1) / a.E : a.M;      // mean rows per expert
    const int tb_auto = bf16 ? (tb_max < 32 ? tb_max : 32) : tb_max;
    while (tb < tb_auto && tb < 2 * per) tb *= 2;
  }
  if (tb > tb_max) tb = tb_max;
  pl.tb = tb;
  // bf16 tokens: four e2m1 terms for the smallest blocks (weight streaming decides there), else two e4m3 terms
  pl.f4 = (bf16 && !pin_f8 && (pin_f4 || tb == 16)) ? 1 : 0;
  pl.split = bf16 ? (pl.f4 ? 4 : 2) : 1;
  pl.n_mma = pl.split > 1 ? pl.split * tb : (tb < 32 ? 32 : tb);     // a scale chunk serves 32 columns at a time
  pl.KT = (int)cdiv64(a.K, 128);
  pl.NB = (int)cdiv64(a.N, 128);
  pl.grid_m = a.slice_sizes ? blocks_bound(a.E, a.M, tb) : cdiv64(a.M, tb);
  // three weight blocks per CTA tile share one token tile (fewer token bytes per weight byte); one block when there
  // would be too few tiles to fill the SMs
  const int64_t items3 = pl.grid_m * cdiv64(pl.NB, 3);
  pl.mb = (a.tile_n == 128) ? 1 : ((a.tile_n == 384 || items3 >= (int64_t)moe_sm_count()) ? 3 : 1);
  // too few tiles for three blocks each, four-term form: single weight blocks, three k steps of one block per stage
  // (a stage of one 8 KB tile does not keep a copy pipeline busy)
  pl.km = (pl.f4 && tb == 16 && pl.mb == 1 && a.tile_n == 0 && pl.KT >= 3) ? 1 : 0;
  pl.n_groups = (int)cdiv64(pl.NB, pl.mb);
  pl.chunk_bytes = (int64_t)pl.n_mma * (pl.f4 ? 64 : 128) + 1024;
  const int ctl_bytes = MX_CTL_BYTES;
  if (pl.km) {
    pl.mb = 3;                                       // tiles of a stage; n_groups stays the number of weight blocks
    pl.stage_bytes = 3 * MX_W_TILE_TX + 3 * (int)pl.chunk_bytes + 2048;
    int st = (MX_SMEM_LIMIT - 1024 - ctl_bytes) / pl.stage_bytes;
    pl.stages = st > 5 ? 5 : st;
    pl.acc_bufs = 2;
  } else {
    pl.stage_bytes = pl.mb * (pl.f4 ? MX_W_TILE_TX : MX_W_TILE) + (int)pl.chunk_bytes + 2048;
    int st = (MX_SMEM_LIMIT - 1024 - ctl_bytes) / pl.stage_bytes;
    pl.stages = st > MX_MAX_STAGES ? MX_MAX_STAGES : st;
    pl.acc_bufs = (2 * pl.mb * pl.n_mma <= MX_SF_BASE) ? 2 : 1;
  }
  pl.ws_bytes = pl.grid_m * pl.KT * pl.chunk_bytes;
  return pl;
}

int make_w_map(const MoeGemmArgs& a, const MxPlan& pl, int n_blocks, CUtensorMap* map) {
  static PFN_cuTensorMapEncodeTiled_v12000 encode = nullptr;
  static std::mutex mu;
  {
    std::lock_guard<std::mutex> lk(mu);
    if (!encode) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult qr;
      MOE_CHECK_CUDA(cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &fn, 12000, cudaEnableDefault, &qr));
      if (qr != cudaDriverEntryPointSuccess || !fn) {
        moe_set_error("moe_grouped_gemm: the driver does not provide cuTensorMapEncodeTiled");
        return MOE_ERR_UNSUPPORTED;
      }
      encode = (PFN_cuTensorMapEncodeTiled_v12000)fn;
    }
  }
  // [tile][128 rows][128 e2m1 = 64 bytes].  Byte-per-element form: the TMA unit writes 16 elements per 16 bytes of
  // shared memory (128-byte rows, 128-byte swizzle); packed form: the 64-byte rows as they are, 64-byte swizzle.
  const cuuint64_t tiles = (cuuint64_t)a.E * (cuuint64_t)pl.KT * (cuuint64_t)pl.NB;
  const cuuint64_t inner = pl.f4 ? 64 : 128;
  const cuuint64_t dims[3] = {inner, 128, tiles};
  const cuuint64_t strides[2] = {64, 64 * 128};
  const cuuint32_t box[3] = {(cuuint32_t)inner, 128, (cuuint32_t)n_blocks};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = encode(map, pl.f4 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 3,
                            const_cast<void*>(a.w), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            pl.f4 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    moe_set_error("moe_grouped_gemm: cuTensorMapEncodeTiled (packed e2m1 weights) failed with code %d (%llu tiles)", (int)r,
                  (unsigned long long)tiles);
    return MOE_ERR_CUDA;
  }
  return MOE_OK;
}

// launch with the programmatic-stream-serialization attribute (see pdl_wait above)
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

template <typename TY, int MB, bool F4, bool KM = false>
int launch_mx(const GemmParams& p, const MxParams& q, const MxPlan& pl, const MxMaps& w_map, int idle_sms, cudaStream_t st) {
  const int smem = pl.stages * pl.stage_bytes + MX_CTL_BYTES + 1024;
  const int64_t items = pl.grid_m * pl.n_groups;
  int sms = moe_sm_count() - idle_sms;
  if (sms < 1) sms = 1;
  const int grid = (int)(items < sms ? items : sms);
  MOE_CHECK_CUDA(cudaFuncSetAttribute(gemm_mx_kernel<TY, MB, F4, KM>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  MOE_CHECK_CUDA(launch_pdl(gemm_mx_kernel<TY, MB, F4, KM>, dim3(grid), dim3(MX_THREADS), (size_t)smem, st, p, q, w_map));
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}

template <typename TY>
int launch_mx_ty(const GemmParams& p, const MxParams& q, const MxPlan& pl, const MxMaps& w_map, int idle_sms, cudaStream_t st) {
  if (pl.km) return launch_mx<TY, 3, true, true>(p, q, pl, w_map, idle_sms, st);
  if (pl.f4) return pl.mb == 3 ? launch_mx<TY, 3, true>(p, q, pl, w_map, idle_sms, st) : launch_mx<TY, 1, true>(p, q, pl, w_map, idle_sms, st);
  return pl.mb == 3 ? launch_mx<TY, 3, false>(p, q, pl, w_map, idle_sms, st) : launch_mx<TY, 1, false>(p, q, pl, w_map, idle_sms, st);
}

}  // namespace

bool moe_gemm_mx_supported(const MoeGemmArgs& a, const char** why) {
  if (a.w_kind != MOE_W_MX4_B200MX) { *why = "weights are not in the block-scaled B200 layout"; return false; }
  if (a.x_dtype != MOE_BF16 && a.x_dtype != MOE_F8E4M3) { *why = "activations are neither bf16 nor e4m3"; return false; }
  if (a.y_dtype != MOE_BF16 && a.y_dtype != MOE_F32 && a.y_dtype != MOE_F8E4M3) { *why = "output is neither bf16, fp32 nor e4m3"; return false; }
  if ((uintptr_t)a.x % 16 != 0 || (a.ld_x * (a.x_dtype == MOE_BF16 ? 2 : 1)) % 16 != 0) {
    *why = "activation rows are not 16-byte aligned"; return false;
  }
  if ((uintptr_t)a.w % 32 != 0 || (uintptr_t)a.w_scale % 16 != 0) { *why = "weights are not 32-byte aligned"; return false; }
  if (a.K % 32 != 0) { *why = "K is not a multiple of 32"; return false; }
  if (a.x_scale && a.x_dtype != MOE_F8E4M3) { *why = "activation scales need e4m3 activations"; return false; }
  if (a.kernel == MOE_GEMM_MX_F4 && a.x_dtype != MOE_BF16) { *why = "the four-term form is for bf16 activations"; return false; }
  if ((int64_t)a.E * cdiv64(a.K, 128) * cdiv64(a.N, 128) >= 2147483647LL) { *why = "too many weight tiles"; return false; }
  *why = "";
  return true;
}

extern "C" __attribute__((visibility("default"))) size_t moe_gemm_mx_workspace_bytes(const MoeGemmArgs* a) {
  if (!a || a->M <= 0 || a->E <= 0) return 0;
  return (size_t)mx_plan(*a).ws_bytes;
}

int moe_gemm_mx_launch(const GemmParams& p_in, const MoeGemmArgs& a, cudaStream_t st) {
  const MxPlan pl = mx_plan(a);
  if (pl.grid_m == 0) return MOE_OK;
  MOE_CHECK_ARG(a.mx_workspace != nullptr && a.mx_workspace_bytes >= pl.ws_bytes && (uintptr_t)a.mx_workspace % 1024 == 0,
                "moe_grouped_gemm: the block-scaled kernel needs mx_workspace of moe_gemm_mx_workspace_bytes() = %lld "
                "bytes, 1024-byte aligned (got %lld)", (long long)pl.ws_bytes, (long long)a.mx_workspace_bytes);
  MOE_CHECK_ARG(pl.stages >= 2, "moe_grouped_gemm: block-scaled tile does not fit shared memory");
  GemmParams p = p_in;
  if (a.slice_sizes) {
    int row = 0;
    while ((16 << row) < pl.tb) ++row;
    p.block_offs = a.block_offs_16 + row * a.ld_block_offs;
    p.block_sched = a.block_sched_16 + row * a.ld_block_sched;
  }
  PackParams pk;
  pk.x = a.x; pk.ld_x = a.ld_x; pk.rows_x = a.rows_x;
  pk.x_scale = a.x_scale; pk.ld_xs = a.ld_x_scale;
  pk.gather = a.gather_indx;
  pk.K = a.K; pk.KT = pl.KT; pk.tb = pl.tb; pk.n_mma = pl.n_mma;
  pk.chunk_bytes = pl.chunk_bytes;
  pk.out = (uint8_t*)a.mx_workspace;
  const dim3 pgrid((unsigned)pl.grid_m, (unsigned)pl.KT);
  MOE_CHECK_ARG(pl.grid_m < 2147483647LL, "moe_grouped_gemm: too many token blocks");
  if (pl.f4) MOE_CHECK_CUDA(launch_pdl(mx_pack_x4_kernel, pgrid, dim3(256), 0, st, p, pk));
  else if (pl.split > 1) MOE_CHECK_CUDA(launch_pdl(mx_pack_x_kernel<true>, pgrid, dim3(256), 0, st, p, pk));
  else MOE_CHECK_CUDA(launch_pdl(mx_pack_x_kernel<false>, pgrid, dim3(256), 0, st, p, pk));
  MOE_CHECK_LAUNCH();

  MxParams q;
  q.xq = (const uint8_t*)a.mx_workspace; q.chunk_bytes = pl.chunk_bytes;
  q.n_mma = pl.n_mma; q.tb = pl.tb; q.split = pl.split;
  q.KT = pl.KT; q.NB = pl.NB; q.stages = pl.stages; q.stage_bytes = pl.stage_bytes; q.acc_bufs = pl.acc_bufs;
  q.n_groups = pl.n_groups; q.grid_m = pl.grid_m;
  MxMaps w_map;
  for (int nb = 1; nb <= 3; ++nb)
    if (int rc = make_w_map(a, pl, nb <= pl.mb ? nb : pl.mb, &w_map.m[nb - 1])) return rc;
  const int idle = a.idle_sms > 0 ? a.idle_sms : 0;
  if (a.y_dtype == MOE_F8E4M3) return launch_mx_ty<__nv_fp8_e4m3>(p, q, pl, w_map, idle, st);
  if (a.y_dtype == MOE_BF16) return launch_mx_ty<__nv_bfloat16>(p, q, pl, w_map, idle, st);
  return launch_mx_ty<float>(p, q, pl, w_map, idle, st);
}
