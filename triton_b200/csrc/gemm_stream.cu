// Ragged grouped GEMM for the decode regime: a handful of token rows per expert, every active expert's MXFP4 weights
// read exactly once, bound by HBM.
//
// A work item is (expert, block of up to 16 of its rows, 128 weight rows).  Each CTA takes a contiguous range of
// items, so the token rows of an expert are staged in shared memory once and reused for all of its weight tiles.
// Seventeen warps: warp 16 (one thread) streams the packed weight tiles of its items through a ring of 8.5 KB stages
// with cp.async.bulk (the B200 layout makes every tile contiguous); warps 0-15 are two groups of eight, one for the
// even and one for the odd 128-k tiles, and inside a group each warp owns 16 weight rows: registers <- packed words
// of the stage, shifts and masks turn them into fp16 A fragments (an e2m1 code with its three magnitude bits at fp16
// bits 11:9 is value * 2^-14 exactly), the token rows sit in shared memory as fp16 B fragments (each row scaled by a
// power of two that puts its largest element in [2^11, 2^12): exact for every element within 2^25 of the row maximum,
// error at most max * 2^-25 for smaller ones, which go subnormal in fp16), and mma.sync m16n8k16 accumulates one 32-k scale group into fp32, which is then multiplied by the group's
// e8m0 scale and added to the running sum; the two groups' sums meet in shared memory before the epilogue.
// No warp waits for another one except through the weight ring, so there is no per-step hand-off chain as in the
// tcgen05 pipeline; the legacy tensor path (a quarter of the tcgen05 rate) is far more than 16 tokens need.
// Every wait on the ring is bounded like in the tcgen05 kernel.
#include "gemm_tc_common.cuh"
#include <cuda_fp16.h>

namespace {

constexpr int S_CONSUMER_WARPS = 16;     // two groups of eight: even / odd 128-k weight tiles of an item
constexpr int S_THREADS = (S_CONSUMER_WARPS + 1) * 32;
constexpr int S_STAGES = 12;             // ring of (8 KB values + 512 B scales) stages
constexpr int S_STAGE_BYTES = 2 * RAWV_BYTES + RAWS_BYTES;
constexpr int S_ROWS = 16;               // token rows per item (two n8 blocks)
constexpr int S_MAX_KG = 96;             // 32-k groups the staged token rows can hold (K <= 3072)
constexpr int S_MAX_EXPERTS = 1024;

struct StreamSmem {
  static constexpr int OFF_RING = 0;
  static constexpr int OFF_X = OFF_RING + S_STAGES * S_STAGE_BYTES;          // [K/32][2 blocks][8 rows][64 B] fp16
  static constexpr int OFF_RED = OFF_X + S_MAX_KG * 1024;                      // [2][8 warps][32 lanes][8] float partial sums
  static constexpr int OFF_XEXP = OFF_RED + 2 * 8 * 32 * 8 * 4;                // float[16]: 2^(row exponent)
  static constexpr int OFF_BAR = OFF_XEXP + 64;
  static constexpr int OFF_MISC = OFF_BAR + (2 * S_STAGES + 3) * 8;
  static constexpr int OFF_PREFIX = OFF_MISC + 16;
  static constexpr int BYTES = OFF_PREFIX + (S_MAX_EXPERTS + 1) * 4;
  static constexpr int ALLOC = BYTES + 1024;
  static_assert(ALLOC <= 232448, "shared memory budget");
};

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// the same with a zero accumulator input (no registers to clear)
__device__ __forceinline__ void mma_f16_16816_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                   uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
// pair i of word w (nibble i of the low half-word is k = 2i, of the high half-word k = 2i + 1) -> fp16x2 of
// value * 2^-14: the three magnitude bits at fp16 bits 11:9 (exponent bias 15 against e2m1's 1, subnormal 0.5 included)
template <int I> __device__ __forceinline__ uint32_t e2m1_pair_f16(uint32_t w) {
  const uint32_t mag = (I < 3 ? (w << (9 - 4 * I)) : (w >> (4 * I - 9))) & 0x0E000E00u;
  const uint32_t sgn = (I < 3 ? (w << (12 - 4 * I)) : w) & 0x80008000u;
  return mag | sgn;
}
// e8m0 byte g of a scale word -> 2^(byte - 127) as fp32 bits (byte 0 -> 0.0)
template <int G> __device__ __forceinline__ float scale_f32(uint32_t sc) {
  return __uint_as_float(__byte_perm(sc, 0u, 0x4440u | G) << 23);
}

// item -> (expert, first row of the block, rows in the block, weight tile along n)
struct Item { int e; int64_t row0; int rows; int nt; };

template <typename TY>
__global__ void __launch_bounds__(S_THREADS, 1) gemm_stream_kernel(const GemmParams p) {
  using C = StreamSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t bar0 = sbase + C::OFF_BAR;
  auto BAR_FULL = [&](int s) { return bar0 + 8u * (uint32_t)s; };
  auto BAR_EMPTY = [&](int s) { return bar0 + 8u * (uint32_t)(S_STAGES + s); };
  const uint32_t BAR_X_FREE = bar0 + 8u * (uint32_t)(2 * S_STAGES), BAR_X_READY = BAR_X_FREE + 8u, BAR_RED = BAR_X_FREE + 16u;
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + C::OFF_MISC);
  int32_t* s_prefix = reinterpret_cast<int32_t*>(smem + C::OFF_PREFIX);
  float* s_xexp = reinterpret_cast<float*>(smem + C::OFF_XEXP);
  Ctl ctl{s_abort, p.status};

  const int NT = (p.N + HALF_N - 1) / HALF_N;
  const int KT_TILES = (p.K + TILE_K - 1) / TILE_K;
  const int KG = p.K >> 5;                                  // 32-k groups (K % 32 == 0)
  const int n_experts = p.slice_sizes ? p.E : 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S_STAGES; ++s) {
      mbar_init(BAR_FULL(s), 1);
      mbar_init(BAR_EMPTY(s), 8);                             // the eight warps of the group that reads the stage
    }
    mbar_init(BAR_X_FREE, S_CONSUMER_WARPS);
    mbar_init(BAR_X_READY, S_CONSUMER_WARPS);
    mbar_init(BAR_RED, S_CONSUMER_WARPS);
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // items per expert: ceil(rows / 16) row blocks x NT weight tiles; exclusive prefix in shared memory
  for (int e = threadIdx.x; e < n_experts; e += S_THREADS) {
    const int rows = p.slice_sizes ? max(p.slice_sizes[e], 0) : (int)p.M;
    s_prefix[e + 1] = ((rows + S_ROWS - 1) / S_ROWS) * NT;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    s_prefix[0] = 0;
    for (int e = 1; e <= n_experts; ++e) {
      run += s_prefix[e];
      s_prefix[e] = run;
    }
  }
  __syncthreads();
  const int64_t total = s_prefix[n_experts];
  const int64_t i_begin = total * blockIdx.x / gridDim.x, i_end = total * (blockIdx.x + 1) / gridDim.x;

  auto item_at = [&](int64_t i, Item& it) {
    int lo = 0, hi = n_experts;                             // largest e with prefix[e] <= i
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (s_prefix[mid] <= i) lo = mid; else hi = mid;
    }
    const int j = (int)(i - s_prefix[lo]);
    const int blk = j / NT;
    it.e = lo;
    it.nt = j - blk * NT;
    const int rows_e = p.slice_sizes ? p.slice_sizes[lo] : (int)p.M;
    it.row0 = (p.slice_sizes ? (int64_t)p.slice_offs[lo] : 0) + (int64_t)blk * S_ROWS;
    it.rows = min(S_ROWS, rows_e - blk * S_ROWS);
  };

  if (warp == S_CONSUMER_WARPS) {
    // ================================= weight producer =================================================
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      const uint8_t* wv = (const uint8_t*)p.w;
      const uint8_t* ws = p.w_scale;
      for (int64_t i = i_begin; i < i_end && ok; ++i) {
        Item m;
        item_at(i, m);
        const int64_t tile0 = ((int64_t)m.e * NT + m.nt) * KT_TILES;
        for (int kt = 0; kt < KT_TILES; ++kt, ++it) {
          const int s = it % S_STAGES;
          ok = mbar_wait(BAR_EMPTY(s), ((it / S_STAGES) & 1u) ^ 1u, ctl, 701);
          if (!ok) break;
          const uint32_t dst = sbase + C::OFF_RING + s * S_STAGE_BYTES;
          mbar_expect_tx(BAR_FULL(s), (uint32_t)S_STAGE_BYTES);
          bulk_g2s(dst, wv + (tile0 + kt) * (2 * RAWV_BYTES), 2 * RAWV_BYTES, BAR_FULL(s));
          bulk_g2s(dst + 2 * RAWV_BYTES, ws + (tile0 + kt) * RAWS_BYTES, RAWS_BYTES, BAR_FULL(s));
        }
      }
      if (!ok) {
        const uint32_t lo = it > (uint32_t)S_STAGES ? it - S_STAGES : 0;
        for (uint32_t j = lo; j < it; ++j)
          for (uint32_t t = 0; t < (1u << 16) && !mbar_test(BAR_FULL(j % S_STAGES), (j / S_STAGES) & 1u); ++t) __nanosleep(64);
      }
    }
  } else {
    // ================================= consumers ========================================================
    const int wrow = warp & 7, khalf = warp >> 3;              // 16-row slab of the tile, parity of the k tiles taken
    const int qrow = lane >> 2, c4 = lane & 3;                 // fragment row inside the slab, k word of a quad
    const int r_lo = wrow * 16 + qrow, r_hi = r_lo + 8;        // the two weight rows of this thread inside the tile
    const bool swiglu = p.activation == MOE_ACT_SWIGLU;
    uint32_t it = 0, xphase = 0, rphase = 0;
    bool ok = true;
    int cur_e = -1;
    int64_t cur_row0 = -1;
    // barrier among the consumer warps with a bounded wait (a CTA-wide bar.sync could not be left on abort)
    auto consumer_sync = [&](uint32_t bar, uint32_t phase) -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(bar);
      return __all_sync(0xFFFFFFFFu, mbar_wait(bar, phase & 1u, ctl, 703));
    };
    for (int64_t i = i_begin; i < i_end && ok; ++i) {
      Item m;
      item_at(i, m);
      if (m.e != cur_e || m.row0 != cur_row0) {
        // ---- stage the block's token rows (warp w takes row w): fp16, each row scaled by a power of two,
        // [32-k group][n8 block][row][64 B]
        ok = consumer_sync(BAR_X_FREE, xphase);                // everyone is done with the previous block's rows
        if (!ok) break;
        const int row = warp;
        int64_t src = -1;
        if (row < m.rows) {
          const int64_t mm = m.row0 + row;
          src = p.gather_indx ? (int64_t)p.gather_indx[mm] : mm;
          if (src >= p.rows_x) src = -1;
        }
        const __nv_bfloat16* xr = src >= 0 ? (const __nv_bfloat16*)p.x + src * p.ld_x : nullptr;
        float mx = 0.0f;
        if (xr)
          for (int k8 = lane; k8 < (p.K >> 3); k8 += 32) {
            const uint4 v = *reinterpret_cast<const uint4*>(xr + k8 * 8);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = __bfloat1622float2(h[j]);
              mx = fmaxf(mx, fmaxf(fabsf(f.x), fabsf(f.y)));
            }
          }
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        // row exponent: the largest element lands in [2^11, 2^12) (products with |w| <= 6 stay far below the fp16
        // maximum inside the tensor core's exact fp32 accumulation); rows of zeros or without a source use 0
        int ex = 0;
        if (mx > 0.0f && mx < 3.0e38f) ex = (int)((__float_as_uint(mx) >> 23) & 0xFF) - 127 - 11;
        ex = max(-100, min(100, ex));
        const float down = __uint_as_float((uint32_t)(127 - ex) << 23);     // 2^-ex
        if (lane == 0) s_xexp[row] = __uint_as_float((uint32_t)(127 + ex + 14) << 23);   // 2^ex * 2^14 undoes both scalings
        const int blk = row >> 3, n = row & 7;
        for (int k8 = lane; k8 < KT_TILES * 16; k8 += 32) {      // up to the end of the last 128-k tile: zeros past K
          uint4 out = make_uint4(0, 0, 0, 0);
          if (xr && k8 < (p.K >> 3)) {
            const uint4 v = *reinterpret_cast<const uint4*>(xr + k8 * 8);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
            float f[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 t2 = __bfloat1622float2(h[j]);
              f[2 * j] = t2.x * down;
              f[2 * j + 1] = t2.y * down;
            }
            __half2 o2[4] = {__floats2half2_rn(f[0], f[1]), __floats2half2_rn(f[2], f[3]), __floats2half2_rn(f[4], f[5]),
                             __floats2half2_rn(f[6], f[7])};
            out = *reinterpret_cast<const uint4*>(o2);
          }
          const int g = k8 >> 2, c = k8 & 3;
          *reinterpret_cast<uint4*>(smem + C::OFF_X + ((g * 2 + blk) * 8 + n) * 64 + c * 16) = out;
        }
        ok = consumer_sync(BAR_X_READY, xphase);
        if (!ok) break;
        ++xphase;
        cur_e = m.e;
        cur_row0 = m.row0;
      }
      const int nblk = m.rows > 8 ? 2 : 1;
      float acc[2][4];
#pragma unroll
      for (int b = 0; b < 2; ++b)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[b][j] = 0.0f;

      for (int kt = 0; kt < KT_TILES; ++kt, ++it) {
        if ((kt & 1) != khalf) continue;
        const int s = it % S_STAGES;
        ok = __all_sync(0xFFFFFFFFu, mbar_wait(BAR_FULL(s), (it / S_STAGES) & 1u, ctl, 702));
        if (!ok) break;
        const uint32_t stage = sbase + C::OFF_RING + s * S_STAGE_BYTES;
        const uint32_t sc_lo = lds32(stage + 2 * RAWV_BYTES + r_lo * 4);
        const uint32_t sc_hi = lds32(stage + 2 * RAWV_BYTES + r_hi * 4);
        // all four 32-k groups of the tile, unconditionally: past K the packed weights and their scales are zero
        // padding and the staged token rows are zeros
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          {
            const uint32_t wl = lds32(stage + g * 2048 + r_lo * 16 + c4 * 4);
            const uint32_t wh = lds32(stage + g * 2048 + r_hi * 16 + c4 * 4);
            const float fl = g == 0 ? scale_f32<0>(sc_lo) : g == 1 ? scale_f32<1>(sc_lo) : g == 2 ? scale_f32<2>(sc_lo) : scale_f32<3>(sc_lo);
            const float fh = g == 0 ? scale_f32<0>(sc_hi) : g == 1 ? scale_f32<1>(sc_hi) : g == 2 ? scale_f32<2>(sc_hi) : scale_f32<3>(sc_hi);
            const uint32_t p0 = e2m1_pair_f16<0>(wl), p1 = e2m1_pair_f16<1>(wl), p2 = e2m1_pair_f16<2>(wl),
                           p3 = e2m1_pair_f16<3>(wl);
            const uint32_t q0 = e2m1_pair_f16<0>(wh), q1 = e2m1_pair_f16<1>(wh), q2 = e2m1_pair_f16<2>(wh),
                           q3 = e2m1_pair_f16<3>(wh);
            const uint32_t xg = sbase + C::OFF_X + ((kt * 4 + g) * 2) * 512 + qrow * 64 + c4 * 16;
#pragma unroll
            for (int b = 0; b < 2; ++b) {
              if (b < nblk) {
                const uint4 xb = lds128(xg + b * 512);
                float d[4];
                mma_f16_16816_zero(d, p0, q0, p1, q1, xb.x, xb.y);
                mma_f16_16816(d, p2, q2, p3, q3, xb.z, xb.w);
                acc[b][0] = fmaf(fl, d[0], acc[b][0]);
                acc[b][1] = fmaf(fl, d[1], acc[b][1]);
                acc[b][2] = fmaf(fh, d[2], acc[b][2]);
                acc[b][3] = fmaf(fh, d[3], acc[b][3]);
              }
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(BAR_EMPTY(s));
      }
      if (!ok) break;

      // ---- the odd-k group hands its partial sums to the even-k group (double-buffered by item) -------------
      float* red = reinterpret_cast<float*>(smem + C::OFF_RED) + (((rphase & 1u) * 8 + wrow) * 32 + lane) * 8;
      if (khalf == 1) {
#pragma unroll
        for (int b = 0; b < 2; ++b) *reinterpret_cast<float4*>(red + 4 * b) = make_float4(acc[b][0], acc[b][1], acc[b][2], acc[b][3]);
      }
      ok = consumer_sync(BAR_RED, rphase);
      ++rphase;
      if (!ok) break;
      if (khalf == 1) continue;
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        const float4 o = *reinterpret_cast<const float4*>(red + 4 * b);
        acc[b][0] += o.x; acc[b][1] += o.y; acc[b][2] += o.z; acc[b][3] += o.w;
      }

      // ---- epilogue: thread holds rows r_lo / r_hi of the tile for tokens 8 b + 2 c4 + {0, 1} --------------
      const int n_lo = m.nt * HALF_N + r_lo, n_hi = n_lo + 8;
      const float bias_lo = (p.bias && n_lo < p.N) ? load_bias(p.bias, p.bias_dtype, (int64_t)m.e * p.ld_bias + n_lo) : 0.0f;
      const float bias_hi = (p.bias && n_hi < p.N) ? load_bias(p.bias, p.bias_dtype, (int64_t)m.e * p.ld_bias + n_hi) : 0.0f;
#pragma unroll
      for (int b = 0; b < 2; ++b) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int t = b * 8 + c4 * 2 + j;                    // token row inside the block
          const bool live = b < nblk && t < m.rows;
          const int64_t mm = m.row0 + (live ? t : 0);
          int64_t dst = -1;
          float beta = 1.0f, gamma = 1.0f, undo = 0.0f;
          if (live) {
            dst = p.scatter_indx ? (int64_t)p.scatter_indx[mm] : mm;
            if (p.betas) beta = p.betas[mm];
            if (p.gammas) gamma = p.gammas[mm];
            undo = s_xexp[t];
          }
          float v_lo = acc[b][j] * undo + bias_lo * beta;
          float v_hi = acc[b][2 + j] * undo + bias_hi * beta;
          if (p.has_out_alpha) { v_lo *= p.out_alpha; v_hi *= p.out_alpha; }
          if (swiglu) {
            // gate / linear pairs are weight rows (2i, 2i + 1): fragment rows qrow and qrow ^ 1, four lanes apart
            const float o_lo = __shfl_xor_sync(0xFFFFFFFFu, v_lo, 4);
            const float o_hi = __shfl_xor_sync(0xFFFFFFFFu, v_hi, 4);
            if (!(qrow & 1) && dst >= 0) {
              TY* yrow = gemm_out_row<TY>(p, dst);
              if (n_lo + 1 < p.N)
                yrow[n_lo >> 1] = from_f32<TY>(gemm_swiglu(v_lo, o_lo, p.act_alpha, p.act_limit, p.act_has_limit) * gamma);
              if (n_hi + 1 < p.N)
                yrow[n_hi >> 1] = from_f32<TY>(gemm_swiglu(v_hi, o_hi, p.act_alpha, p.act_limit, p.act_has_limit) * gamma);
            }
          } else if (dst >= 0) {
            TY* yrow = gemm_out_row<TY>(p, dst);
            if (n_lo < p.N) yrow[n_lo] = from_f32<TY>(v_lo * gamma);
            if (n_hi < p.N) yrow[n_hi] = from_f32<TY>(v_hi * gamma);
          }
        }
      }
    }
  }
}

}  // namespace

bool moe_gemm_stream_supported(const MoeGemmArgs& a, const char** why) {
  if (a.K > S_MAX_KG * 32) { *why = "K exceeds what the staged token rows hold"; return false; }
  if (a.slice_sizes && a.E > S_MAX_EXPERTS) { *why = "too many experts"; return false; }
  *why = "";
  return true;
}

int moe_gemm_stream_launch(const GemmParams& p, const MoeGemmArgs& a, cudaStream_t st) {
  const int sms = (moe_sm_count() - (a.idle_sms > 0 ? a.idle_sms : 0)) > 0 ? moe_sm_count() - (a.idle_sms > 0 ? a.idle_sms : 0) : 1;
  // at most one CTA per SM (shared memory); fewer when there cannot be that many items
  const int64_t nt = cdiv64(a.N, HALF_N);
  const int64_t max_items = (a.slice_sizes ? (int64_t)a.E + cdiv64(a.M, S_ROWS) : cdiv64(a.M, S_ROWS)) * nt;
  const int grid = (int)(max_items < sms ? (max_items > 0 ? max_items : 1) : sms);
  if (a.y_dtype == MOE_BF16) {
    MOE_CHECK_CUDA(cudaFuncSetAttribute(gemm_stream_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        StreamSmem::ALLOC));
    gemm_stream_kernel<__nv_bfloat16><<<grid, S_THREADS, StreamSmem::ALLOC, st>>>(p);
  } else {
    MOE_CHECK_CUDA(cudaFuncSetAttribute(gemm_stream_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        StreamSmem::ALLOC));
    gemm_stream_kernel<float><<<grid, S_THREADS, StreamSmem::ALLOC, st>>>(p);
  }
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}
