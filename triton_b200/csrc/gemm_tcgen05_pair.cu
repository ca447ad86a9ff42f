// Ragged grouped GEMM, bf16 activations x MXFP4 weights, on a pair of SMs (tcgen05 cta_group::2).
//
// A cluster of two CTAs computes one 256-token x 256-column output tile per pass.  CTA `rank` of the pair
//   * gathers token rows [128 rank, 128 rank + 128) of the tile (its half of the MMA's M operand),
//   * streams and dequantises weight rows [128 rank, 128 rank + 128) of the tile (its half of the N operand),
//   * owns accumulator rows [128 rank, +128) x 256 columns in its tensor memory and writes them out.
// One thread of the even CTA issues M = 256, N = 256, K = 16 MMAs that read both CTAs' shared memory, so each SM
// fills and reads half of the operand bytes a single-SM 256 x 256 tile needs, and the accumulator takes 256 of the
// 512 tensor-memory columns: two buffers, so the epilogue of one tile overlaps the main loop of the next.
//
// Warp roles in each CTA (576 threads):
//   warp 0        even CTA: MMA issuer (one thread).  Odd CTA: relay, forwards "my stage is full" to the even CTA.
//   warp 1        weight producer: cp.async.bulk of packed weight tiles (8 KB values + 512 B scales per 128 k)
//   warps 2-5     activation loader.  Consecutive token rows: one thread, one TMA tile copy (128 rows x 64 k) per
//                 stage.  Gathered rows: 128 threads, 16-byte cp.async copies into the 128-byte-swizzled stage.
//   warps 6-13    dequantiser: packed e2m1 + e8m0 -> bf16 B stage
//   warps 14-17   epilogue: tcgen05.ld, bias * beta, out_alpha, SwiGLU, gamma, cast, store
// Barriers of a stage: A_FULL, B_FULL (local), PEER_FULL (even CTA only, arrived on by the odd CTA's relay),
// AB_EMPTY (each CTA, arrived on by the MMA's commit, which signals both CTAs).  ACC_FULL is signalled in both CTAs by
// the commit after a tile's last MMA; ACC_EMPTY lives in the even CTA and collects the eight epilogue warps of the
// pair.  Every wait is bounded like in the single-SM kernel; both CTAs meet at a cluster barrier before tensor
// memory is released.
#include "gemm_tc_common.cuh"
#include <mutex>

namespace {

constexpr int PAIR_THREADS = 576;
constexpr int P_WARP_LOADER0 = 2, P_WARP_DEQ0 = 6, P_WARP_EPI0 = 14;
constexpr int P_STAGES = 6;              // operand stages of 64 k
constexpr int P_RAW_STAGES = 3;          // packed-weight stages of 128 k
constexpr int P_TILE_N = 256;
constexpr int P_ACC_COLS = 256;

struct PairSmem {
  static constexpr int A_STAGE = SUBTILE_BYTES, B_STAGE = SUBTILE_BYTES;
  static constexpr int RAWV_STAGE = 2 * RAWV_BYTES, RAWS_STAGE = RAWS_BYTES;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + P_STAGES * A_STAGE;
  static constexpr int OFF_RAWV = OFF_B + P_STAGES * B_STAGE;
  static constexpr int OFF_RAWS = OFF_RAWV + P_RAW_STAGES * RAWV_STAGE;
  static constexpr int OFF_BIAS = OFF_RAWS + P_RAW_STAGES * RAWS_STAGE;   // float, [4 epilogue warps][256]
  static constexpr int OFF_BAR = OFF_BIAS + 4 * P_TILE_N * 4;
  static constexpr int NUM_BARS = 2 * P_RAW_STAGES + 4 * P_STAGES + 4 + 1;
  static constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;                  // tmem base, abort flag
  static constexpr int OFF_PREFIX = OFF_MISC + 16;
  static constexpr int BYTES = OFF_PREFIX + (MAX_PREFIX_EXPERTS + 1) * 4;
  static constexpr int ALLOC = BYTES + 1024;
  static_assert(ALLOC <= 232448, "shared memory budget");
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on the barrier at the same shared-memory offset in CTA `cta` of the cluster.  Default (CTA-scope release)
// semantics: a cluster-scope release costs about a thousand cycles per arrival while copies are in flight, and what
// the arrival publishes here is either a go-ahead for the tensor core of the SM that already holds the data (stage
// full) or the end of tensor-memory reads that were fenced by tcgen05.fence (accumulator drained).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar, uint32_t cta) {
  asm volatile(
      "{\n\t.reg .b32 ra;\n\t"
      "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
      "mbarrier.arrive.shared::cluster.b64 _, [ra];\n\t}" ::"r"(bar),
      "r"(cta)
      : "memory");
}
__device__ __forceinline__ bool mbar_try_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// bounded wait on a barrier that threads of the other CTA arrive on
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, const Ctl& ctl, int code) {
  if (mbar_try_cluster(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (;;) {
    if (mbar_try_cluster(bar, parity)) return true;
    if (*ctl.abort_flag) return false;
    if (global_ns() - t0 > WAIT_LIMIT_NS) {
      *ctl.abort_flag = 1;
      if (ctl.status) atomicExch(ctl.status, code);
      return false;
    }
  }
}

// instruction descriptor of the pair MMA: D fp32, A/B bf16, both K-major, M = 256 over the two CTAs
__device__ __forceinline__ constexpr uint32_t make_idesc_pair(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}
__device__ __forceinline__ void mma_bf16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on the barrier at this offset in both CTAs of the pair once every MMA issued so far has completed
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
      "h"((uint16_t)3)
      : "memory");
}
__device__ __forceinline__ void mma_commit_pair_local(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

template <typename TY>
__global__ void __launch_bounds__(PAIR_THREADS, 1)
gemm_tc_pair_kernel(const GemmParams p, const int64_t grid_m_static, const __grid_constant__ CUtensorMap x_map) {
  using C = PairSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();             // 0: even CTA (issues the MMAs), 1: odd CTA
  const int64_t pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const bool use_gather = p.gather_indx != nullptr;

  const uint32_t bar0 = sbase + C::OFF_BAR;
  auto BAR_RAW_FULL = [&](int s) { return bar0 + 8u * (uint32_t)s; };
  auto BAR_RAW_EMPTY = [&](int s) { return bar0 + 8u * (uint32_t)(P_RAW_STAGES + s); };
  auto BAR_A_FULL = [&](int s) { return bar0 + 8u * (uint32_t)(2 * P_RAW_STAGES + s); };
  auto BAR_B_FULL = [&](int s) { return bar0 + 8u * (uint32_t)(2 * P_RAW_STAGES + P_STAGES + s); };
  auto BAR_PEER_FULL = [&](int s) { return bar0 + 8u * (uint32_t)(2 * P_RAW_STAGES + 2 * P_STAGES + s); };
  auto BAR_AB_EMPTY = [&](int s) { return bar0 + 8u * (uint32_t)(2 * P_RAW_STAGES + 3 * P_STAGES + s); };
  auto BAR_ACC_FULL = [&](int a) { return bar0 + 8u * (uint32_t)(2 * P_RAW_STAGES + 4 * P_STAGES + a); };
  auto BAR_ACC_EMPTY = [&](int a) { return bar0 + 8u * (uint32_t)(2 * P_RAW_STAGES + 4 * P_STAGES + 2 + a); };
  const uint32_t BAR_DRAIN = bar0 + 8u * (uint32_t)(2 * P_RAW_STAGES + 4 * P_STAGES + 4);

  volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(smem + C::OFF_MISC);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + C::OFF_MISC + 4);
  int32_t* s_prefix = reinterpret_cast<int32_t*>(smem + C::OFF_PREFIX);
  Ctl ctl{s_abort, p.status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_RAW_STAGES; ++s) {
      mbar_init(BAR_RAW_FULL(s), 1);
      mbar_init(BAR_RAW_EMPTY(s), 8);                 // the eight dequantiser warps
    }
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(BAR_A_FULL(s), use_gather ? 128 : 1);  // 128 cp.async loader threads, or the TMA thread's expect_tx
      mbar_init(BAR_B_FULL(s), 8);
      mbar_init(BAR_PEER_FULL(s), 1);
      mbar_init(BAR_AB_EMPTY(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(BAR_ACC_FULL(a), 1);
      mbar_init(BAR_ACC_EMPTY(a), 8);                 // four epilogue warps in each CTA
    }
    mbar_init(BAR_DRAIN, 1);
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sbase + C::OFF_MISC),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  if (p.slice_sizes != nullptr) {
    // tile prefix over experts: expert e has ceil(slice_sizes[e] / 256) tiles
    for (int e = threadIdx.x; e < p.E; e += PAIR_THREADS)
      s_prefix[e + 1] = (max(p.slice_sizes[e], 0) + 2 * HALF_M - 1) / (2 * HALF_M);
    __syncthreads();
    if (threadIdx.x == 0) {
      int run = 0;
      s_prefix[0] = 0;
      for (int e = 1; e <= p.E; ++e) {
        run += s_prefix[e];
        s_prefix[e] = run;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                  // the other CTA's barriers exist before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;

  const int NT128 = (p.N + HALF_N - 1) / HALF_N;        // weight tiles along n in memory
  const int NT = (NT128 + 1) / 2;                        // pair tiles along n
  const int KT = (p.K + BLOCK_K - 1) / BLOCK_K;           // 64-k steps
  const int KT_TILES = (p.K + TILE_K - 1) / TILE_K;      // 128-k weight tiles per (expert, n tile)
  int64_t useful_m = grid_m_static;
  if (p.slice_sizes) useful_m = (int64_t)s_prefix[p.E];
  const int64_t n_tiles = useful_m * NT;

  if (warp == 0) {
    if (lane == 0 && rank == 0) {
      // ================================= MMA issuer (even CTA) ==========================================
      uint32_t it = 0, tc = 0;
      bool ok = true;
      const uint32_t idesc = make_idesc_pair(P_TILE_N);
      for (int64_t tile = pair; tile < n_tiles && ok; tile += n_pairs, ++tc) {
        const uint32_t ab = tc & 1u;
        ok = mbar_wait_cluster(BAR_ACC_EMPTY(ab), ((tc >> 1) & 1u) ^ 1u, ctl, 101);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + ab * P_ACC_COLS;
        for (int kt = 0; kt < KT; ++kt, ++it) {
          const int s = it % P_STAGES;
          const uint32_t ph = (it / P_STAGES) & 1u;
          ok = mbar_wait(BAR_A_FULL(s), ph, ctl, 102);
          ok = ok && mbar_wait(BAR_B_FULL(s), ph, ctl, 103);
          ok = ok && mbar_wait_cluster(BAR_PEER_FULL(s), ph, ctl, 105);
          if (!ok) break;
          fence_proxy_async();          // the A stage was written by cp.async (generic proxy) of other threads
          tc_fence_after();
          const uint64_t adesc = make_desc(sbase + C::OFF_A + s * C::A_STAGE);
          const uint64_t bdesc = make_desc(sbase + C::OFF_B + s * C::B_STAGE);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            mma_bf16_pair(d_tmem, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc, (kt | kk) ? 1u : 0u);
          mma_commit_pair(BAR_AB_EMPTY(s));
        }
        if (ok) mma_commit_pair(BAR_ACC_FULL(ab));
      }
      // every MMA issued by this thread has retired before tensor memory is freed
      mma_commit_pair_local(BAR_DRAIN);
      mbar_wait(BAR_DRAIN, 0, ctl, 104);
    } else if (lane == 0) {
      // ================================= relay (odd CTA) ================================================
      uint32_t it = 0;
      bool ok = true;
      for (int64_t tile = pair; tile < n_tiles && ok; tile += n_pairs) {
        for (int kt = 0; kt < KT; ++kt, ++it) {
          const int s = it % P_STAGES;
          const uint32_t ph = (it / P_STAGES) & 1u;
          ok = mbar_wait(BAR_A_FULL(s), ph, ctl, 112);
          ok = ok && mbar_wait(BAR_B_FULL(s), ph, ctl, 113);
          if (!ok) break;
          fence_proxy_async();
          mbar_arrive_cluster(BAR_PEER_FULL(s), 0);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ================================= weight producer =================================================
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      const uint8_t* wv = (const uint8_t*)p.w;
      const uint8_t* ws = p.w_scale;
      for (int64_t tile = pair; tile < n_tiles && ok; tile += n_pairs) {
        int e; int64_t row0; int rows;
        map_tile<2>(p, s_prefix, tile / NT, e, row0, rows);
        const int nt = (int)(tile % NT) * 2 + (int)rank;      // this CTA's weight tile along n
        if (nt >= NT128) continue;                            // no such weight rows: the stage keeps stale data
        const int64_t tile0 = ((int64_t)e * NT128 + nt) * KT_TILES;
        for (int rt = 0; rt < KT_TILES; ++rt, ++it) {
          const int s = it % P_RAW_STAGES;
          ok = mbar_wait(BAR_RAW_EMPTY(s), ((it / P_RAW_STAGES) & 1u) ^ 1u, ctl, 201);
          if (!ok) break;
          mbar_expect_tx(BAR_RAW_FULL(s), (uint32_t)(2 * RAWV_BYTES + RAWS_BYTES));
          bulk_g2s(sbase + C::OFF_RAWV + s * C::RAWV_STAGE, wv + (tile0 + rt) * (2 * RAWV_BYTES), 2 * RAWV_BYTES,
                   BAR_RAW_FULL(s));
          bulk_g2s(sbase + C::OFF_RAWS + s * C::RAWS_STAGE, ws + (tile0 + rt) * RAWS_BYTES, RAWS_BYTES, BAR_RAW_FULL(s));
        }
      }
      if (!ok) {
        // aborting: let the copies that were already issued land before the CTA leaves
        const uint32_t lo = it > (uint32_t)P_RAW_STAGES ? it - P_RAW_STAGES : 0;
        for (uint32_t j = lo; j < it; ++j)
          for (uint32_t i = 0; i < (1u << 16) && !mbar_test(BAR_RAW_FULL(j % P_RAW_STAGES), (j / P_RAW_STAGES) & 1u); ++i)
            __nanosleep(64);
      }
    }
    __syncwarp();
  } else if (warp < P_WARP_DEQ0) {
    // ================================= activation loader ==============================================
    if (!use_gather) {
      // Token rows are consecutive in memory: one thread moves this CTA's whole 128-row x 64-k stage with a single
      // TMA tile copy.  Rows past the end of the expert's segment belong to the next expert (or read as zeros past
      // the end of the matrix) and only reach accumulator rows that are never stored.
      if (warp == P_WARP_LOADER0 && lane == 0) {
        uint32_t it = 0;
        bool ok = true;
        for (int64_t tile = pair; tile < n_tiles && ok; tile += n_pairs) {
          int e; int64_t row0; int rows;
          map_tile<2>(p, s_prefix, tile / NT, e, row0, rows);
          const bool any = rows > (int)rank * HALF_M;
          const int r_first = (int)(row0 + (int64_t)rank * HALF_M);
          for (int kt = 0; kt < KT; ++kt, ++it) {
            const int s = it % P_STAGES;
            ok = mbar_wait(BAR_AB_EMPTY(s), ((it / P_STAGES) & 1u) ^ 1u, ctl, 301);
            if (!ok) break;
            if (any) {
              mbar_expect_tx(BAR_A_FULL(s), (uint32_t)C::A_STAGE);
              tma_tile_2d(sbase + C::OFF_A + s * C::A_STAGE, &x_map, kt * BLOCK_K, r_first, BAR_A_FULL(s));
            } else {
              mbar_arrive(BAR_A_FULL(s));
            }
          }
        }
        if (!ok) {
          // aborting: let the copies that were already issued land before the CTA leaves
          const uint32_t lo = it > (uint32_t)P_STAGES ? it - P_STAGES : 0;
          for (uint32_t j = lo; j < it; ++j)
            for (uint32_t i = 0; i < (1u << 16) && !mbar_test(BAR_A_FULL(j % P_STAGES), (j / P_STAGES) & 1u); ++i)
              __nanosleep(64);
        }
      }
    } else {
    // Gathered token rows: 128 threads move this CTA's 128 x 128-byte stage with 16-byte cp.async copies, thread t owns
    // chunk (t & 7) of rows (t >> 3) + 16 i.  The source of each row is kept in registers for the whole tile and
    // looked up one tile ahead.  (A TMA row gather moves only four 128-byte rows per instruction and sustains about
    // one instruction per 70 cycles, far below what a stage per 500 cycles needs.)
    constexpr int NR = 8;
    const int t = threadIdx.x - P_WARP_LOADER0 * 32;
    const int c8 = t & 7;
    const int rbase = t >> 3;
    const uint8_t* Xb = (const uint8_t*)p.x;
    const uint32_t ld16 = (uint32_t)(p.ld_x >> 3);
    uint32_t dst_off[NR];
#pragma unroll
    for (int i = 0; i < NR; ++i) {
      const int r = rbase + 16 * i;
      dst_off[i] = (uint32_t)(r * 128 + ((c8 ^ (r & 7)) << 4));
    }
    auto load_rows = [&](int64_t tile, uint32_t (&src16)[NR], bool& any) {
      int e; int64_t row0; int rows;
      map_tile<2>(p, s_prefix, tile / NT, e, row0, rows);
      any = rows > (int)rank * HALF_M;
#pragma unroll
      for (int i = 0; i < NR; ++i) {
        const int r = (int)rank * HALF_M + rbase + 16 * i;
        int64_t src = -1;
        if (r < rows) {
          const int64_t m = row0 + r;
          src = p.gather_indx ? (int64_t)p.gather_indx[m] : m;
          if (src >= p.rows_x) src = -1;
        }
        src16[i] = src < 0 ? 0xFFFFFFFFu : (uint32_t)src * ld16;
      }
    };
    uint32_t src16[NR], nxt16[NR];
    bool any = false, nxt_any = false;
    uint32_t it = 0;
    bool ok = true;
    if (pair < n_tiles) load_rows(pair, src16, any);
    for (int64_t tile = pair; tile < n_tiles && ok; tile += n_pairs) {
      const int64_t t2 = tile + n_pairs;
      if (t2 < n_tiles) load_rows(t2, nxt16, nxt_any);
      for (int kt = 0; kt < KT; ++kt, ++it) {
        const int s = it % P_STAGES;
        ok = __all_sync(0xFFFFFFFFu, mbar_wait(BAR_AB_EMPTY(s), ((it / P_STAGES) & 1u) ^ 1u, ctl, 301));
        if (!ok) break;
        const int k = kt * BLOCK_K + c8 * 8;
        const int kleft = p.K - k;
        const uint32_t kbytes = kleft >= 8 ? 16u : (kleft > 0 ? (uint32_t)kleft * 2u : 0u);
        const uint32_t stage = sbase + C::OFF_A + s * C::A_STAGE;
        const uint32_t kc16 = (uint32_t)(k >> 3);
        if (any) {                                            // a half without tokens keeps stale data
#pragma unroll
          for (int i = 0; i < NR; ++i) {
            const bool live = src16[i] != 0xFFFFFFFFu && kbytes;
            const uint8_t* g = live ? Xb + ((uint64_t)(src16[i] + kc16) << 4) : Xb;
            cp_async16(stage + dst_off[i], g, live ? kbytes : 0u);
          }
        }
        cp_async_arrive_noinc(BAR_A_FULL(s));
      }
#pragma unroll
      for (int i = 0; i < NR; ++i) src16[i] = nxt16[i];
      any = nxt_any;
    }
    cp_async_wait_all();
    }
  } else if (warp < P_WARP_EPI0) {
    // ================================= dequantiser ======================================================
    // One unit per thread and stage: (weight row, 32-k scale group) = one 16-byte load, one scale byte, four
    // 16-byte swizzled stores.  A quarter-warp holds one scale group of 8 consecutive rows: the load (128 contiguous
    // bytes) and the stores (8 distinct 16-byte columns) are free of bank conflicts.
    const int dw = warp - P_WARP_DEQ0;              // 0..7
    const int g = (lane >> 3) & 1;                  // scale group inside the 64-k stage
    const int r = dw * 16 + (lane >> 4) * 8 + (lane & 7);
    const int x7 = r & 7;
    uint32_t it = 0, raw_base = 0;
    bool ok = true;
    for (int64_t tile = pair; tile < n_tiles && ok; tile += n_pairs) {
      const bool b_live = (int)(tile % NT) * 2 + (int)rank < NT128;
      for (int kt = 0; kt < KT; ++kt, ++it) {
        const int s = it % P_STAGES;
        const uint32_t ph = (it / P_STAGES) & 1u;
        const uint32_t itr = raw_base + (uint32_t)(kt >> 1);
        const int rs = itr % P_RAW_STAGES;
        bool got = mbar_wait(BAR_AB_EMPTY(s), ph ^ 1u, ctl, 402);
        if (b_live) got = got && mbar_wait(BAR_RAW_FULL(rs), (itr / P_RAW_STAGES) & 1u, ctl, 401);
        ok = __all_sync(0xFFFFFFFFu, got);
        if (!ok) break;
        if (b_live) {
          const uint32_t rv = sbase + C::OFF_RAWV + rs * C::RAWV_STAGE + ((kt & 1) ? RAWV_BYTES : 0) + g * HALF_N * 16;
          const uint32_t rsc = sbase + C::OFF_RAWS + rs * C::RAWS_STAGE + (kt & 1) * 2 + g;
          const uint4 raw = lds128(rv + r * 16);
          const uint32_t sbu = lds8(rsc + r * 4);
          const uint32_t row = sbase + C::OFF_B + s * C::B_STAGE + r * 128;
          const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
          if (sbu <= 128u) {
            const uint32_t c = sbu ? ((sbu + 126u) << 7) : 0u;
            const uint32_t c2 = c * 0x10001u;
#pragma unroll
            for (int q = 0; q < 4; ++q) sts128(row + (((g * 4 + q) ^ x7) << 4), dequant8(w[q], c2));
          } else {
#pragma unroll
            for (int q = 0; q < 4; ++q)
              sts128(row + (((g * 4 + q) ^ x7) << 4), dequant8_wide(w[q], sbu));
          }
          fence_proxy_async();
        }
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(BAR_B_FULL(s));
          if (b_live && ((kt & 1) || kt == KT - 1)) mbar_arrive(BAR_RAW_EMPTY(rs));
        }
      }
      if (b_live) raw_base += (uint32_t)KT_TILES;
    }
  } else {
    // ================================= epilogue =========================================================
    const int q = warp & 3;                         // tensor-memory lane quarter of this warp
    float* s_bias = reinterpret_cast<float*>(smem + C::OFF_BIAS) + q * P_TILE_N;    // private to this warp
    const bool swiglu = p.activation == MOE_ACT_SWIGLU;
    const bool y_vec = ((uintptr_t)p.y % 16 == 0) && (p.ld_y % 8 == 0);
    uint32_t tc = 0;
    bool ok = true;
    for (int64_t tile = pair; tile < n_tiles && ok; tile += n_pairs, ++tc) {
      int e; int64_t row0; int rows;
      map_tile<2>(p, s_prefix, tile / NT, e, row0, rows);
      const int n0 = (int)(tile % NT) * P_TILE_N;
      const uint32_t ab = tc & 1u;
      __syncwarp();
#pragma unroll
      for (int jb = 0; jb < P_TILE_N / 32; ++jb) {
        const int gn = n0 + jb * 32 + lane;
        s_bias[jb * 32 + lane] = (p.bias && gn < p.N) ? load_bias(p.bias, p.bias_dtype, (int64_t)e * p.ld_bias + gn) : 0.0f;
      }
      __syncwarp();
      const int r = (int)rank * HALF_M + q * 32 + lane;      // token row inside the tile
      const int64_t m = row0 + r;
      const bool row_live = r < rows;
      int64_t dst = m;
      float beta = 1.0f, gamma = 1.0f;
      if (row_live) {
        if (p.scatter_indx) dst = p.scatter_indx[m];
        if (p.betas) beta = p.betas[m];
        if (p.gammas) gamma = p.gammas[m];
      }
      const bool store_row = row_live && dst >= 0;
      TY* yrow = store_row ? gemm_out_row<TY>(p, dst) : nullptr;
      ok = __all_sync(0xFFFFFFFFu, mbar_wait(BAR_ACC_FULL(ab), (tc >> 1) & 1u, ctl, 501));
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + ab * P_ACC_COLS;
      // two register buffers: the tensor-memory load of the next 16 columns is in flight while this one is
      // turned into output
      auto emit = [&](const uint32_t (&raw)[16], int c0) {
        if (!store_row || n0 + c0 >= p.N) return;
        float v[16];
#pragma unroll
        for (int jx = 0; jx < 16; ++jx) {
          float a = __uint_as_float(raw[jx]) + s_bias[c0 + jx] * beta;
          if (p.has_out_alpha) a *= p.out_alpha;
          v[jx] = a;
        }
        const int ncols = min(16, p.N - (n0 + c0));
        if (swiglu) {
          float o[8];
#pragma unroll
          for (int jx = 0; jx < 8; ++jx)
            o[jx] = gemm_swiglu(v[2 * jx], v[2 * jx + 1], p.act_alpha, p.act_limit, p.act_has_limit) * gamma;
          store_out<TY, 8>(yrow + ((n0 + c0) >> 1), o, y_vec && ncols == 16, ncols >> 1);
        } else {
#pragma unroll
          for (int jx = 0; jx < 16; ++jx) v[jx] *= gamma;
          store_out<TY, 16>(yrow + (n0 + c0), v, y_vec && ncols == 16, ncols);
        }
      };
      uint32_t raw0[16], raw1[16];
      tmem_ld16(taddr, raw0);
#pragma unroll 1
      for (int c0 = 0; c0 < P_TILE_N; c0 += 32) {
        tmem_ld_wait();
        tmem_ld16(taddr + (uint32_t)(c0 + 16), raw1);
        emit(raw0, c0);
        tmem_ld_wait();
        if (c0 + 32 < P_TILE_N) tmem_ld16(taddr + (uint32_t)(c0 + 32), raw0);
        emit(raw1, c0 + 16);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(BAR_ACC_EMPTY(ab), 0);
    }
  }

  // ---- teardown ----------------------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                  // neither CTA's memories go away while the other still works
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

// upper bound on the number of row blocks of `block` rows (triton_kernels tensor_details/ragged_tensor.py:73-77)
int64_t n_blocks_bound_pair(int64_t n_slices, int64_t n_rows, int64_t block) {
  if (n_rows <= n_slices) return n_rows;
  const int64_t a = n_rows + 1 - n_slices;
  return n_slices - 1 + (a + block - 1) / block;
}

template <typename TY> int launch_pair(const GemmParams& p, int64_t grid_m, int64_t N, cudaStream_t st) {
  auto kernel = gemm_tc_pair_kernel<TY>;
  CUtensorMap x_map;
  if (int rc = make_x_map(p, &x_map)) return rc;
  // per device: opt in to the shared-memory size once, and ask how many pairs can be resident at a time
  static std::mutex mu;
  static int max_pairs[64] = {0};
  int dev = 0;
  MOE_CHECK_CUDA(cudaGetDevice(&dev));
  int pairs_resident;
  {
    std::lock_guard<std::mutex> lk(mu);
    if (dev < 64 && max_pairs[dev] == 0) {
      MOE_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem::ALLOC));
      cudaLaunchConfig_t q = {};
      q.gridDim = dim3(2 * (unsigned)(moe_sm_count() / 2), 1, 1);
      q.blockDim = dim3(PAIR_THREADS, 1, 1);
      q.dynamicSmemBytes = PairSmem::ALLOC;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
      q.attrs = at; q.numAttrs = 1;
      int n = 0;
      MOE_CHECK_CUDA(cudaOccupancyMaxActiveClusters(&n, kernel, &q));
      max_pairs[dev] = n > 0 ? n : -1;
    }
    pairs_resident = dev < 64 ? max_pairs[dev] : moe_sm_count() / 2;
  }
  if (pairs_resident <= 0) {
    moe_set_error("moe_grouped_gemm: no pair of SMs can hold the cluster kernel on this device");
    return MOE_ERR_UNSUPPORTED;
  }
  const int64_t tiles = grid_m * cdiv64(N, P_TILE_N);
  const int64_t pairs = tiles < pairs_resident ? tiles : pairs_resident;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
  cfg.blockDim = dim3(PAIR_THREADS, 1, 1);
  cfg.dynamicSmemBytes = PairSmem::ALLOC;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  moe_count_launch();
  MOE_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kernel, p, grid_m, x_map));
  return MOE_OK;
}

}  // namespace

bool moe_gemm_tc_pair_supported(const MoeGemmArgs& a, const char** why) {
  if (a.slice_sizes && a.E > MAX_PREFIX_EXPERTS) { *why = "more experts than the 256-row tile schedule indexes"; return false; }
  *why = "";
  return true;
}

int moe_gemm_tc_pair_launch(const GemmParams& p, const MoeGemmArgs& a, cudaStream_t st) {
  const int64_t grid_m = a.slice_sizes ? n_blocks_bound_pair(a.E, a.M, 256) : cdiv64(a.M, 256);
  if (grid_m == 0) return MOE_OK;
  if (a.y_dtype == MOE_BF16) return launch_pair<__nv_bfloat16>(p, grid_m, a.N, st);
  return launch_pair<float>(p, grid_m, a.N, st);
}
