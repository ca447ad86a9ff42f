// Ragged grouped GEMM on the 5th-generation tensor cores (tcgen05) of sm_100a:
//   bf16 activations (gathered rows) x MXFP4 weights in the tile-contiguous layout of layout.cu,
//   fp32 accumulators in tensor memory, fused bias / SwiGLU / routing-weight / scatter epilogue.
//
// No tcgen05 MMA kind multiplies bf16 by e2m1, so the weights are dequantised inside the SM to bf16
// (e2m1 x 2^e is exact in bf16) and the contraction runs as kind::f16 with bf16 operands -- the same
// arithmetic as the reference, which upcasts the weight tile in registers before its bf16 MMA
// (triton_kernels matmul_details/opt_flags_details/opt_flags_nvidia.py:154-161).
//
// One persistent CTA per SM, 18 warps, specialised:
//   warp 0       tensor-memory allocation, MMA issue (one elected lane)
//   warp 1       weight producer: one bulk copy per value tile (8 KB) and scale tile (512 B) and k step
//   warps 2-5    activation loader.  256-row tiles of consecutive token rows: one thread, one TMA tile copy
//                (128 rows x 64 k, 128-byte swizzle) per half stage.  Otherwise 16-byte cp.async of (gathered)
//                token rows into the 128B-swizzled K-major operand tile, zero fill for missing rows and the
//                K tail; the source offsets of a thread's rows stay in registers for the whole tile
//   warps 6-13   dequantiser: packed e2m1 + e8m0 -> bf16, written into the swizzled K-major B tile; a thread
//                takes the 32 k values of one (row, scale group) at a time: one 16-byte load, one scale byte
//   warps 14-17  epilogue: tcgen05.ld of the accumulator, bias*beta, out_alpha, SwiGLU, gamma, cast, store
// Tile (128 or 256 token rows) x (128 or 256 weight rows), 64 k per stage, 5, 4 or 3 stages (see Cfg).
// Rings: raw weights (producer -> dequantiser), A and B operand stages (-> MMA), one or two accumulator
// buffers (MMA -> epilogue).  Every mbarrier wait is bounded: when a wait expires the CTA raises a
// shared abort flag, writes the caller's status word, drains its copies, frees tensor memory and
// returns, so a protocol error can not hang the device.
#include "gemm_tc_common.cuh"

#ifndef MOE_STAGES_SMALL
#define MOE_STAGES_SMALL 5
#endif
#ifndef MOE_RAW_STAGES_SMALL
#define MOE_RAW_STAGES_SMALL 6
#endif

namespace {

constexpr int NUM_THREADS = 608;          // 19 warps (the register file still allows 96 registers per thread)
constexpr int LOADER_WARPS = 4, DEQUANT_WARPS = 8;
constexpr int WARP_LOADER0 = 2, WARP_DEQ0 = 6, WARP_EPI0 = 14;
// Shared-memory map for a CTA tile of (MH x 128 token rows) x (NH x 128 weight rows), 64 k per stage.
//   MH = 1, NH = 1: 6 stages, two accumulator buffers   (small problems: many CTAs, short tiles)
//   MH = 2, NH = 1: 4 stages, two accumulator buffers
//   MH = 2, NH = 2: 3 stages, one accumulator buffer    (prefill: most MMA work per pipeline hand-off)
// The MH halves of a token tile share every dequantised weight stage, the NH halves share every activation stage.
template <int MH, int NH> struct Cfg {
  static constexpr int STAGES = (MH == 1) ? MOE_STAGES_SMALL : (NH == 1 ? 4 : 3);
  // Packed weights travel in stages of RAWK 64-k steps: a whole 128-k weight tile (one 8 KB + one 512 B bulk copy)
  // when the CTA tile is one weight tile wide, so that the single producer thread spends half as many
  // operations per byte; 64 k per stage (two n halves) for the 256-wide CTA tile.
  static constexpr int RAWK = (NH == 1) ? 2 : 1;
  static constexpr int RAW_STAGES = (MH == 1) ? MOE_RAW_STAGES_SMALL : 3;
  static constexpr int ACC_BUFS = (MH * NH * 128 <= 256) ? 2 : 1;       // accumulator buffers in the 512 TMEM columns
  static constexpr int ACC_COLS = MH * NH * 128;
  static constexpr int A_STAGE_BYTES = MH * SUBTILE_BYTES;
  static constexpr int B_STAGE_BYTES = NH * SUBTILE_BYTES;
  static constexpr int RAWV_STAGE = NH * RAWV_BYTES * RAWK;
  static constexpr int RAWS_STAGE = NH * RAWS_BYTES;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + STAGES * A_STAGE_BYTES;
  static constexpr int OFF_RAWV = OFF_B + STAGES * B_STAGE_BYTES;
  static constexpr int OFF_RAWS = OFF_RAWV + RAW_STAGES * RAWV_STAGE;
  static constexpr int OFF_BIAS = OFF_RAWS + RAW_STAGES * RAWS_STAGE;   // float bias, [4 epilogue warps][NH * 128]
  static constexpr int OFF_BAR = OFF_BIAS + 4 * NH * HALF_N * 4;        // mbarriers
  static constexpr int NUM_BARS = 3 * STAGES + 2 * RAW_STAGES + 4 + 1;
  static constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;               // tmem base, abort flag
  static constexpr int OFF_PREFIX = OFF_MISC + 16;                      // MH = 2: int32 tile prefix over experts
  static constexpr int OFF_ROWS = OFF_PREFIX;                           // MH = 1: source rows, [4 loader warps][2][128]
  static constexpr int SMEM_BYTES = OFF_PREFIX + (MH == 2 ? (MAX_PREFIX_EXPERTS + 1) * 4 : 4 * 2 * 128 * 4);
  // MH = 1 interleaves pipeline steps over the warps of a role (see the loader and the dequantiser)
  static constexpr int DEQ_GROUPS = (MH == 1) ? 4 : 1;
  static constexpr int A_FULL_COUNT = (MH == 1) ? 32 : LOADER_WARPS * 32;
  static constexpr int B_FULL_COUNT = DEQUANT_WARPS / DEQ_GROUPS;
  static constexpr int RAW_EMPTY_COUNT = (DEQUANT_WARPS / DEQ_GROUPS) * ((NH == 1 && DEQ_GROUPS > 1) ? 2 : 1);
  static constexpr int SMEM_ALLOC = SMEM_BYTES + 1024;                  // slack for 1024-byte alignment
  static_assert(SMEM_ALLOC <= 232448, "shared memory budget");
};

template <typename TY, int MH, int NH>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const GemmParams p, const int64_t grid_m_static, const __grid_constant__ CUtensorMap x_map) {
  using C = Cfg<MH, NH>;
  constexpr int STAGES = C::STAGES;
  constexpr int RAW_STAGES = C::RAW_STAGES;
  constexpr int ACC_BUFS = C::ACC_BUFS;
  constexpr int B_STAGE_BYTES = C::B_STAGE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // 256-row tiles of consecutive token rows are fetched by TMA tile copies (x_map), everything else by cp.async
  const bool use_tma = MH == 2 && p.gather_indx == nullptr;
  // second epilogue group (see the epilogue role): only where the loader warps are free and the epilogue is heavy
  const int epi_groups = (use_tma && p.activation == MOE_ACT_SWIGLU) ? 2 : 1;
  const bool epi_extra = epi_groups == 2 && ((warp > WARP_LOADER0 && warp < WARP_DEQ0) || warp == WARP_EPI0 + 4);

  const uint32_t bar0 = sbase + C::OFF_BAR;
  auto BAR_RAW_FULL = [&](int s) { return bar0 + 8u * (uint32_t)s; };
  auto BAR_RAW_EMPTY = [&](int s) { return bar0 + 8u * (uint32_t)(RAW_STAGES + s); };
  auto BAR_A_FULL = [&](int s) { return bar0 + 8u * (uint32_t)(2 * RAW_STAGES + s); };
  auto BAR_B_FULL = [&](int s) { return bar0 + 8u * (uint32_t)(2 * RAW_STAGES + STAGES + s); };
  auto BAR_AB_EMPTY = [&](int s) { return bar0 + 8u * (uint32_t)(2 * RAW_STAGES + 2 * STAGES + s); };
  auto BAR_ACC_FULL = [&](int a) { return bar0 + 8u * (uint32_t)(2 * RAW_STAGES + 3 * STAGES + a); };
  auto BAR_ACC_EMPTY = [&](int a) { return bar0 + 8u * (uint32_t)(2 * RAW_STAGES + 3 * STAGES + 2 + a); };
  const uint32_t BAR_DRAIN = bar0 + 8u * (uint32_t)(2 * RAW_STAGES + 3 * STAGES + 4);

  volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(smem + C::OFF_MISC);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + C::OFF_MISC + 4);
  int32_t* s_prefix = reinterpret_cast<int32_t*>(smem + C::OFF_PREFIX);
  Ctl ctl{s_abort, p.status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < RAW_STAGES; ++s) {
      mbar_init(BAR_RAW_FULL(s), 1);
      mbar_init(BAR_RAW_EMPTY(s), C::RAW_EMPTY_COUNT);
    }
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(BAR_A_FULL(s), use_tma ? 1 : C::A_FULL_COUNT);
      mbar_init(BAR_B_FULL(s), C::B_FULL_COUNT);
      mbar_init(BAR_AB_EMPTY(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(BAR_ACC_FULL(a), 1);
      mbar_init(BAR_ACC_EMPTY(a), epi_groups * 4);
    }
    mbar_init(BAR_DRAIN, 1);
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sbase + C::OFF_MISC),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if constexpr (MH == 2) {
    // tile prefix over experts: expert e has ceil(slice_sizes[e] / 256) tiles.  (Taken from the sizes, not from
    // differences of block_offs: after an expert-parallel remap block_offs keeps global cumulative values.)
    if (p.slice_sizes != nullptr) {
      for (int e = threadIdx.x; e < p.E; e += NUM_THREADS)
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
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;

  // ---- tile schedule shared by every role -----------------------------------------------------------
  const int NT128 = (p.N + HALF_N - 1) / HALF_N;        // weight tiles along n in memory
  const int NT = (NT128 + NH - 1) / NH;                  // CTA tiles along n
  const int KT = (p.K + BLOCK_K - 1) / BLOCK_K;           // 64-k steps
  const int KT_TILES = (p.K + TILE_K - 1) / TILE_K;      // 128-k weight tiles per (expert, n tile)
  int64_t useful_m = grid_m_static;
  if (p.slice_sizes) useful_m = (MH == 2) ? (int64_t)s_prefix[p.E] : (int64_t)p.block_offs[p.E];
  const int64_t n_tiles = useful_m * NT;

  if (warp == 0) {
    // ================================= MMA issuer ===================================================
    if (lane == 0) {
      uint32_t it = 0, tc = 0;
      bool ok = true;
      for (int64_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++tc) {
        int halves = 1, rows_cur = HALF_M;
        {
          int e; int64_t row0;
          map_tile<MH>(p, s_prefix, tile / NT, e, row0, rows_cur);
          halves = (MH == 2 && rows_cur > HALF_M) ? 2 : 1;
        }
        const int nh_live = min(NH, NT128 - (int)(tile % NT) * NH);
        // MH == 1 swaps the operands: the dequantised weight tile is the M = 128 operand and the token tile the
        // N operand, with N = the tile's rows rounded up to 16, so that a tile of a few tokens costs a few columns
        // of MMA time instead of a full 128 x 128 product.  The accumulator is then [weight row][token].
        const int n_tok = max(16, (min(rows_cur, HALF_M) + 15) & ~15);
        const uint32_t idesc = make_idesc(MH == 1 ? n_tok : nh_live * HALF_N);
        const uint32_t ab = tc % ACC_BUFS;
        ok = mbar_wait(BAR_ACC_EMPTY(ab), ((tc / ACC_BUFS) & 1u) ^ 1u, ctl, 101);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + ab * C::ACC_COLS;
        for (int kt = 0; kt < KT; ++kt, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          ok = mbar_wait(BAR_A_FULL(s), ph, ctl, 102);
          ok = ok && mbar_wait(BAR_B_FULL(s), ph, ctl, 103);
          if (!ok) break;
          fence_proxy_async();          // the A tile was written by cp.async (generic proxy) of other threads
          tc_fence_after();
          const uint64_t adesc = make_desc(sbase + C::OFF_A + s * C::A_STAGE_BYTES);
          const uint64_t bdesc = make_desc(sbase + C::OFF_B + s * B_STAGE_BYTES);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            if constexpr (MH == 1)
              mma_bf16(d_tmem, bdesc + (uint64_t)(kk * 2), adesc + (uint64_t)(kk * 2), idesc, (kt | kk) ? 1u : 0u);
            else
              mma_bf16(d_tmem, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc, (kt | kk) ? 1u : 0u);
            if (MH == 2 && halves == 2)
              mma_bf16(d_tmem + NH * HALF_N, adesc + (uint64_t)((SUBTILE_BYTES >> 4) + kk * 2),
                       bdesc + (uint64_t)(kk * 2), idesc, (kt | kk) ? 1u : 0u);
          }
          mma_commit(BAR_AB_EMPTY(s));
        }
        if (ok) mma_commit(BAR_ACC_FULL(ab));
      }
      // make sure every MMA issued by this thread has retired before tensor memory is freed
      mma_commit(BAR_DRAIN);
      mbar_wait(BAR_DRAIN, 0, ctl, 104);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ================================= weight producer =================================================
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      const uint8_t* wv = (const uint8_t*)p.w;
      const uint8_t* ws = p.w_scale;
      for (int64_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        int e; int64_t row0; int rows;
        map_tile<MH>(p, s_prefix, tile / NT, e, row0, rows);     // every tile below n_tiles is a real one
        const int nt0 = (int)(tile % NT) * NH;                   // first weight tile along n
        const int nh_live = min(NH, NT128 - nt0);
        const int64_t tile0 = ((int64_t)e * NT128 + nt0) * KT_TILES;
        const uint8_t* cur_wv = wv + tile0 * (2 * RAWV_BYTES);
        const int64_t half_stride = (int64_t)KT_TILES * (2 * RAWV_BYTES);     // next weight tile along n
        constexpr int RAWK = C::RAWK;
        const int n_raw = RAWK == 2 ? KT_TILES : KT;                          // raw stages of this tile
        for (int rt = 0; rt < n_raw; ++rt, ++it) {
          const int s = it % RAW_STAGES;
          ok = mbar_wait(BAR_RAW_EMPTY(s), ((it / RAW_STAGES) & 1u) ^ 1u, ctl, 201);
          if (!ok) break;
          mbar_expect_tx(BAR_RAW_FULL(s), (uint32_t)nh_live * (RAWK * RAWV_BYTES + RAWS_BYTES));
          for (int h = 0; h < nh_live; ++h) {
            bulk_g2s(sbase + C::OFF_RAWV + s * C::RAWV_STAGE + h * (RAWK * RAWV_BYTES),
                     cur_wv + h * half_stride + (int64_t)rt * (RAWK * RAWV_BYTES), RAWK * RAWV_BYTES, BAR_RAW_FULL(s));
            bulk_g2s(sbase + C::OFF_RAWS + s * C::RAWS_STAGE + h * RAWS_BYTES,
                     ws + (tile0 + (int64_t)h * KT_TILES + (RAWK == 2 ? rt : (rt >> 1))) * RAWS_BYTES, RAWS_BYTES,
                     BAR_RAW_FULL(s));
          }
        }
      }
      if (!ok) {
        // aborting: let the copies that were already issued land before the CTA leaves
        const uint32_t lo = it > (uint32_t)RAW_STAGES ? it - RAW_STAGES : 0;
        for (uint32_t j = lo; j < it; ++j)
          for (uint32_t i = 0; i < (1u << 16) && !mbar_test(BAR_RAW_FULL(j % RAW_STAGES), (j / RAW_STAGES) & 1u); ++i) __nanosleep(64);
      }
    }
    __syncwarp();
  } else if (warp < WARP_DEQ0 && !epi_extra) {
    // ================================= activation loader ==============================================
    if constexpr (MH == 1) {
      // Small-tile variant: each of the four loader warps takes every fourth pipeline step and moves that whole
      // stage by itself, so four stages are in flight inside the role and the per-step latency of one warp
      // (barrier wake-up, address arithmetic) is hidden.  Lane l owns 16-byte chunk (l & 7) of rows (l >> 3) + 4 i.
      // Only rows that exist are copied: the MMA rows of missing tokens read whatever the stage held before,
      // which only reaches accumulator rows that are never stored.  Each warp keeps its own table of the tile's
      // source rows in shared memory (double-buffered by tile, filled one tile ahead).
      const int lw = warp - WARP_LOADER0;             // 0..3
      const int c8 = lane & 7;
      const int rq = lane >> 3;
      const uint8_t* Xb = (const uint8_t*)p.x;
      const uint32_t ld16 = (uint32_t)(p.ld_x >> 3);
      uint32_t* tab = reinterpret_cast<uint32_t*>(smem + C::OFF_ROWS) + lw * 256;
      auto fill_table = [&](int64_t tile, int buf) -> int {
        int e; int64_t row0; int rows;
        map_tile<MH>(p, s_prefix, tile / NT, e, row0, rows);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int r = lane + 32 * j;
          int64_t src = -1;
          if (r < rows) {
            const int64_t m = row0 + r;
            src = p.gather_indx ? (int64_t)p.gather_indx[m] : m;
            if (src >= p.rows_x) src = -1;
          }
          tab[buf * 128 + r] = src < 0 ? 0xFFFFFFFFu : (uint32_t)src * ld16;
        }
        return rows;
      };
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      int rows = 0, rows_next = 0;
      if ((int64_t)blockIdx.x < n_tiles) rows = fill_table(blockIdx.x, 0);
      for (int64_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++tcount) {
        const int buf = tcount & 1;
        const int64_t t2 = tile + gridDim.x;
        if (t2 < n_tiles) rows_next = fill_table(t2, buf ^ 1);
        __syncwarp();
        const uint32_t* trow = tab + buf * 128;
        for (int kt = 0; kt < KT; ++kt, ++it) {
          if ((int)(it & 3u) != lw) continue;
          const int s = it % STAGES;
          ok = __all_sync(0xFFFFFFFFu, mbar_wait(BAR_AB_EMPTY(s), ((it / STAGES) & 1u) ^ 1u, ctl, 301));
          if (!ok) break;
          const int k = kt * BLOCK_K + c8 * 8;
          const int kleft = p.K - k;
          const uint32_t kbytes = kleft >= 8 ? 16u : (kleft > 0 ? (uint32_t)kleft * 2u : 0u);
          const uint32_t stage = sbase + C::OFF_A + s * C::A_STAGE_BYTES;
          const uint32_t kc16 = (uint32_t)(k >> 3);
          for (int r = rq; r < rows; r += 4) {
            const uint32_t so = trow[r];
            const bool live = so != 0xFFFFFFFFu && kbytes;
            const uint8_t* g = live ? Xb + ((uint64_t)(so + kc16) << 4) : Xb;
            cp_async16(stage + (uint32_t)(r * 128 + ((c8 ^ (r & 7)) << 4)), g, live ? kbytes : 0u);
          }
          cp_async_arrive_noinc(BAR_A_FULL(s));
        }
        rows = rows_next;
      }
      cp_async_wait_all();
    } else if (use_tma) {
      // Consecutive token rows: one thread moves the stage with one TMA tile copy (128 rows x 64 k) per live half.
      // Rows past the end of the expert's segment belong to the next expert (or read as zeros past the end of the
      // matrix) and only reach accumulator rows that are never stored.
      if (warp == WARP_LOADER0 && lane == 0) {
        uint32_t it = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
          int e; int64_t row0; int rows;
          map_tile<MH>(p, s_prefix, tile / NT, e, row0, rows);
          const int halves = rows > HALF_M ? 2 : 1;
          for (int kt = 0; kt < KT; ++kt, ++it) {
            const int s = it % STAGES;
            ok = mbar_wait(BAR_AB_EMPTY(s), ((it / STAGES) & 1u) ^ 1u, ctl, 301);
            if (!ok) break;
            mbar_expect_tx(BAR_A_FULL(s), (uint32_t)(halves * SUBTILE_BYTES));
            for (int h = 0; h < halves; ++h)
              tma_tile_2d(sbase + C::OFF_A + s * C::A_STAGE_BYTES + h * SUBTILE_BYTES, &x_map, kt * BLOCK_K,
                          (int)row0 + h * HALF_M, BAR_A_FULL(s));
          }
        }
        if (!ok) {
          // aborting: let the copies that were already issued land before the CTA leaves
          const uint32_t lo = it > (uint32_t)STAGES ? it - STAGES : 0;
          for (uint32_t j = lo; j < it; ++j)
            for (uint32_t i = 0; i < (1u << 16) && !mbar_test(BAR_A_FULL(j % STAGES), (j / STAGES) & 1u); ++i)
              __nanosleep(64);
        }
      }
    } else {
    // 128 threads move the (MH x 128) x 128-byte stage: thread t owns 16-byte chunk (t & 7) of rows
    // (t >> 3) + 16 i.  The source of each row (byte offset / 16 into x, or none) is kept in registers for the
    // whole tile.  A stage is published by cp.async.mbarrier.arrive.noinc: the barrier completes when the
    // copies of all 128 threads have landed, and no thread ever waits for its own copies.
    constexpr int NR = 8 * MH;                      // rows per thread
    const int t = threadIdx.x - WARP_LOADER0 * 32;  // 0..127
    const int c8 = t & 7;
    const int rbase = t >> 3;
    const uint8_t* Xb = (const uint8_t*)p.x;
    const uint32_t ld16 = (uint32_t)(p.ld_x >> 3);  // row pitch in 16-byte units
    uint32_t dst_off[NR];
#pragma unroll
    for (int i = 0; i < NR; ++i) {
      const int r = rbase + 16 * i;                 // rows 128.. land in the second 16 KB sub-tile
      dst_off[i] = (uint32_t)(r * 128 + ((c8 ^ (r & 7)) << 4));
    }
    uint32_t it = 0;
    bool ok = true;
    // source rows of a tile: looked up one tile ahead, so that the dependent loads (schedule -> offsets ->
    // gather index) of the next tile fly while the current tile streams
    auto load_rows = [&](int64_t tile, uint32_t (&src16)[NR], int& nr_live) {
      int e; int64_t row0; int rows;
      map_tile<MH>(p, s_prefix, tile / NT, e, row0, rows);
      nr_live = (MH == 2 && rows > HALF_M) ? NR : 8;            // the MMA skips an empty second half
#pragma unroll
      for (int i = 0; i < NR; ++i) {
        const int r = rbase + 16 * i;
        int64_t src = -1;
        if (r < rows) {
          const int64_t m = row0 + r;
          src = p.gather_indx ? (int64_t)p.gather_indx[m] : m;
          if (src >= p.rows_x) src = -1;
        }
        src16[i] = src < 0 ? 0xFFFFFFFFu : (uint32_t)src * ld16;   // 0xFFFFFFFF: no source row
      }
    };
    uint32_t src16[NR], nxt16[NR];
    int nr_live = 8, nxt_live = 8;
    if ((int64_t)blockIdx.x < n_tiles) load_rows(blockIdx.x, src16, nr_live);
    for (int64_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
      const int64_t t2 = tile + gridDim.x;
      if (t2 < n_tiles) load_rows(t2, nxt16, nxt_live);
      for (int kt = 0; kt < KT; ++kt, ++it) {
        const int s = it % STAGES;
        ok = __all_sync(0xFFFFFFFFu, mbar_wait(BAR_AB_EMPTY(s), ((it / STAGES) & 1u) ^ 1u, ctl, 301));
        if (!ok) break;
        const int k = kt * BLOCK_K + c8 * 8;
        const int kleft = p.K - k;
        const uint32_t kbytes = kleft >= 8 ? 16u : (kleft > 0 ? (uint32_t)kleft * 2u : 0u);
        const uint32_t stage = sbase + C::OFF_A + s * C::A_STAGE_BYTES;
        const uint32_t kc16 = (uint32_t)(k >> 3);
#pragma unroll
        for (int i = 0; i < NR; ++i) {
          if (i < nr_live) {
            const bool live = src16[i] != 0xFFFFFFFFu && kbytes;
            const uint8_t* g = live ? Xb + ((uint64_t)(src16[i] + kc16) << 4) : Xb;
            cp_async16(stage + dst_off[i], g, live ? kbytes : 0u);
          }
        }
        cp_async_arrive_noinc(BAR_A_FULL(s));
      }
#pragma unroll
      for (int i = 0; i < NR; ++i) src16[i] = nxt16[i];
      nr_live = nxt_live;
    }
    cp_async_wait_all();
    }
  } else if (warp >= WARP_DEQ0 && warp < WARP_EPI0) {
    // ================================= dequantiser ======================================================
    // A unit is one (weight row, 32-k scale group): one 16-byte load, one scale byte, four 16-byte swizzled stores;
    // a stage holds 256 units per weight tile.  The eight warps work in G groups and group (step mod G) converts
    // the whole stage: G = 1 for the large tiles (all 256 threads on every stage: shortest latency per stage),
    // G = 4 for the small-tile configuration, where the hand-off latency of a stage, not the arithmetic, bounds
    // the step rate and four stages in flight hide it.  A quarter-warp holds one scale group of 8 consecutive
    // rows, which keeps the load (128 contiguous bytes) and the stores (8 distinct 16-byte columns) free of bank
    // conflicts.
    constexpr int G = C::DEQ_GROUPS;
    constexpr int WPG = DEQUANT_WARPS / G;          // warps per group
    constexpr int U = G;                            // units per thread, weight tile and stage
    constexpr int RAWK = C::RAWK;
    const int dw = warp - WARP_DEQ0;                // 0..7
    const int grp = dw / WPG, gw = dw % WPG;
    const int g = (lane >> 3) & 1;                  // scale group inside the 64-k stage
    const int r0 = gw * 16 + (lane >> 4) * 8 + (lane & 7);   // rows r0 + 16 WPG u
    const int n_raw = RAWK == 2 ? KT_TILES : KT;    // packed-weight stages per tile
    uint32_t it = 0, raw_base = 0;                  // operand-ring step; packed-weight stage of the tile's first step
    bool ok = true;
    for (int64_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, raw_base += n_raw) {
      const int nh_live = min(NH, NT128 - (int)(tile % NT) * NH);
      for (int kt = 0; kt < KT; ++kt, ++it) {
        if (G > 1 && (int)(it % G) != grp) continue;
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1u;
        const uint32_t itr = raw_base + (RAWK == 2 ? (kt >> 1) : kt);
        const int rs = itr % RAW_STAGES;
        bool got = mbar_wait(BAR_AB_EMPTY(s), ph ^ 1u, ctl, 402);
        got = got && mbar_wait(BAR_RAW_FULL(rs), (itr / RAW_STAGES) & 1u, ctl, 401);
        ok = __all_sync(0xFFFFFFFFu, got);
        if (!ok) break;
        const uint32_t half_off = (RAWK == 2 && (kt & 1)) ? RAWV_BYTES : 0;
        uint4 raw[NH][U];
        uint32_t sb[NH][U];
#pragma unroll
        for (int h = 0; h < NH; ++h) {
          if (h < nh_live) {
            const uint32_t rv = sbase + C::OFF_RAWV + rs * C::RAWV_STAGE + h * (RAWK * RAWV_BYTES) + half_off + g * HALF_N * 16;
            const uint32_t rsc = sbase + C::OFF_RAWS + rs * C::RAWS_STAGE + h * RAWS_BYTES + (kt & 1) * 2 + g;
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const int r = r0 + 16 * WPG * u;
              raw[h][u] = lds128(rv + r * 16);
              sb[h][u] = lds8(rsc + r * 4);
            }
          }
        }
#pragma unroll
        for (int h = 0; h < NH; ++h) {
          if (h < nh_live) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const int r = r0 + 16 * WPG * u;
              const int x7 = r & 7;
              const uint32_t row = sbase + C::OFF_B + s * B_STAGE_BYTES + h * SUBTILE_BYTES + r * 128;
              const uint32_t w[4] = {raw[h][u].x, raw[h][u].y, raw[h][u].z, raw[h][u].w};
              const uint32_t sbu = sb[h][u];
              if (sbu <= 128u) {
                const uint32_t c = sbu ? ((sbu + 126u) << 7) : 0u;
                const uint32_t c2 = c * 0x10001u;
#pragma unroll
                for (int q = 0; q < 4; ++q)
                  sts128(row + (((g * 4 + q) ^ x7) << 4), dequant8(w[q], c2));
              } else {
#pragma unroll
                for (int q = 0; q < 4; ++q)
                  sts128(row + (((g * 4 + q) ^ x7) << 4), dequant8_wide(w[q], sbu));
              }
            }
          }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(BAR_B_FULL(s));
          // the packed stage is released by whoever read it: with G > 1 the two halves of a 128-k stage are read by
          // two different groups (each arrives), and the lone first half at the end of an odd tile arrives twice
          if (G > 1) {
            mbar_arrive(BAR_RAW_EMPTY(rs));
            if (RAWK == 2 && kt == KT - 1 && !(kt & 1)) mbar_arrive(BAR_RAW_EMPTY(rs));
          } else if (RAWK == 1 || (kt & 1) || kt == KT - 1) {
            mbar_arrive(BAR_RAW_EMPTY(rs));
          }
        }
      }
    }
  } else if (warp < WARP_EPI0 + 4 || epi_extra) {
    // ================================= epilogue =========================================================
    // Four warps, one per tensor-memory lane quarter.  With the single-thread TMA loader and a SwiGLU epilogue (the
    // arithmetic-heavy one), the three warps the loader leaves idle and warp 18 form a second group and each group
    // drains half of the tile's columns.
    const int q = warp & 3;                         // tensor-memory lane quarter of this warp
    constexpr int TILE_N = NH * HALF_N;
    const int grp = epi_extra ? 1 : 0;
    const int cols = TILE_N / epi_groups, c_begin = grp * cols, c_end = c_begin + cols;
    float* s_bias = reinterpret_cast<float*>(smem + C::OFF_BIAS) + (grp * 4 + q) * cols;   // private to this warp
    const bool swiglu = p.activation == MOE_ACT_SWIGLU;
    const bool y_vec = ((uintptr_t)p.y % 16 == 0) && (p.ld_y % 8 == 0);
    uint32_t tc = 0;
    bool ok = true;
    for (int64_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++tc) {
      int e; int64_t row0; int rows;
      map_tile<MH>(p, s_prefix, tile / NT, e, row0, rows);
      const int halves = rows > HALF_M ? 2 : 1;
      const int n0 = (int)(tile % NT) * TILE_N;
      const uint32_t ab = tc % ACC_BUFS;
      // stage this tile's bias columns (each warp keeps its own copy: no CTA-level barrier in this role)
      __syncwarp();
      for (int jb = 0; jb < cols / 32; ++jb) {
        const int gn = n0 + c_begin + jb * 32 + lane;
        s_bias[jb * 32 + lane] = (p.bias && gn < p.N) ? load_bias(p.bias, p.bias_dtype, (int64_t)e * p.ld_bias + gn) : 0.0f;
      }
      __syncwarp();
      if constexpr (MH == 1) {
        // Transposed accumulator [weight row = lane][token = column].  Lane l of warp quarter q owns output column
        // n0 + 32 q + l; token parameters (destination row, beta, gamma) sit one token per lane and are broadcast
        // by shuffle; for SwiGLU the even lane holds the gate and the odd lane the linear half of a pair.
        const int n = n0 + q * 32 + lane;
        const float bias_n = s_bias[q * 32 + lane];
        const int n_tok = max(16, (min(rows, HALF_M) + 15) & ~15);
        ok = __all_sync(0xFFFFFFFFu, mbar_wait(BAR_ACC_FULL(ab), (tc / ACC_BUFS) & 1u, ctl, 501));
        if (!ok) break;
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + ab * C::ACC_COLS;
        for (int c0 = 0; c0 < n_tok; c0 += 32) {
          uint32_t raw[32];
          tmem_ld32(taddr + (uint32_t)c0, raw);
          tmem_ld_wait();
          // parameters of token c0 + lane
          const int tj = c0 + lane;
          TY* dst_l = nullptr;                              // output row of this lane's token (none: not stored)
          float beta_l = 1.0f, gamma_l = 1.0f;
          if (tj < rows) {
            const int64_t m = row0 + tj;
            const int64_t d = p.scatter_indx ? (int64_t)p.scatter_indx[m] : m;
            if (d >= 0) dst_l = gemm_out_row<TY>(p, d);
            if (p.betas) beta_l = p.betas[m];
            if (p.gammas) gamma_l = p.gammas[m];
          }
          const int jmax = min(32, rows - c0);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (j < jmax) {                                   // warp-uniform
              TY* yrow = (TY*)__shfl_sync(0xFFFFFFFFu, (unsigned long long)dst_l, j);
              const float beta = __shfl_sync(0xFFFFFFFFu, beta_l, j);
              const float gamma = __shfl_sync(0xFFFFFFFFu, gamma_l, j);
              float a = __uint_as_float(raw[j]) + bias_n * beta;
              if (p.has_out_alpha) a *= p.out_alpha;
              if (swiglu) {
                const float other = __shfl_xor_sync(0xFFFFFFFFu, a, 1);
                if (!(lane & 1) && yrow != nullptr && n + 1 < p.N)
                  yrow[n >> 1] =
                      from_f32<TY>(gemm_swiglu(a, other, p.act_alpha, p.act_limit, p.act_has_limit) * gamma);
              } else if (yrow != nullptr && n < p.N) {
                yrow[n] = from_f32<TY>(a * gamma);
              }
            }
          }
        }
      } else {
      ok = __all_sync(0xFFFFFFFFu, mbar_wait(BAR_ACC_FULL(ab), (tc / ACC_BUFS) & 1u, ctl, 501));
      if (!ok) break;
      tc_fence_after();
      for (int h = 0; h < halves; ++h) {
        const int r = h * HALF_M + q * 32 + lane;   // accumulator row = token row inside the tile
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
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + ab * C::ACC_COLS + h * TILE_N;
        // two register buffers: the tensor-memory load of the next 16 columns is in flight while this one is
        // turned into output
        auto emit = [&](const uint32_t (&raw)[16], int c0) {
          if (!store_row || n0 + c0 >= p.N) return;
          float v[16];
          const uint32_t bias_addr = smem_u32(s_bias) + (uint32_t)(c0 - c_begin) * 4u;
#pragma unroll
          for (int j4 = 0; j4 < 4; ++j4) {
            const uint4 b4 = lds128(bias_addr + j4 * 16);
            const float bv[4] = {__uint_as_float(b4.x), __uint_as_float(b4.y), __uint_as_float(b4.z), __uint_as_float(b4.w)};
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
              float a = __uint_as_float(raw[j4 * 4 + jj]) + bv[jj] * beta;
              if (p.has_out_alpha) a *= p.out_alpha;
              v[j4 * 4 + jj] = a;
            }
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
        tmem_ld16(taddr + (uint32_t)c_begin, raw0);
#pragma unroll 1
        for (int c0 = c_begin; c0 < c_end; c0 += 32) {
          tmem_ld_wait();
          tmem_ld16(taddr + (uint32_t)(c0 + 16), raw1);
          emit(raw0, c0);
          tmem_ld_wait();
          if (c0 + 32 < c_end) tmem_ld16(taddr + (uint32_t)(c0 + 32), raw0);
          emit(raw1, c0 + 16);
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
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

}  // namespace

bool moe_gemm_tc_supported(const MoeGemmArgs& a, const char** why) {
  if (a.w_kind != MOE_W_MX4_B200) { *why = "weights are not in the B200 tiled layout"; return false; }
  if (a.x_dtype != MOE_BF16) { *why = "activations are not bf16"; return false; }
  if (a.y_dtype != MOE_BF16 && a.y_dtype != MOE_F32) { *why = "output is neither bf16 nor fp32"; return false; }
  if ((uintptr_t)a.x % 16 != 0 || a.ld_x % 8 != 0) { *why = "activation rows are not 16-byte aligned"; return false; }
  if ((uintptr_t)a.w % 16 != 0 || (uintptr_t)a.w_scale % 16 != 0) { *why = "weights are not 16-byte aligned"; return false; }
  if ((double)a.rows_x * (double)a.ld_x * 2.0 >= 68719476736.0 * 0.99) { *why = "activations exceed 64 GB"; return false; }
  if (a.tile_m != 0 && a.tile_m != 16 && a.tile_m != 32 && a.tile_m != 64 && a.tile_m != 128 && a.tile_m != 256) {
    *why = "tile_m must be 0, 16, 32, 64, 128 or 256"; return false;
  }
  if (a.tile_n != 0 && a.tile_n != 128 && a.tile_n != 256) { *why = "tile_n must be 0, 128 or 256"; return false; }
  *why = "";
  return true;
}

// upper bound on the number of row blocks of `block` rows (triton_kernels tensor_details/ragged_tensor.py:73-77)
static int64_t n_blocks_bound(int64_t n_slices, int64_t n_rows, int64_t block) {
  if (n_rows <= n_slices) return n_rows;
  const int64_t a = n_rows + 1 - n_slices;   // -(n_slices - n_rows - 1)
  return n_slices - 1 + (a + block - 1) / block;
}

template <typename TY, int MH, int NH>
static int launch_tc(const GemmParams& p, int64_t grid_m, int64_t N, int idle_sms, cudaStream_t st) {
  const int64_t tiles = grid_m * cdiv64(N, HALF_N * NH);
  // persistent CTAs, one per SM, minus the SMs the caller keeps free for kernels of another stream (matmul_set_idle_sms)
  const int sms = max(1, moe_sm_count() - max(idle_sms, 0));
  const int grid = (int)(tiles < sms ? tiles : sms);
  MOE_CHECK_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<TY, MH, NH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      Cfg<MH, NH>::SMEM_ALLOC));
  CUtensorMap x_map;
  memset(&x_map, 0, sizeof(x_map));
  if (MH == 2 && p.gather_indx == nullptr)
    if (int rc = make_x_map(p, &x_map)) return rc;
  gemm_tc_kernel<TY, MH, NH><<<grid, NUM_THREADS, Cfg<MH, NH>::SMEM_ALLOC, st>>>(p, grid_m, x_map);
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}

template <typename TY>
static int launch_tc_shape(const GemmParams& p, int mh, int nh, int64_t grid_m, int64_t N, int idle_sms, cudaStream_t st) {
  if (mh == 2 && nh == 2) return launch_tc<TY, 2, 2>(p, grid_m, N, idle_sms, st);
  if (mh == 2) return launch_tc<TY, 2, 1>(p, grid_m, N, idle_sms, st);
  return launch_tc<TY, 1, 1>(p, grid_m, N, idle_sms, st);
}

int moe_gemm_tc_launch(const GemmParams& p_in, const MoeGemmArgs& a, cudaStream_t st) {
  GemmParams p = p_in;
  // Tile shape.  256-row token tiles halve the dequantiser work per FLOP and 256-wide weight tiles halve the
  // activation traffic and double the MMA work per pipeline hand-off.  Measured, the 256 x 256 configuration wins from
  // about a dozen rows per expert on (a tile with at most 128 rows skips its second MMA half): 64 rows per expert
  // 0.51 -> 0.31 ms, 128 rows 0.70 -> 0.36 ms for a 32-expert layer.  128 x 128 tiles remain for the few-row problems
  // the streaming kernel cannot take.
  const int64_t rows_per_expert = a.M / (a.E > 0 ? a.E : 1);
  // token tiles of 16 / 32 / 64 rows run as the 128-row configuration, whose MMA spans only the rows present (rounded
  // up to 16)
  int mh = a.tile_m == 256 ? 2 : (a.tile_m != 0 ? 1 : (rows_per_expert >= 12 ? 2 : 1));
  if (mh == 2 && a.slice_sizes && a.E > MAX_PREFIX_EXPERTS) mh = 1;
  int nh = a.tile_n == 256 ? 2 : (a.tile_n == 128 ? 1 : ((mh == 2 && a.N >= 1024) ? 2 : 1));
  if (mh == 1) nh = 1;
  int64_t grid_m;
  if (a.slice_sizes) {
    p.block_offs = a.block_offs_16 + 3 * a.ld_block_offs;      // block size 128
    p.block_sched = a.block_sched_16 + 3 * a.ld_block_sched;
    grid_m = n_blocks_bound(a.E, a.M, 128 * mh);
  } else {
    grid_m = cdiv64(a.M, 128 * mh);
  }
  if (grid_m == 0) return MOE_OK;
  if (a.y_dtype == MOE_BF16) return launch_tc_shape<__nv_bfloat16>(p, mh, nh, grid_m, a.N, a.idle_sms, st);
  return launch_tc_shape<float>(p, mh, nh, grid_m, a.N, a.idle_sms, st);
}
