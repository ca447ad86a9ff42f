// Router: logits = x @ Wg + bg on the tensor cores with the top-k selection (+ softmax over the selected logits) and
// the expert bitmatrix in the epilogue -- the logits never travel through HBM and a routing step loses a launch.
//
// The reference runs the two steps apart: `logits = matmul(x, wg, bg)` then `topk(logits, k)`
// (triton_kernels bench/bench_mlp.py:70, topk.py:25-141); the selection rule, the softmax and the bitmatrix layout
// are those of topk_details/_topk_forward.py:91-150 (largest value first, equal values to the smaller expert index).
//
// One CTA per (block of 128 tokens, slice of K).  Warp 0 streams x and Wg^T tiles (128 x 64 bf16 and E x 64 bf16, TMA,
// 128-byte swizzle) through a ring of stages, warp 1 issues tcgen05.mma.kind::f16 (M = 128 tokens, N = E experts) into
// one fp32 accumulator in tensor memory, warps 2-17 select: they spill the accumulator to shared memory and several
// threads per token row add the bias and keep the k best in registers.  With few tokens K is cut into slices so that many SMs pull the
// operands: every slice adds its partial logits into an fp32 scratch with red.global.add, and the CTA that finishes
// last for a token block (a counter per block) reads the sums back, does the selection and leaves scratch and counter
// zero, as it found them.
// Every mbarrier wait is bounded.
#include "gemm_tc_common.cuh"
#include "topk_select.cuh"

namespace {

constexpr int RT_THREADS = 576;        // warp 0 producer, 1 MMA, 2-17 selection
constexpr int RT_MAT_LD = 136;         // row pitch of the logits matrix in shared memory: 8 (mod 32) keeps the P x rows of a warp on distinct banks
constexpr int RT_STAGES_MAX = 6;
constexpr int RT_BLOCK_T = 128;

struct RouterParams {
  int64_t T;
  int E, n_mma, k, KT;            // experts, E rounded up to 16, picks per token, 64-k steps
  int splits, stages;
  int apply_softmax;
  int round_bf16;                 // logits rounded to bf16 before the selection (a bf16 router output, as the two-launch form has it)
  const void* bias; int bias_dtype;
  float* logits_out; int64_t ld_logits;
  void* vals; int vals_dtype; int64_t ld_vals;
  int16_t* indx; int64_t ld_indx;
  uint32_t* bitmatrix; int64_t bm_stride_row, bm_stride_word;
  float* acc;                     // [blocks * 128, n_mma] partial sums (splits > 1)
  int32_t* counters;              // [blocks]
  int32_t* status;
};

template <int K>
__device__ __forceinline__ void rt_store_row(const RouterParams& p, int64_t row, const TopK<K>& tk) {
  float v[K];
  int e[K];
#pragma unroll
  for (int i = 0; i < K; ++i) {
    v[i] = sel_key_float(tk.key[i]);
    e[i] = tk.idx[i];
  }
  if (p.apply_softmax) {
    const float mx = v[0];
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < K; ++i) sum += expf(v[i] - mx);
#pragma unroll
    for (int i = 0; i < K; ++i) v[i] = __fdiv_rn(expf(v[i] - mx), sum);
  }
#pragma unroll
  for (int i = 0; i < K; ++i) {
    if (p.vals_dtype == MOE_F32) ((float*)p.vals)[row * p.ld_vals + i] = v[i];
    else ((__nv_bfloat16*)p.vals)[row * p.ld_vals + i] = __float2bfloat16(v[i]);
    p.indx[row * p.ld_indx + i] = (int16_t)e[i];
  }
  const int words = (p.E + 31) >> 5;
  for (int w = 0; w < words; ++w) {
    uint32_t bits = 0;
#pragma unroll
    for (int i = 0; i < K; ++i)
      if ((e[i] >> 5) == w) bits |= 1u << (e[i] & 31);
    p.bitmatrix[row * p.bm_stride_row + (int64_t)w * p.bm_stride_word] = bits;
  }
}

template <int K>
__global__ void __launch_bounds__(RT_THREADS, 1)
router_topk_kernel(const RouterParams p, const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  __shared__ __align__(8) uint64_t bars[2 * RT_STAGES_MAX + 1];
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  __shared__ int s_last;
  __shared__ float s_bias[256];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int STAGES = p.stages;
  const uint32_t X_BYTES = RT_BLOCK_T * 128u, W_BYTES = (uint32_t)p.n_mma * 128u;
  const uint32_t stage_bytes = X_BYTES + ((W_BYTES + 1023u) & ~1023u);
  auto BAR_FULL = [&](int s) { return smem_u32(&bars[s]); };
  auto BAR_EMPTY = [&](int s) { return smem_u32(&bars[RT_STAGES_MAX + s]); };
  const uint32_t BAR_ACC = smem_u32(&bars[2 * RT_STAGES_MAX]);
  Ctl ctl{&s_abort, p.status};
  const uint32_t tmem_cols = p.n_mma <= 32 ? 32u : p.n_mma <= 64 ? 64u : p.n_mma <= 128 ? 128u : 256u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < RT_STAGES_MAX; ++s) {
      mbar_init(BAR_FULL(s), 1);
      mbar_init(BAR_EMPTY(s), 1);
    }
    mbar_init(BAR_ACC, 1);
    s_abort = 0;
    s_last = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x == 32) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&x_map) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&w_map) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;

  const int64_t blk = blockIdx.x;
  const int split = blockIdx.y;
  const int kt0 = (int)((int64_t)p.KT * split / p.splits), kt1 = (int)((int64_t)p.KT * (split + 1) / p.splits);
  const int n_steps = kt1 - kt0;

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      int it = 0;
      for (; it < n_steps && ok; ++it) {
        const int s = it % STAGES;
        ok = mbar_wait(BAR_EMPTY(s), ((it / STAGES) & 1u) ^ 1u, ctl, 801);
        if (!ok) break;
        const uint32_t st = sbase + (uint32_t)s * stage_bytes;
        mbar_expect_tx(BAR_FULL(s), X_BYTES + W_BYTES);
        // token blocks start at different k steps: CTAs that run side by side do not all ask for the same Wg tile
        const int kt = kt0 + (int)((it + blk * 5) % n_steps);
        tma_tile_2d(st, &x_map, kt * 64, (int)(blk * RT_BLOCK_T), BAR_FULL(s));
        tma_tile_2d(st + X_BYTES, &w_map, kt * 64, 0, BAR_FULL(s));
      }
      if (!ok) {
        const int lo = it > STAGES ? it - STAGES : 0;
        for (int j = lo; j < it; ++j)
          for (uint32_t i = 0; i < (1u << 16) && !mbar_test(BAR_FULL(j % STAGES), (j / STAGES) & 1u); ++i) __nanosleep(64);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      const uint32_t idesc = make_idesc(p.n_mma);
      for (int it = 0; it < n_steps && ok; ++it) {
        const int s = it % STAGES;
        ok = mbar_wait(BAR_FULL(s), (it / STAGES) & 1u, ctl, 802);
        if (!ok) break;
        tc_fence_after();
        const uint32_t st = sbase + (uint32_t)s * stage_bytes;
        const uint64_t adesc = make_desc(st), bdesc = make_desc(st + X_BYTES);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          mma_bf16(tmem, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc, (it | kk) ? 1u : 0u);
        mma_commit(BAR_EMPTY(s));
      }
      mma_commit(BAR_ACC);              // arrives when every MMA above has retired
      if (!ok) mbar_wait(BAR_ACC, 0, ctl, 803);
    }
    __syncwarp();
  } else {
    // ---- selection: 16 warps ------------------------------------------------------------------------------
    // Stage A brings the block's logits into shared memory as [expert][token row] (the operand stages are free by now):
    // from tensor memory when this CTA holds the whole sum, else each warp adds its share of the partial sums into the
    // global scratch and the CTA that arrives last copies the totals back.  Stage B: P threads per token row (adjacent
    // lanes), each walks every P-th expert with its own best-k list, the lists of a row meet by shuffles.  A single
    // thread per row spent 12 us of dependent compare-and-select chains on 128 experts.
    const int qd = warp & 3, grp = (warp - 2) >> 2;            // lane quarter of tensor memory, share of its columns
    const int sid = threadIdx.x - 64;
    const int r = qd * 32 + lane;
    // the bias once per CTA, while the main loop runs (read per logit from global memory it made the selection wait on
    // one load after the other)
    if (sid < 256) s_bias[sid] = (p.bias && sid < p.E) ? load_bias(p.bias, p.bias_dtype, sid) : 0.0f;
    mbar_wait(BAR_ACC, 0, ctl, 804);
    asm volatile("bar.sync 1, 512;" ::: "memory");
    const bool ok = *(volatile int*)&s_abort == 0;              // the same answer in all sixteen warps
    tc_fence_after();
    const uint32_t taddr = tmem + ((uint32_t)(qd * 32) << 16);
    const int rows_blk = (int)min((int64_t)RT_BLOCK_T, p.T - blk * RT_BLOCK_T);
    float* mat = reinterpret_cast<float*>(smem);
    bool finish = p.splits == 1;
    if (ok) {
      float* dst = p.acc + blk * RT_BLOCK_T * p.n_mma + r;      // scratch of a block: [expert][token row]
      for (int c0 = grp * 16; c0 < p.n_mma; c0 += 64) {
        uint32_t v[16];
        tmem_ld16(taddr + (uint32_t)c0, v);
        tmem_ld_wait();
        if (p.splits == 1) {
#pragma unroll
          for (int j = 0; j < 16; ++j) mat[(c0 + j) * RT_MAT_LD + r] = __uint_as_float(v[j]);
        } else if (r < rows_blk) {
#pragma unroll
          for (int j = 0; j < 16; ++j) atomicAdd(dst + (c0 + j) * RT_BLOCK_T, __uint_as_float(v[j]));
        }
      }
      if (p.splits > 1) {
        __threadfence();
        asm volatile("bar.sync 1, 512;" ::: "memory");
        if (sid == 0) {
          const int prev = atomicAdd(p.counters + blk, 1);
          s_last = (prev == p.splits - 1) ? 1 : 0;
          __threadfence();
        }
        asm volatile("bar.sync 1, 512;" ::: "memory");
        finish = s_last != 0;
        if (finish) {
          // the live rows only, eight independent loads per thread at a time (one after the other this copy took 8 us)
          const float* src = p.acc + blk * RT_BLOCK_T * p.n_mma;
          int lr = 0;
          while ((1 << lr) < rows_blk) ++lr;
          const int total = p.n_mma << lr;
          for (int i0 = sid; i0 < total; i0 += 512 * 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int i = i0 + u * 512;
              v[u] = i < total ? __ldcg(src + (i >> lr) * RT_BLOCK_T + (i & ((1 << lr) - 1))) : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int i = i0 + u * 512;
              if (i < total) {
                mat[(i >> lr) * RT_MAT_LD + (i & ((1 << lr) - 1))] = v[u];
                // leave the scratch as it was found: all zero
                const_cast<float*>(src)[(i >> lr) * RT_BLOCK_T + (i & ((1 << lr) - 1))] = 0.0f;
              }
            }
          }
          if (sid == 0) p.counters[blk] = 0;
        }
      }
      asm volatile("bar.sync 1, 512;" ::: "memory");
    }
    if (ok && finish) {
      // P threads per row: 4 for a full block, 8 when the block holds at most 64 rows (more threads per row would
      // spend in merge rounds what they save on the walk)
      const int lp = rows_blk <= 64 ? 3 : 2;
      const int P = 1 << lp;
      const int part = lane & (P - 1);
      const int rr = (sid >> 5) * (32 >> lp) + (lane >> lp);
      const int64_t row = blk * RT_BLOCK_T + rr;
      const bool live = rr < rows_blk;
      constexpr int NSUB = K <= 4 ? 2 : 1;
      TopK<K> sub[NSUB];
      const int rq = rr & (RT_BLOCK_T - 1);
#pragma unroll 1
      for (int e0 = part; e0 < p.E; e0 += P * NSUB * 4) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
          for (int u = 0; u < NSUB; ++u) {          // the lists alternate: independent chains side by side
            const int e = e0 + (j * NSUB + u) * P;
            if (e < p.E) {
              float x = mat[e * RT_MAT_LD + rq] + s_bias[e];
              if (p.round_bf16) x = __bfloat162float(__float2bfloat16(x));
              if (p.logits_out && live) p.logits_out[row * p.ld_logits + e] = x;
              sub[u].push(x, e);
            }
          }
        }
      }
      TopK<K> tk = sub[0];
#pragma unroll
      for (int u = 1; u < NSUB; ++u) {
#pragma unroll
        for (int i = 0; i < K; ++i) tk.push_any(sub[u].key[i], sub[u].idx[i]);
      }
      tk.merge_lanes(P);
      if (live && part == 0) rt_store_row<K>(p, row, tk);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
  }
}

int rt_make_map(const void* base, int64_t rows, int64_t K, int64_t ld, int box_rows, CUtensorMap* map) {
  static PFN_cuTensorMapEncodeTiled_v12000 encode = nullptr;
  static std::mutex mu;
  {
    std::lock_guard<std::mutex> lk(mu);
    if (!encode) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult qr;
      MOE_CHECK_CUDA(cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &fn, 12000, cudaEnableDefault, &qr));
      if (qr != cudaDriverEntryPointSuccess || !fn) {
        moe_set_error("moe_router_topk: the driver does not provide cuTensorMapEncodeTiled");
        return MOE_ERR_UNSUPPORTED;
      }
      encode = (PFN_cuTensorMapEncodeTiled_v12000)fn;
    }
  }
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    moe_set_error("moe_router_topk: cuTensorMapEncodeTiled failed with code %d (rows %lld, K %lld, pitch %lld)", (int)r,
                  (long long)rows, (long long)K, (long long)ld);
    return MOE_ERR_CUDA;
  }
  return MOE_OK;
}

struct RouterPlan {
  int64_t blocks;
  int n_mma, KT, splits, stages;
  size_t acc_off, ws_bytes;
};

RouterPlan rt_plan(int64_t T, int64_t K, int E) {
  RouterPlan pl;
  pl.blocks = cdiv64(T, RT_BLOCK_T);
  pl.n_mma = (E + 15) / 16 * 16;
  pl.KT = (int)cdiv64(K, 64);
  // few token blocks: cut K so that many SMs pull a share of the operands.  Every slice adds a full block of partial
  // logits to the scratch, so slices get longer as blocks get more: at least 2 k steps with one block, 12 from six on
  int64_t s = moe_sm_count() / (pl.blocks > 0 ? pl.blocks : 1);
  const int64_t min_steps = pl.blocks >= 6 ? 12 : 2 * pl.blocks;
  if (s > pl.KT / min_steps) s = pl.KT / min_steps;
  if (s < 1) s = 1;
  pl.splits = (int)s;
  const int stage_bytes = RT_BLOCK_T * 128 + ((pl.n_mma * 128 + 1023) & ~1023);
  int st = (200 * 1024) / stage_bytes;
  pl.stages = st > RT_STAGES_MAX ? RT_STAGES_MAX : st;
  pl.acc_off = (size_t)((pl.blocks * 4 + 255) / 256 * 256);
  pl.ws_bytes = pl.splits > 1 ? pl.acc_off + (size_t)pl.blocks * RT_BLOCK_T * pl.n_mma * 4 : 0;
  return pl;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) size_t moe_router_topk_workspace_bytes(int64_t T, int64_t K, int E) {
  if (T <= 0 || K <= 0 || E <= 0) return 0;
  return rt_plan(T, K, E).ws_bytes;
}

extern "C" __attribute__((visibility("default"))) int moe_router_topk(
    const void* x, int64_t T, int64_t K, int64_t ld_x, const void* wg_t, int64_t ld_wg, const void* bias, int bias_dtype, int E,
    int k, int apply_softmax, int round_bf16, float* logits_out, int64_t ld_logits, void* vals, int vals_dtype, int64_t ld_vals, int16_t* indx,
    int64_t ld_indx, uint32_t* bitmatrix, int64_t bm_stride_row, int64_t bm_stride_word, void* workspace, size_t workspace_bytes,
    int32_t* status, void* stream) {
  if (T == 0) return MOE_OK;
  MOE_CHECK_ARG(x && wg_t && vals && indx && bitmatrix, "moe_router_topk: NULL argument");
  MOE_CHECK_ARG(T > 0 && K > 0 && E > 0, "moe_router_topk: T, K and E must be positive");
  if (E > 256 || !(k == 1 || k == 2 || k == 4 || k == 8 || k == 16) || k > E) {
    moe_set_error("moe_router_topk: needs at most 256 experts and k in {1, 2, 4, 8, 16} (got E = %d, k = %d)", E, k);
    return MOE_ERR_UNSUPPORTED;
  }
  if (K % 8 != 0 || ld_x % 8 != 0 || ld_wg % 8 != 0 || (uintptr_t)x % 16 != 0 || (uintptr_t)wg_t % 16 != 0) {
    moe_set_error("moe_router_topk: x and Wg^T need 16-byte aligned rows (K, pitches multiples of 8 bf16)");
    return MOE_ERR_UNSUPPORTED;
  }
  MOE_CHECK_ARG(vals_dtype == MOE_F32 || vals_dtype == MOE_BF16, "moe_router_topk: values are fp32 or bf16");
  MOE_CHECK_ARG(!bias || bias_dtype == MOE_F32 || bias_dtype == MOE_BF16, "moe_router_topk: bias is fp32 or bf16");
  MOE_CHECK_ARG(T < (1ll << 31) - 256, "moe_router_topk: too many tokens");
  const RouterPlan pl = rt_plan(T, K, E);
  cudaStream_t st = (cudaStream_t)stream;
  RouterParams p;
  p.T = T; p.E = E; p.n_mma = pl.n_mma; p.k = k; p.KT = pl.KT; p.splits = pl.splits; p.stages = pl.stages;
  p.apply_softmax = apply_softmax; p.round_bf16 = round_bf16;
  p.bias = bias; p.bias_dtype = bias_dtype;
  p.logits_out = logits_out; p.ld_logits = ld_logits;
  p.vals = vals; p.vals_dtype = vals_dtype; p.ld_vals = ld_vals;
  p.indx = indx; p.ld_indx = ld_indx;
  p.bitmatrix = bitmatrix; p.bm_stride_row = bm_stride_row; p.bm_stride_word = bm_stride_word;
  p.acc = nullptr; p.counters = nullptr; p.status = status;
  if (pl.splits > 1) {
    MOE_CHECK_ARG(workspace && workspace_bytes >= pl.ws_bytes && (uintptr_t)workspace % 16 == 0,
                  "moe_router_topk: needs a 16-byte aligned workspace of moe_router_topk_workspace_bytes() = %lld bytes (got %lld)",
                  (long long)pl.ws_bytes, (long long)workspace_bytes);
    p.counters = (int32_t*)workspace;
    p.acc = (float*)((uint8_t*)workspace + pl.acc_off);
  }
  CUtensorMap x_map, w_map;
  if (int rc = rt_make_map(x, T, K, ld_x, RT_BLOCK_T, &x_map)) return rc;
  if (int rc = rt_make_map(wg_t, E, K, ld_wg, pl.n_mma, &w_map)) return rc;
  const int stage_bytes = RT_BLOCK_T * 128 + ((pl.n_mma * 128 + 1023) & ~1023);
  const int smem = pl.stages * stage_bytes + 1024;
  const dim3 grid((unsigned)pl.blocks, (unsigned)pl.splits);
#define RT_LAUNCH(KK)                                                                                                    \
  do {                                                                                                                   \
    MOE_CHECK_CUDA(cudaFuncSetAttribute(router_topk_kernel<KK>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));     \
    router_topk_kernel<KK><<<grid, RT_THREADS, smem, st>>>(p, x_map, w_map);                                             \
  } while (0)
  switch (k) {
    case 1: RT_LAUNCH(1); break;
    case 2: RT_LAUNCH(2); break;
    case 4: RT_LAUNCH(4); break;
    case 8: RT_LAUNCH(8); break;
    default: RT_LAUNCH(16); break;
  }
#undef RT_LAUNCH
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}
