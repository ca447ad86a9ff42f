// Routing kernels for sm_100a: top-k (+softmax) + expert bitmatrix, the expert histogram with the
// stable expert-major sort of the (token, slot) entries, and the ragged-segment metadata.
//
// Semantics follow triton_kernels topk_details/_topk_forward.py:15-150, tensor_details/bitmatrix.py:43-150
// and tensor_details/ragged_tensor.py:128-210, 310-381; the kernels themselves are organised
// differently (one warp per token row for the top-k; a three-pass counting sort instead of
// per-block bitonic sorts; one launch each for the ragged metadata and its remap).
#include "common.cuh"
#include "topk_select.cuh"

namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kMaxTopK = 64;

// order-preserving map float -> uint32 (larger float <=> larger key)
__device__ __forceinline__ uint32_t float_key(float f) {
  uint32_t b = __float_as_uint(f);
  return b ^ ((b & 0x80000000u) ? 0xFFFFFFFFu : 0x80000000u);
}
__device__ __forceinline__ float key_float(uint32_t k) {
  uint32_t b = k ^ ((k & 0x80000000u) ? 0x80000000u : 0xFFFFFFFFu);
  return __uint_as_float(b);
}

__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    unsigned long long other = __shfl_xor_sync(0xFFFFFFFFu, v, o);
    v = other > v ? other : v;
  }
  return v;
}

// One warp per token row.  Selection i picks the largest packed key (value key << 32 | ~index) that is
// smaller than the key picked by selection i-1, so equal values resolve to the smaller expert index and
// the k results come out sorted by (value desc, index asc).  The row is re-read from L1 for each pick.
template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) topk_kernel(
    const T* __restrict__ logits, int64_t ld_logits, int64_t T_rows, int E, int k, int apply_softmax,
    T* __restrict__ vals, int64_t ld_vals, int16_t* __restrict__ indx, int64_t ld_indx,
    uint32_t* __restrict__ bitmatrix, int64_t bm_stride_row, int64_t bm_stride_word,
    const int32_t* __restrict__ n_rows_dev, int use_provided_indx) {
  __shared__ float s_val[kWarpsPerBlock][kMaxTopK];
  __shared__ int s_idx[kWarpsPerBlock][kMaxTopK];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarpsPerBlock + warp;
  const int64_t n_rows = n_rows_dev ? (int64_t)*n_rows_dev : T_rows;
  if (row >= T_rows || row >= n_rows) return;
  const T* x = logits + row * ld_logits;

  if (use_provided_indx) {
    for (int j = lane; j < k; j += 32) {
      int e = indx[row * ld_indx + j];
      s_idx[warp][j] = e;
      s_val[warp][j] = to_f32<T>(x[e]);
    }
  } else {
    // rows of up to 256 experts are read once and kept as packed keys in registers
    constexpr int kRegKeys = 8;
    unsigned long long keys[kRegKeys];
    const bool in_regs = E <= 32 * kRegKeys;
    if (in_regs) {
#pragma unroll
      for (int u = 0; u < kRegKeys; ++u) {
        const int e = lane + 32 * u;
        keys[u] = e < E ? (((unsigned long long)float_key(to_f32<T>(x[e])) << 32) | (uint32_t)(~(uint32_t)e)) : 0ull;
      }
    }
    unsigned long long prev = ~0ull;
    for (int j = 0; j < k; ++j) {
      unsigned long long best = 0ull;
      if (in_regs) {
#pragma unroll
        for (int u = 0; u < kRegKeys; ++u)
          if (keys[u] < prev && keys[u] > best) best = keys[u];
      } else {
        for (int e = lane; e < E; e += 32) {
          unsigned long long key = ((unsigned long long)float_key(to_f32<T>(x[e])) << 32) | (uint32_t)(~(uint32_t)e);
          if (key < prev && key > best) best = key;
        }
      }
      best = warp_max_u64(best);
      prev = best;
      if (lane == 0) {
        s_idx[warp][j] = (int)(~(uint32_t)(best & 0xFFFFFFFFull));
        s_val[warp][j] = key_float((uint32_t)(best >> 32));
      }
    }
  }
  __syncwarp();

  if (apply_softmax) {
    float mx = -INFINITY;
    for (int j = 0; j < k; ++j) mx = fmaxf(mx, s_val[warp][j]);
    float sum = 0.0f;
    for (int j = 0; j < k; ++j) sum += expf(s_val[warp][j] - mx);
    for (int j = lane; j < k; j += 32) vals[row * ld_vals + j] = from_f32<T>(__fdiv_rn(expf(s_val[warp][j] - mx), sum));
  } else {
    for (int j = lane; j < k; j += 32) vals[row * ld_vals + j] = from_f32<T>(s_val[warp][j]);
  }
  if (!use_provided_indx)
    for (int j = lane; j < k; j += 32) indx[row * ld_indx + j] = (int16_t)s_idx[warp][j];

  const int words = (E + 31) >> 5;
  for (int w = lane; w < words; w += 32) {
    uint32_t bits = 0;
    for (int j = 0; j < k; ++j) {
      int e = s_idx[warp][j];
      if ((e >> 5) == w) bits |= 1u << (e & 31);
    }
    bitmatrix[row * bm_stride_row + (int64_t)w * bm_stride_word] = bits;
  }
}

// Four lanes per token row (k in {1, 2, 4, 8, 16}, every row valid, no provided indices).  Lane `part` of a row's four
// walks the chunks of four experts c = part, part + 4, ... with best-k lists in registers (two lists side by side for
// k <= 4: independent insertion chains), the four lanes' lists meet by shuffles, lane 0 writes values and indices and the
// four lanes share the bitmatrix words.  With HIST the block (256 rows) also counts its picks per expert into
// partial[block][e], the first pass of the expert sort.  The warp-per-row kernel above spends its time in k rounds of
// 64-bit warp reductions per row: 19.6 us for 16384 x 128 logits against about 5 us here.
template <typename T, int K>
__device__ __forceinline__ TopK<K> quad_select(const T* __restrict__ x, int E, int part) {
  constexpr int NL = K <= 4 ? 2 : 1;
  TopK<K> sub[NL];
  for (int c0 = part; c0 * 4 < E; c0 += 4 * NL) {
    float v[NL][4];
#pragma unroll
    for (int u = 0; u < NL; ++u)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int e = (c0 + 4 * u) * 4 + i;
        v[u][i] = e < E ? to_f32<T>(x[e]) : 0.0f;
      }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int u = 0; u < NL; ++u) {               // the lists alternate; each takes its experts in ascending order
        const int e = (c0 + 4 * u) * 4 + i;
        if (e < E) sub[u].push(v[u][i], e);
      }
  }
  TopK<K> tk = sub[0];
#pragma unroll
  for (int u = 1; u < NL; ++u)
#pragma unroll
    for (int i = 0; i < K; ++i) tk.push_any(sub[u].key[i], sub[u].idx[i]);
  tk.merge_lanes(4);
  return tk;
}

// values (softmax over the picks), indices, bitmatrix words of one row; `hist` (shared memory, may be NULL) counts the picks
template <typename T, int K>
__device__ __forceinline__ void quad_store(const TopK<K>& tk, int part, int64_t row, int E, int apply_softmax, T* __restrict__ vals,
                                           int64_t ld_vals, int16_t* __restrict__ indx, int64_t ld_indx,
                                           uint32_t* __restrict__ bitmatrix, int64_t bm_stride_row, int64_t bm_stride_word,
                                           int32_t* hist) {
  if (part == 0) {
    float v[K];
#pragma unroll
    for (int i = 0; i < K; ++i) v[i] = sel_key_float(tk.key[i]);
    if (apply_softmax) {
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < K; ++i) mx = fmaxf(mx, v[i]);
      float sum = 0.0f;
#pragma unroll
      for (int i = 0; i < K; ++i) sum += expf(v[i] - mx);
#pragma unroll
      for (int i = 0; i < K; ++i) v[i] = __fdiv_rn(expf(v[i] - mx), sum);
    }
#pragma unroll
    for (int i = 0; i < K; ++i) {
      vals[row * ld_vals + i] = from_f32<T>(v[i]);
      indx[row * ld_indx + i] = (int16_t)tk.idx[i];
      if (hist) atomicAdd(&hist[tk.idx[i]], 1);
    }
  }
  const int words = (E + 31) >> 5;
  for (int w = part; w < words; w += 4) {
    uint32_t bits = 0;
#pragma unroll
    for (int i = 0; i < K; ++i)
      if ((tk.idx[i] >> 5) == w) bits |= 1u << (tk.idx[i] & 31);
    bitmatrix[row * bm_stride_row + (int64_t)w * bm_stride_word] = bits;
  }
}

template <typename T, int K, bool HIST>
__global__ void __launch_bounds__(HIST ? 1024 : 256) topk_quad_kernel(
    const T* __restrict__ logits, int64_t ld_logits, int64_t T_rows, int E, int apply_softmax, T* __restrict__ vals,
    int64_t ld_vals, int16_t* __restrict__ indx, int64_t ld_indx, uint32_t* __restrict__ bitmatrix, int64_t bm_stride_row,
    int64_t bm_stride_word, int32_t* __restrict__ partial) {
  extern __shared__ int32_t s_hist[];                     // [E] with HIST
  if constexpr (HIST) {
    for (int e = threadIdx.x; e < E; e += blockDim.x) s_hist[e] = 0;
    __syncthreads();
  }
  const int part = threadIdx.x & 3;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 2) + (threadIdx.x >> 2);
  const bool live = row < T_rows;
  const T* x = logits + (live ? row : 0) * ld_logits;      // rows past the end walk row 0 and store nothing
  const TopK<K> tk = quad_select<T, K>(x, E, part);
  if (live)
    quad_store<T, K>(tk, part, row, E, apply_softmax, vals, ld_vals, indx, ld_indx, bitmatrix, bm_stride_row, bm_stride_word,
                     HIST ? s_hist : nullptr);
  if constexpr (HIST) {
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) partial[(int64_t)blockIdx.x * E + e] = s_hist[e];
  }
}

// ---------------------------------------------------------------------------------------------------
// Expert histogram + stable expert-major sort.  Flat entry i = token * k + slot, expert c = indx[i]
// (negative, or token >= n_rows: dropped).  row_sorted[i] = col_offs[c] + #{j < i : indx[j] == c},
// col_sorted = inverse permutation; both -1 padded.
//   pass 1: per block of kTokPerBlock tokens, a shared-memory histogram -> partial[blk][e]; global
//           histogram by atomics; both index arrays pre-filled with -1.
//   pass 2: exclusive scan of partial[.][e] over blocks, exclusive scan of col_sum -> col_offs.
//   pass 3: rank inside the block: each warp owns 32 consecutive tokens and ranks them in order with
//           warp match, on top of the counts of the warps before it.
constexpr int kTokPerBlock = 256;

__device__ __forceinline__ int entry_expert(const int16_t* indx, int64_t ld_indx, int k, int64_t token, int slot,
                                            int64_t n_rows, int E) {
  if (token >= n_rows) return -1;
  int c = indx[token * ld_indx + slot];
  return (c < 0 || c >= E) ? -1 : c;
}

__global__ void __launch_bounds__(256) bm_hist_kernel(const int16_t* __restrict__ indx, int64_t ld_indx, int64_t T_rows,
                                                      int E, int k, const int32_t* __restrict__ n_rows_dev,
                                                      int32_t* __restrict__ col_sum, int32_t* __restrict__ partial,
                                                      int32_t* __restrict__ col_sorted, int32_t* __restrict__ row_sorted) {
  extern __shared__ int32_t s_cnt[];
  const int64_t n_rows = n_rows_dev ? min((int64_t)*n_rows_dev, T_rows) : T_rows;
  for (int e = threadIdx.x; e < E; e += blockDim.x) s_cnt[e] = 0;
  __syncthreads();
  const int64_t tok0 = (int64_t)blockIdx.x * kTokPerBlock;
  const int64_t n_ent = (int64_t)kTokPerBlock * k;
  for (int64_t j = threadIdx.x; j < n_ent; j += blockDim.x) {
    const int64_t token = tok0 + j / k;
    if (token >= T_rows) break;
    const int slot = (int)(j % k);
    const int64_t flat = token * k + slot;
    col_sorted[flat] = -1;
    row_sorted[flat] = -1;
    int c = entry_expert(indx, ld_indx, k, token, slot, n_rows, E);
    if (c >= 0) atomicAdd(&s_cnt[c], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int v = s_cnt[e];
    partial[(int64_t)blockIdx.x * E + e] = v;
    if (v) atomicAdd(&col_sum[e], v);
  }
}

// block-wide exclusive scan of `n` ints (in place allowed), returns nothing; one block only.
__device__ void block_exclusive_scan(const int32_t* in, int32_t* out, int n, int32_t* s_warp /*[33]*/) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  int carry = 0;
  for (int base = 0; base < n; base += blockDim.x) {
    int i = base + threadIdx.x;
    int v = (i < n) ? in[i] : 0;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
      if (lane >= o) inc += t;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      int w = (lane < nwarps) ? s_warp[lane] : 0;
      int winc = w;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int t = __shfl_up_sync(0xFFFFFFFFu, winc, o);
        if (lane >= o) winc += t;
      }
      s_warp[lane] = winc - w;          // exclusive warp offsets
      if (lane == 31) s_warp[32] = winc;  // chunk total
    }
    __syncthreads();
    if (i < n) out[i] = carry + s_warp[warp] + inc - v;
    carry += s_warp[32];
    __syncthreads();
  }
}

__global__ void __launch_bounds__(1024) bm_scan_kernel(int32_t* __restrict__ partial, int64_t n_blocks, int E,
                                                       const int32_t* __restrict__ col_sum,
                                                       int32_t* __restrict__ col_offs) {
  __shared__ int32_t s_warp[33];
  if (blockIdx.x == 0) {
    block_exclusive_scan(col_sum, col_offs, E, s_warp);
    return;
  }
  // remaining blocks: one thread per expert walks the blocks of tokens
  const int e = (blockIdx.x - 1) * blockDim.x + threadIdx.x;
  if (e >= E) return;
  // sixteen loads in flight per thread: the walk is a chain of L2 round trips otherwise
  int run = 0;
  for (int64_t b0 = 0; b0 < n_blocks; b0 += 16) {
    int v[16];
#pragma unroll
    for (int u = 0; u < 16; ++u) v[u] = b0 + u < n_blocks ? partial[(b0 + u) * E + e] : 0;
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      if (b0 + u < n_blocks) partial[(b0 + u) * E + e] = run;
      run += v[u];
    }
  }
}

// Positions of the entries of one block of blockDim.x tokens starting at token `tok_base`: `base[e]` is where the
// block's entries of expert e start (expert offset + entries of earlier blocks); s_cnt holds [warps][E] counters.
__device__ __forceinline__ void rank_block(const int16_t* __restrict__ indx, int64_t ld_indx, int64_t T_rows, int E, int k,
                                           int64_t n_rows, const int32_t* base_a, const int32_t* base_b, int64_t tok_base,
                                           int32_t* __restrict__ col_sorted, int32_t* __restrict__ row_sorted, int32_t* s_cnt) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  int32_t* my = s_cnt + (int64_t)warp * E;
  for (int i = threadIdx.x; i < nwarps * E; i += blockDim.x) s_cnt[i] = 0;
  __syncthreads();
  const int64_t tok0 = tok_base + warp * 32;
  const int n_ent = 32 * k;
  // count the entries of this warp's 32 tokens
  for (int j = lane; j < n_ent; j += 32) {
    int c = entry_expert(indx, ld_indx, k, tok0 + j / k, j % k, n_rows, E);
    if (c >= 0) atomicAdd(&my[c], 1);
  }
  __syncthreads();
  // turn the per-warp counts into starting offsets: base + counts of the warps before this one
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = (base_a ? base_a[e] : 0) + base_b[e];
    for (int w = 0; w < nwarps; ++w) {
      int v = s_cnt[w * E + e];
      s_cnt[w * E + e] = run;
      run += v;
    }
  }
  __syncthreads();
  // rank in order, 32 entries at a time
  for (int j0 = 0; j0 < n_ent; j0 += 32) {
    const int j = j0 + lane;
    const int64_t token = tok0 + j / k;
    const int slot = j % k;
    int c = (j < n_ent && token < T_rows) ? entry_expert(indx, ld_indx, k, token, slot, n_rows, E) : -1;
    const unsigned peers = __match_any_sync(0xFFFFFFFFu, c);
    const int before = __popc(peers & ((1u << lane) - 1u));
    int base = 0;
    if (c >= 0) base = my[c];
    __syncwarp();
    if (c >= 0 && before == 0) my[c] = base + __popc(peers);
    __syncwarp();
    if (c >= 0) {
      const int pos = base + before;
      const int64_t flat = token * k + slot;
      row_sorted[flat] = pos;
      col_sorted[pos] = (int32_t)flat;
    }
  }
}

__global__ void __launch_bounds__(256) bm_rank_kernel(const int16_t* __restrict__ indx, int64_t ld_indx, int64_t T_rows,
                                                      int E, int k, const int32_t* __restrict__ n_rows_dev,
                                                      const int32_t* __restrict__ partial,
                                                      const int32_t* __restrict__ col_offs,
                                                      int32_t* __restrict__ col_sorted, int32_t* __restrict__ row_sorted) {
  extern __shared__ int32_t s_cnt[];  // [warps][E]; a block covers blockDim.x tokens, the blocks of `partial`
  const int64_t n_rows = n_rows_dev ? min((int64_t)*n_rows_dev, T_rows) : T_rows;
  rank_block(indx, ld_indx, T_rows, E, k, n_rows, partial + (int64_t)blockIdx.x * E, col_offs, (int64_t)blockIdx.x * blockDim.x,
             col_sorted, row_sorted, s_cnt);
}

// ---------------------------------------------------------------------------------------------------
// Ragged metadata.  blockIdx.x = 0: slice_offs (block size 1); 1..4: block sizes 16,32,64,128.
// Every block scans its own offsets into shared memory; blockIdx.y == 0 writes them out; all blocks of
// a row fill their chunk of the schedule by binary search: sched[p] = ((p - offs[e]) << 16) | e.
constexpr int kSchedChunk = 4096;

__global__ void __launch_bounds__(1024) ragged_kernel(const int32_t* __restrict__ slice_sizes, int E,
                                                      int32_t* __restrict__ slice_offs, int32_t* __restrict__ block_offs,
                                                      int64_t ld_block_offs, int32_t* __restrict__ block_sched,
                                                      int64_t ld_sched, int64_t n_sched) {
  extern __shared__ int32_t s_offs[];  // [E + 1] then scratch [E + 1]
  __shared__ int32_t s_warp[33];
  const int row = blockIdx.x;                     // 0 = slice_offs
  const int log2bs = row == 0 ? 0 : row + 3;
  int32_t* s_nb = s_offs + (E + 1);
  for (int e = threadIdx.x; e <= E; e += blockDim.x)
    s_nb[e] = (e < E) ? (int32_t)(((int64_t)max(slice_sizes[e], 0) + ((1 << log2bs) - 1)) >> log2bs) : 0;
  __syncthreads();
  block_exclusive_scan(s_nb, s_offs, E + 1, s_warp);
  __syncthreads();
  int32_t* dst = row == 0 ? slice_offs : block_offs + (int64_t)(row - 1) * ld_block_offs;
  if (blockIdx.y == 0)
    for (int e = threadIdx.x; e <= E; e += blockDim.x) dst[e] = s_offs[e];
  if (row == 0) return;
  const int32_t total = s_offs[E];
  int32_t* sched = block_sched + (int64_t)(row - 1) * ld_sched;
  const int64_t p0 = (int64_t)blockIdx.y * kSchedChunk;
  for (int64_t p = p0 + threadIdx.x; p < min(p0 + kSchedChunk, n_sched); p += blockDim.x) {
    int32_t v = -1;
    if (p < total) {
      int lo = 0, hi = E;  // largest e with offs[e] <= p
      while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (s_offs[mid] <= p) lo = mid; else hi = mid;
      }
      v = (int32_t)(((uint32_t)(p - s_offs[lo]) << 16) | (uint32_t)lo);
    }
    sched[p] = v;
  }
}

// Stable compaction by one block: out[rank(i)] = val(i) for kept i, tail filled with -1. Returns the count.
template <typename ValFn, typename KeepFn>
__device__ int block_compact(int32_t* out, int64_t n, ValFn val, KeepFn keep, int32_t* s_warp) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  int carry = 0;
  for (int64_t base = 0; base < n; base += blockDim.x) {
    const int64_t i = base + threadIdx.x;
    const bool kp = (i < n) && keep(i);
    const unsigned m = __ballot_sync(0xFFFFFFFFu, kp);
    if (lane == 0) s_warp[warp] = __popc(m);
    __syncthreads();
    int off = 0, tot = 0;
    for (int w = 0; w < nwarps; ++w) {
      int c = s_warp[w];
      if (w < warp) off += c;
      tot += c;
    }
    if (kp) out[carry + off + __popc(m & ((1u << lane) - 1u))] = val(i);
    carry += tot;
    __syncthreads();
  }
  for (int64_t i = carry + threadIdx.x; i < n; i += blockDim.x) out[i] = -1;
  return carry;
}

__global__ void __launch_bounds__(1024) ragged_remap_kernel(
    const int32_t* __restrict__ slice_sizes, const int32_t* __restrict__ slice_offs,
    const int32_t* __restrict__ block_offs, int64_t ld_block_offs, const int32_t* __restrict__ block_sched,
    int64_t ld_sched, int64_t n_sched, const int32_t* __restrict__ slice_map, int E, int32_t* __restrict__ o_sizes,
    int32_t* __restrict__ o_offs, int32_t* __restrict__ o_block_offs, int32_t* __restrict__ o_sched) {
  __shared__ int32_t s_warp[32];
  const int b = blockIdx.x;
  auto keep_slice = [&](int64_t i) { return i < E && slice_map[i] != -1; };
  if (b == 0) {
    block_compact(o_sizes, E, [&](int64_t i) { return slice_sizes[i]; }, keep_slice, s_warp);
    __syncthreads();
    block_compact(o_offs, E + 1, [&](int64_t i) { return slice_offs[i]; }, keep_slice, s_warp);
    __syncthreads();
  }
  const int32_t* bo = block_offs + (int64_t)b * ld_block_offs;
  const int32_t* bs = block_sched + (int64_t)b * ld_sched;
  int32_t* obo = o_block_offs + (int64_t)b * ld_block_offs;
  int32_t* obs = o_sched + (int64_t)b * ld_sched;
  const int n_kept = block_compact(obo, E + 1, [&](int64_t i) { return bo[i]; }, keep_slice, s_warp);
  __syncthreads();
  const int n_blk = block_compact(
      obs, n_sched,
      [&](int64_t i) {
        uint32_t v = (uint32_t)bs[i];
        return (int32_t)((v & 0xFFFF0000u) | (uint32_t)slice_map[v & 0xFFFFu]);
      },
      [&](int64_t i) {
        uint32_t v = (uint32_t)bs[i];
        uint32_t s = v & 0xFFFFu;
        return s != 0xFFFFu && (int)s < E && slice_map[s] != -1;
      },
      s_warp);
  __syncthreads();
  if (threadIdx.x == 0) obo[n_kept] = n_blk;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) int moe_topk_fwd(const void* logits, int dtype, int64_t T, int E, int k, int apply_softmax,
                            int64_t ld_logits, void* vals, int64_t ld_vals, int16_t* indx, int64_t ld_indx,
                            uint32_t* bitmatrix, int64_t bm_stride_row, int64_t bm_stride_word,
                            const int32_t* n_rows_dev, int use_provided_indx, void* stream) {
  MOE_CHECK_ARG(T >= 0 && E > 0 && E < 32768, "moe_topk_fwd: need 0 < n_expts < 32768, got %d", E);
  MOE_CHECK_ARG(k > 0 && k <= kMaxTopK && k <= E, "moe_topk_fwd: need 0 < k <= min(%d, n_expts), got %d", kMaxTopK, k);
  if (T == 0) return MOE_OK;
  MOE_CHECK_ARG(logits && vals && indx && bitmatrix, "moe_topk_fwd: NULL pointer");
  cudaStream_t st = (cudaStream_t)stream;
  if (!use_provided_indx && n_rows_dev == nullptr && (k == 1 || k == 2 || k == 4 || k == 8 || k == 16)) {
    const int qgrid = (int)cdiv64(T, 64);
#define MOE_TOPK_QUAD(KK)                                                                                                 \
  MOE_DISPATCH_FLOAT(dtype, Tv, {                                                                                         \
    topk_quad_kernel<Tv, KK, false><<<qgrid, 256, 0, st>>>((const Tv*)logits, ld_logits, T, E, apply_softmax, (Tv*)vals,   \
                                                           ld_vals, indx, ld_indx, bitmatrix, bm_stride_row,               \
                                                           bm_stride_word, nullptr);                                       \
  })
    switch (k) {
      case 1: MOE_TOPK_QUAD(1); break;
      case 2: MOE_TOPK_QUAD(2); break;
      case 4: MOE_TOPK_QUAD(4); break;
      case 8: MOE_TOPK_QUAD(8); break;
      default: MOE_TOPK_QUAD(16); break;
    }
#undef MOE_TOPK_QUAD
    MOE_CHECK_LAUNCH();
    return MOE_OK;
  }
  const int grid = (int)cdiv64(T, kWarpsPerBlock);
  MOE_DISPATCH_FLOAT(dtype, Tv, {
    topk_kernel<Tv><<<grid, kWarpsPerBlock * 32, 0, st>>>((const Tv*)logits, ld_logits, T, E, k, apply_softmax,
                                                          (Tv*)vals, ld_vals, indx, ld_indx, bitmatrix, bm_stride_row,
                                                          bm_stride_word, n_rows_dev, use_provided_indx);
  });
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}

extern "C" __attribute__((visibility("default"))) size_t moe_bitmatrix_metadata_workspace(int64_t T, int E, int k) {
  (void)k;
  const int64_t nb = cdiv64(T > 0 ? T : 1, kTokPerBlock);
  return (size_t)((nb * E + E) * (int64_t)sizeof(int32_t));
}

extern "C" __attribute__((visibility("default"))) int moe_bitmatrix_metadata(const int16_t* indx, int64_t ld_indx, int64_t T, int E, int k,
                                      const int32_t* n_rows_dev, int32_t* col_sum, int32_t* col_sorted,
                                      int32_t* row_sorted, void* workspace, size_t workspace_bytes, void* stream) {
  MOE_CHECK_ARG(T >= 0 && E > 0 && k > 0, "moe_bitmatrix_metadata: bad extents T=%lld E=%d k=%d", (long long)T, E, k);
  MOE_CHECK_ARG(col_sum, "moe_bitmatrix_metadata: col_sum is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  MOE_CHECK_CUDA(cudaMemsetAsync(col_sum, 0, sizeof(int32_t) * (size_t)E, st));
  if (T == 0) return MOE_OK;
  MOE_CHECK_ARG(indx && col_sorted && row_sorted && workspace, "moe_bitmatrix_metadata: NULL pointer");
  MOE_CHECK_ARG(workspace_bytes >= moe_bitmatrix_metadata_workspace(T, E, k),
                "moe_bitmatrix_metadata: workspace too small (%zu < %zu)", workspace_bytes,
                moe_bitmatrix_metadata_workspace(T, E, k));
  const size_t smem_rank = (size_t)8 * E * sizeof(int32_t);
  MOE_CHECK_ARG(smem_rank <= 200 * 1024, "moe_bitmatrix_metadata: n_expts=%d too large for the shared-memory counters", E);
  const int64_t nb = cdiv64(T, kTokPerBlock);
  int32_t* partial = (int32_t*)workspace;
  int32_t* col_offs = partial + nb * E;
  bm_hist_kernel<<<(int)nb, 256, (size_t)E * sizeof(int32_t), st>>>(indx, ld_indx, T, E, k, n_rows_dev, col_sum, partial,
                                                                  col_sorted, row_sorted);
  MOE_CHECK_LAUNCH();
  bm_scan_kernel<<<1 + (int)cdiv64(E, 1024), 1024, 0, st>>>(partial, nb, E, col_sum, col_offs);
  MOE_CHECK_LAUNCH();
  if (smem_rank > 48 * 1024)
    MOE_CHECK_CUDA(cudaFuncSetAttribute(bm_rank_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_rank));
  bm_rank_kernel<<<(int)nb, 256, smem_rank, st>>>(indx, ld_indx, T, E, k, n_rows_dev, partial, col_offs, col_sorted,
                                                  row_sorted);
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}

extern "C" __attribute__((visibility("default"))) int moe_ragged_metadata(const int32_t* slice_sizes, int E, int32_t* slice_offs, int32_t* block_offs,
                                   int64_t ld_block_offs, int32_t* block_sched, int64_t ld_sched, int64_t n_sched,
                                   void* stream) {
  MOE_CHECK_ARG(E > 0 && E < 65535, "moe_ragged_metadata: need 0 < n_slices < 65535, got %d", E);
  MOE_CHECK_ARG(slice_sizes && slice_offs && block_offs && (block_sched || n_sched == 0), "moe_ragged_metadata: NULL pointer");
  MOE_CHECK_ARG(ld_block_offs >= E + 1 && ld_sched >= n_sched, "moe_ragged_metadata: leading dimensions too small");
  const size_t smem = (size_t)2 * (E + 1) * sizeof(int32_t);
  cudaStream_t st = (cudaStream_t)stream;
  if (smem > 48 * 1024)
    MOE_CHECK_CUDA(cudaFuncSetAttribute(ragged_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(5, (unsigned)(n_sched > 0 ? cdiv64(n_sched, kSchedChunk) : 1));
  ragged_kernel<<<grid, 1024, smem, st>>>(slice_sizes, E, slice_offs, block_offs, ld_block_offs, block_sched, ld_sched,
                                          n_sched);
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}

extern "C" __attribute__((visibility("default"))) int moe_ragged_metadata_remap(const int32_t* slice_sizes, const int32_t* slice_offs,
                                         const int32_t* block_offs, int64_t ld_block_offs, const int32_t* block_sched,
                                         int64_t ld_sched, int64_t n_sched, const int32_t* slice_map, int E,
                                         int32_t* out_slice_sizes, int32_t* out_slice_offs, int32_t* out_block_offs,
                                         int32_t* out_block_sched, void* stream) {
  MOE_CHECK_ARG(E > 0 && E < 65535, "moe_ragged_metadata_remap: need 0 < n_slices < 65535, got %d", E);
  MOE_CHECK_ARG(slice_sizes && slice_offs && block_offs && slice_map && out_slice_sizes && out_slice_offs &&
                    out_block_offs && (n_sched == 0 || (block_sched && out_block_sched)),
                "moe_ragged_metadata_remap: NULL pointer");
  ragged_remap_kernel<<<4, 1024, 0, (cudaStream_t)stream>>>(slice_sizes, slice_offs, block_offs, ld_block_offs,
                                                            block_sched, ld_sched, n_sched, slice_map, E,
                                                            out_slice_sizes, out_slice_offs, out_block_offs,
                                                            out_block_sched);
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}

// ---------------------------------------------------------------------------------------------------------
// moe_route: the whole routing step in three launches (the standalone entry points above take five); batches of up to
// 256 tokens in one launch of five independent blocks (route_small_kernel, at the end of this section).
//   A  topk_quad_kernel<HIST>   top-k + softmax + bitmatrix row of every token, and the expert histogram of each block
//      (route_topk_hist_kernel  of 128 tokens (partial[blk][e]) in the same pass over the logits;
//       for other k)
//   B  route_scan_ragged_kernel six blocks: exclusive scan of partial over the blocks and the expert totals (col_sum);
//                               their exclusive scan (col_offs = slice_offs); block_offs and block schedules of the four
//                               block sizes of the ragged metadata, which depend on the totals only;
//   C  bm_rank_kernel           positions of the entries (unchanged).
// Every token row is valid in this form (no device-side row bound, no provided indices), so each (token, slot) entry
// receives a position and the index arrays need no -1 pre-fill.
namespace {

constexpr int kRouteTokPerBlock = 128;          // tokens per block of kernels A and C: 128 blocks for 16384 tokens
constexpr int kRouteWarps = 16;                 // warps per block of the warp-per-row form of kernel A: 8 token rows each
constexpr int kRowsPerWarp = kRouteTokPerBlock / kRouteWarps;

// One warp per token row, rows of up to 256 experts held as order-preserving keys in registers.  A pick is two warp
// reductions (redux.sync): the largest value key, then the smallest expert index among the lanes that hold it.
template <typename T>
__global__ void __launch_bounds__(kRouteWarps * 32) route_topk_hist_kernel(
    const T* __restrict__ logits, int64_t ld_logits, int64_t T_rows, int E, int k, int apply_softmax,
    T* __restrict__ vals, int64_t ld_vals, int16_t* __restrict__ indx, int64_t ld_indx,
    uint32_t* __restrict__ bitmatrix, int64_t bm_stride_row, int64_t bm_stride_word, int32_t* __restrict__ partial) {
  extern __shared__ int32_t s_hist[];                     // [E]
  __shared__ float s_val[kRouteWarps][kMaxTopK];
  __shared__ int s_idx[kRouteWarps][kMaxTopK];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = threadIdx.x; e < E; e += blockDim.x) s_hist[e] = 0;
  __syncthreads();
  constexpr int kRegKeys = 8;
  const int64_t row0 = (int64_t)blockIdx.x * kRouteTokPerBlock + warp * kRowsPerWarp;
  const int words = (E + 31) >> 5;
  // the next row's logits are loaded before this row's picks start
  uint32_t nxt[kRegKeys];
  auto load_row = [&](int64_t row) {
#pragma unroll
    for (int u = 0; u < kRegKeys; ++u) {
      const int e = lane + 32 * u;
      nxt[u] = (row < T_rows && e < E) ? float_key(to_f32<T>(logits[row * ld_logits + e])) : 0u;
    }
  };
  load_row(row0);
  for (int i = 0; i < kRowsPerWarp; ++i) {
    const int64_t row = row0 + i;
    if (row >= T_rows) break;                              // warp-uniform
    uint32_t key[kRegKeys];
#pragma unroll
    for (int u = 0; u < kRegKeys; ++u) key[u] = nxt[u];
    if (i + 1 < kRowsPerWarp) load_row(row + 1);
    uint32_t alive = 0;
#pragma unroll
    for (int u = 0; u < kRegKeys; ++u)
      if (lane + 32 * u < E) alive |= 1u << u;
    for (int j = 0; j < k; ++j) {
      uint32_t bk = 0;
      int bu = -1;
#pragma unroll
      for (int u = 0; u < kRegKeys; ++u)
        if (((alive >> u) & 1u) && (bu < 0 || key[u] > bk)) { bk = key[u]; bu = u; }
      const uint32_t m = __reduce_max_sync(0xFFFFFFFFu, bu >= 0 ? bk : 0u);
      const uint32_t cand = (bu >= 0 && bk == m) ? (uint32_t)(lane + 32 * bu) : 0x7FFFFFFFu;
      const uint32_t win = __reduce_min_sync(0xFFFFFFFFu, cand);
      if ((int)(win & 31u) == lane && win != 0x7FFFFFFFu) alive &= ~(1u << (win >> 5));
      if (lane == 0) {
        s_idx[warp][j] = (int)win;
        s_val[warp][j] = key_float(m);
      }
    }
    __syncwarp();
    if (apply_softmax) {
      float mx = -INFINITY;
      for (int j = 0; j < k; ++j) mx = fmaxf(mx, s_val[warp][j]);
      float sum = 0.0f;
      for (int j = 0; j < k; ++j) sum += expf(s_val[warp][j] - mx);
      for (int j = lane; j < k; j += 32) vals[row * ld_vals + j] = from_f32<T>(__fdiv_rn(expf(s_val[warp][j] - mx), sum));
    } else {
      for (int j = lane; j < k; j += 32) vals[row * ld_vals + j] = from_f32<T>(s_val[warp][j]);
    }
    for (int j = lane; j < k; j += 32) {
      const int e = s_idx[warp][j];
      indx[row * ld_indx + j] = (int16_t)e;
      atomicAdd(&s_hist[e], 1);
    }
    for (int w = lane; w < words; w += 32) {
      uint32_t bits = 0;
      for (int j = 0; j < k; ++j) {
        const int e = s_idx[warp][j];
        if ((e >> 5) == w) bits |= 1u << (e & 31);
      }
      bitmatrix[row * bm_stride_row + (int64_t)w * bm_stride_word] = bits;
    }
    __syncwarp();
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) partial[(int64_t)blockIdx.x * E + e] = s_hist[e];
}

// One row of the ragged metadata from the slice sizes in shared memory (s_size[0..E), s_size[E] = 0): row 0 =
// slice_offs (= expert offsets, also written to col_offs when given), rows 1..4 = block_offs and block schedule of the
// block sizes 16..128.  All threads of the block call it.
__device__ void ragged_row(int row, const int32_t* s_size, int E, int32_t* s_nb, int32_t* s_offs, int32_t* s_warp,
                           int32_t* __restrict__ slice_offs, int32_t* __restrict__ col_offs, int32_t* __restrict__ block_offs,
                           int64_t ld_block_offs, int32_t* __restrict__ block_sched, int64_t ld_sched, int64_t n_sched) {
  const int log2bs = row == 0 ? 0 : row + 3;
  for (int i = threadIdx.x; i <= E; i += blockDim.x)
    s_nb[i] = (i < E) ? (int32_t)(((int64_t)s_size[i] + ((1 << log2bs) - 1)) >> log2bs) : 0;
  __syncthreads();
  block_exclusive_scan(s_nb, s_offs, E + 1, s_warp);
  __syncthreads();
  int32_t* dst = row == 0 ? slice_offs : block_offs + (int64_t)(row - 1) * ld_block_offs;
  for (int i = threadIdx.x; i <= E; i += blockDim.x) {
    dst[i] = s_offs[i];
    if (row == 0 && i < E && col_offs) col_offs[i] = s_offs[i];
  }
  if (row > 0) {
    const int32_t tot = s_offs[E];
    int32_t* sched = block_sched + (int64_t)(row - 1) * ld_sched;
    for (int64_t p = threadIdx.x; p < n_sched; p += blockDim.x) {
      int32_t v = -1;
      if (p < tot) {
        int lo = 0, hi = E;  // largest e with offs[e] <= p
        while (hi - lo > 1) {
          const int mid = (lo + hi) >> 1;
          if (s_offs[mid] <= p) lo = mid; else hi = mid;
        }
        v = (int32_t)(((uint32_t)(p - s_offs[lo]) << 16) | (uint32_t)lo);
      }
      sched[p] = v;
    }
  }
  __syncthreads();
}

// Six blocks of 1024 threads.  n_experts <= 1024.
__global__ void __launch_bounds__(1024) route_scan_ragged_kernel(const int32_t* __restrict__ partial_in,
                                                                 int32_t* __restrict__ partial_out, int64_t n_blocks, int E,
                                                                 int32_t* __restrict__ col_sum, int32_t* __restrict__ col_offs,
                                                                 int32_t* __restrict__ slice_offs, int32_t* __restrict__ block_offs,
                                                                 int64_t ld_block_offs, int32_t* __restrict__ block_sched,
                                                                 int64_t ld_sched, int64_t n_sched) {
  extern __shared__ int32_t s_mem[];             // [1024] segment sums, then [E + 1] sizes, [E + 1] scan input, [E + 1] offsets
  __shared__ int32_t s_warp[33];
  int32_t* s_seg = s_mem;
  int32_t* s_size = s_mem + 1024;
  int32_t* s_nb = s_size + (E + 1);
  int32_t* s_offs = s_nb + (E + 1);
  // ---- 1. exclusive scan of partial[.][e] over the blocks of tokens, by S segments of blocks per expert -------------
  int Ep = 1;
  while (Ep < E) Ep <<= 1;
  const int S = 1024 / Ep;                        // threads (segments) per expert
  const int e = threadIdx.x % Ep, seg = threadIdx.x / Ep;
  const int64_t per = (n_blocks + S - 1) / S;
  const int64_t b_lo = min((int64_t)seg * per, n_blocks), b_hi = min(b_lo + per, n_blocks);
  int sum = 0;
  int first[16];                                  // the first 16 counts of this thread's segment stay in registers
#pragma unroll
  for (int u = 0; u < 16; ++u) first[u] = 0;
  if (e < E) {
#pragma unroll
    for (int u = 0; u < 16; ++u) first[u] = b_lo + u < b_hi ? partial_in[(b_lo + u) * E + e] : 0;
#pragma unroll
    for (int u = 0; u < 16; ++u) sum += first[u];
    for (int64_t b0 = b_lo + 16; b0 < b_hi; b0 += 8) {
      int v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = b0 + u < b_hi ? partial_in[(b0 + u) * E + e] : 0;
#pragma unroll
      for (int u = 0; u < 8; ++u) sum += v[u];
    }
  }
  s_seg[threadIdx.x] = sum;
  __syncthreads();
  int run = 0, total = 0;
  for (int s2 = 0; s2 < S; ++s2) {
    const int v = s_seg[s2 * Ep + e];
    if (s2 < seg) run += v;
    total += v;
  }
  // Six blocks share the work after the totals, which each of them forms for itself: block 0 turns the partial counts
  // into running offsets and writes col_sum, blocks 1..5 each build one row of the ragged metadata.  (One block doing
  // all of it was a chain of five scans with their barriers: 17 us for 16384 tokens.)
  const int role = blockIdx.x;
  if (e < E) {
    if (role == 0) {
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        if (b_lo + u < b_hi) partial_out[(b_lo + u) * E + e] = run;
        run += first[u];
      }
      for (int64_t b0 = b_lo + 16; b0 < b_hi; b0 += 8) {
        int v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = b0 + u < b_hi ? partial_in[(b0 + u) * E + e] : 0;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (b0 + u < b_hi) partial_out[(b0 + u) * E + e] = run;
          run += v[u];
        }
      }
      if (seg == 0) col_sum[e] = total;
    }
    if (seg == 0) s_size[e] = total;
  }
  if (threadIdx.x == 0) s_size[E] = 0;
  __syncthreads();
  if (role == 0) return;
  // ---- 2. expert offsets, then the ragged metadata: row 0 = slice_offs (= col_offs), rows 1..4 = block sizes 16..128 --
  ragged_row(role - 1, s_size, E, s_nb, s_offs, s_warp, slice_offs, col_offs, block_offs, ld_block_offs, block_sched, ld_sched,
             n_sched);
}

// The whole routing step of a small batch (at most 256 tokens, at most 256 experts, k in {1, 2, 4, 8, 16}) in ONE launch
// of five blocks of 1024 threads that do not wait on one another: every block selects the top-k of every row for itself
// (four lanes per row; 128 KB of logits at most) and counts the picks; block 0 stores the selection, the expert offsets
// (ragged row 0) and the positions of the entries, blocks 1..4 each build the block_offs row and the schedule of one
// block size.  Repeating the selection five times costs less than what it replaces: a chain of kernel boundaries
// (three launches) or of block barriers (one block doing all five rows took 20 us at 64 tokens).
template <typename T, int K>
__global__ void __launch_bounds__(1024) route_small_kernel(
    const T* __restrict__ logits, int64_t ld_logits, int64_t T_rows, int E, int apply_softmax, T* __restrict__ vals,
    int64_t ld_vals, int16_t* __restrict__ indx, int64_t ld_indx, uint32_t* __restrict__ bitmatrix, int64_t bm_stride_row,
    int64_t bm_stride_word, int32_t* __restrict__ col_sum, int32_t* __restrict__ col_sorted, int32_t* __restrict__ row_sorted,
    int32_t* __restrict__ slice_offs, int32_t* __restrict__ block_offs, int64_t ld_block_offs, int32_t* __restrict__ block_sched,
    int64_t ld_sched, int64_t n_sched) {
  extern __shared__ int32_t s_mem[];            // [E + 1] sizes, [E + 1] scan input, [E + 1] offsets, [E] expert offsets, [32][E] counters
  __shared__ int32_t s_warp[33];
  int32_t* s_size = s_mem;
  int32_t* s_nb = s_size + (E + 1);
  int32_t* s_offs = s_nb + (E + 1);
  int32_t* s_col = s_offs + (E + 1);
  int32_t* s_cnt = s_col + E;
  const int role = blockIdx.x;
  for (int e = threadIdx.x; e <= E; e += blockDim.x) s_size[e] = 0;
  __syncthreads();
  {
    const int part = threadIdx.x & 3;
    const int64_t row = threadIdx.x >> 2;
    const bool live = row < T_rows;
    const T* x = logits + (live ? row : 0) * ld_logits;
    const TopK<K> tk = quad_select<T, K>(x, E, part);
    if (live) {
      if (role == 0) {
        quad_store<T, K>(tk, part, row, E, apply_softmax, vals, ld_vals, indx, ld_indx, bitmatrix, bm_stride_row,
                         bm_stride_word, s_size);
      } else if (part == 0) {
#pragma unroll
        for (int i = 0; i < K; ++i) atomicAdd(&s_size[tk.idx[i]], 1);
      }
    }
  }
  __syncthreads();                               // the picks are counted (block 0: and in global memory)
  if (role > 0) {
    ragged_row(role, s_size, E, s_nb, s_offs, s_warp, slice_offs, nullptr, block_offs, ld_block_offs, block_sched, ld_sched, n_sched);
    return;
  }
  for (int e = threadIdx.x; e < E; e += blockDim.x) col_sum[e] = s_size[e];
  ragged_row(0, s_size, E, s_nb, s_offs, s_warp, slice_offs, nullptr, block_offs, ld_block_offs, block_sched, ld_sched, n_sched);
  for (int e = threadIdx.x; e < E; e += blockDim.x) s_col[e] = s_offs[e];
  __syncthreads();
  rank_block(indx, ld_indx, T_rows, E, K, T_rows, nullptr, s_col, 0, col_sorted, row_sorted, s_cnt);
}

constexpr int kRouteSmallTokens = 256;

}  // namespace

extern "C" __attribute__((visibility("default"))) size_t moe_route_workspace(int64_t T, int E, int k) {
  (void)k;
  const int64_t nb = cdiv64(T > 0 ? T : 1, kRouteTokPerBlock);
  return (size_t)((2 * nb * E + E) * (int64_t)sizeof(int32_t));
}

extern "C" __attribute__((visibility("default"))) int moe_route(
    const void* logits, int dtype, int64_t T, int E, int k, int apply_softmax, int64_t ld_logits, void* vals, int64_t ld_vals,
    int16_t* indx, int64_t ld_indx, uint32_t* bitmatrix, int64_t bm_stride_row, int64_t bm_stride_word, int32_t* col_sum,
    int32_t* col_sorted, int32_t* row_sorted, int32_t* slice_offs, int32_t* block_offs, int64_t ld_block_offs,
    int32_t* block_sched, int64_t ld_sched, int64_t n_sched, void* workspace, size_t workspace_bytes, void* stream) {
  MOE_CHECK_ARG(T > 0 && E > 0 && k > 0 && k <= kMaxTopK && k <= E, "moe_route: bad extents T=%lld E=%d k=%d", (long long)T, E, k);
  if (E > 256) {
    moe_set_error("moe_route: the fused routing handles up to 256 experts (got %d); use the separate entry points", E);
    return MOE_ERR_UNSUPPORTED;
  }
  MOE_CHECK_ARG(logits && vals && indx && bitmatrix && col_sum && col_sorted && row_sorted && slice_offs && block_offs &&
                    (block_sched || n_sched == 0) && workspace,
                "moe_route: NULL pointer");
  MOE_CHECK_ARG(ld_block_offs >= E + 1 && ld_sched >= n_sched, "moe_route: leading dimensions too small");
  MOE_CHECK_ARG(workspace_bytes >= moe_route_workspace(T, E, k), "moe_route: workspace too small (%zu < %zu)", workspace_bytes,
                moe_route_workspace(T, E, k));
  cudaStream_t st = (cudaStream_t)stream;
  if (T <= kRouteSmallTokens && (k == 1 || k == 2 || k == 4 || k == 8 || k == 16)) {
    const size_t smem_s = (size_t)(3 * (E + 1) + E + 32 * E) * sizeof(int32_t);
#define MOE_ROUTE_SMALL(KK)                                                                                              \
  MOE_DISPATCH_FLOAT(dtype, Tv, {                                                                                         \
    route_small_kernel<Tv, KK><<<5, 1024, smem_s, st>>>((const Tv*)logits, ld_logits, T, E, apply_softmax, (Tv*)vals, ld_vals, \
                                                         indx, ld_indx, bitmatrix, bm_stride_row, bm_stride_word, col_sum,  \
                                                         col_sorted, row_sorted, slice_offs, block_offs, ld_block_offs,     \
                                                         block_sched, ld_sched, n_sched);                                   \
  })
    switch (k) {
      case 1: MOE_ROUTE_SMALL(1); break;
      case 2: MOE_ROUTE_SMALL(2); break;
      case 4: MOE_ROUTE_SMALL(4); break;
      case 8: MOE_ROUTE_SMALL(8); break;
      default: MOE_ROUTE_SMALL(16); break;
    }
#undef MOE_ROUTE_SMALL
    MOE_CHECK_LAUNCH();
    return MOE_OK;
  }
  const int64_t nb = cdiv64(T, kRouteTokPerBlock);
  int32_t* partial = (int32_t*)workspace;          // counts per block of tokens, their running offsets, expert offsets
  int32_t* scanned = partial + nb * E;
  int32_t* col_offs = scanned + nb * E;
#define MOE_ROUTE_QUAD(KK)                                                                                               \
  MOE_DISPATCH_FLOAT(dtype, Tv, {                                                                                         \
    topk_quad_kernel<Tv, KK, true><<<(int)nb, 4 * kRouteTokPerBlock, (size_t)E * sizeof(int32_t), st>>>(                                   \
        (const Tv*)logits, ld_logits, T, E, apply_softmax, (Tv*)vals, ld_vals, indx, ld_indx, bitmatrix, bm_stride_row,    \
        bm_stride_word, partial);                                                                                          \
  })
  switch (k) {
    case 1: MOE_ROUTE_QUAD(1); break;
    case 2: MOE_ROUTE_QUAD(2); break;
    case 4: MOE_ROUTE_QUAD(4); break;
    case 8: MOE_ROUTE_QUAD(8); break;
    case 16: MOE_ROUTE_QUAD(16); break;
    default:
      MOE_DISPATCH_FLOAT(dtype, Tv, {
        route_topk_hist_kernel<Tv><<<(int)nb, kRouteWarps * 32, (size_t)E * sizeof(int32_t), st>>>(
            (const Tv*)logits, ld_logits, T, E, k, apply_softmax, (Tv*)vals, ld_vals, indx, ld_indx, bitmatrix, bm_stride_row,
            bm_stride_word, partial);
      });
  }
#undef MOE_ROUTE_QUAD
  MOE_CHECK_LAUNCH();
  const size_t smem_b = (size_t)(1024 + 3 * (E + 1)) * sizeof(int32_t);
  route_scan_ragged_kernel<<<6, 1024, smem_b, st>>>(partial, scanned, nb, E, col_sum, col_offs, slice_offs, block_offs,
                                                    ld_block_offs, block_sched, ld_sched, n_sched);
  MOE_CHECK_LAUNCH();
  const size_t smem_rank = (size_t)(kRouteTokPerBlock / 32) * E * sizeof(int32_t);
  bm_rank_kernel<<<(int)nb, kRouteTokPerBlock, smem_rank, st>>>(indx, ld_indx, T, E, k, nullptr, scanned, col_offs, col_sorted,
                                                                row_sorted);
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}

// ---------------------------------------------------------------------------------------------------------
// moe_bitmatrix_metadata_noalloc: the same histogram + expert-major sort for hosts that cannot give this
// library a scratch buffer because they cannot allocate one at that point -- a serving process that handed
// all device memory to its own pools at start-up, or a latency-critical section in which cudaMalloc (which
// synchronises the device) is not acceptable.  The three sort passes need nb * E + E ints of scratch
// (nb = ceil(T / 256)); here that scratch is a fixed array inside the library image.
//
// Cost: every GPU that loads libmoe_b200.so carries kNoAllocScratchBytes (1 MiB) of device memory until the
// process exits, whether or not this entry point is ever called.
static __device__ __align__(256) int32_t g_bm_scratch[(1 << 20) / sizeof(int32_t)];
constexpr size_t kNoAllocScratchBytes = sizeof(int32_t) * ((1 << 20) / sizeof(int32_t));

// Device address of g_bm_scratch, looked up once per device.  In host code the name g_bm_scratch is only a
// handle for the runtime; the address a kernel can use comes from cudaGetSymbolAddress with that device current.
static void* g_bm_scratch_addr[64] = {nullptr};

extern "C" __attribute__((visibility("default"))) size_t moe_bitmatrix_metadata_noalloc_capacity(void) {
  return kNoAllocScratchBytes;
}

extern "C" __attribute__((visibility("default"))) int moe_bitmatrix_metadata_noalloc(
    const int16_t* indx, int64_t ld_indx, int64_t T, int E, int k, const int32_t* n_rows_dev, int32_t* col_sum,
    int32_t* col_sorted, int32_t* row_sorted, void* stream) {
  MOE_CHECK_ARG(T >= 0 && E > 0 && k > 0, "moe_bitmatrix_metadata_noalloc: bad extents T=%lld E=%d k=%d", (long long)T, E, k);
  const size_t need = moe_bitmatrix_metadata_workspace(T, E, k);
  MOE_CHECK_ARG(need <= kNoAllocScratchBytes,
                "moe_bitmatrix_metadata_noalloc: T=%lld tokens x E=%d experts needs %zu bytes of scratch, the built-in "
                "scratch holds %zu (ceil(T/256) * E + E ints must fit); use moe_bitmatrix_metadata with a caller buffer",
                (long long)T, E, need, kNoAllocScratchBytes);
  int dev = -1;
  MOE_CHECK_CUDA(cudaGetDevice(&dev));
  MOE_CHECK_ARG(dev >= 0 && dev < 64, "moe_bitmatrix_metadata_noalloc: device index %d out of range", dev);
  if (g_bm_scratch_addr[dev] == nullptr) {
    // first call on this device: resolve the symbol (not an allocation; the array is part of the module image)
    void* p = nullptr;
    MOE_CHECK_CUDA(cudaGetSymbolAddress(&p, g_bm_scratch));
    MOE_CHECK_ARG(p != nullptr, "moe_bitmatrix_metadata_noalloc: cudaGetSymbolAddress returned NULL");
    g_bm_scratch_addr[dev] = p;
  }
  // Nothing in the scratch has to start at zero: pass 1 writes every partial[block][expert] and pass 2 every
  // col_offs[expert] before they are read.  col_sum, which must, is cleared by the call below.
  return moe_bitmatrix_metadata(indx, ld_indx, T, E, k, n_rows_dev, col_sum, col_sorted, row_sorted,
                                g_bm_scratch_addr[dev], kNoAllocScratchBytes, stream);
}
