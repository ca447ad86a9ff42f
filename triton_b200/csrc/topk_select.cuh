// Best-k selection in registers, shared by the stand-alone top-k kernels and the router kernel.
//
// Order: larger value first, equal values to the smaller expert index (triton_kernels
// topk_details/_topk_forward.py:29-35 packs `PAD - index` under the value for the same effect).
#pragma once
#include <cstdint>

// order-preserving map float -> uint32 (larger float <=> larger key)
__device__ __forceinline__ uint32_t sel_float_key(float f) {
  const uint32_t b = __float_as_uint(f);
  return b ^ ((b & 0x80000000u) ? 0xFFFFFFFFu : 0x80000000u);
}
__device__ __forceinline__ float sel_key_float(uint32_t k) {
  return __uint_as_float(k ^ ((k & 0x80000000u) ? 0x80000000u : 0xFFFFFFFFu));
}

// The K best (value key, expert) pairs, best first.  An insertion compares the candidate with all K places at once
// (independent compares, then two selects per place) instead of bubbling it down: a thread walks its share of a row
// alone, so the length of the dependent chain is what the selection costs.  `push` takes experts in ascending order
// and keeps the earlier of two equal values ahead with a strict compare; `push_any` takes them in any order and
// compares the expert index too.
template <int K>
struct TopK {
  uint32_t key[K];
  int idx[K];
  __device__ __forceinline__ TopK() {
#pragma unroll
    for (int i = 0; i < K; ++i) { key[i] = 0u; idx[i] = 0x7FFFFFFF; }
  }
  __device__ __forceinline__ void place(uint32_t c, int ci, const bool (&gt)[K]) {
#pragma unroll
    for (int i = K - 1; i > 0; --i) {               // descending: place i - 1 still holds its old entry
      key[i] = gt[i] ? (gt[i - 1] ? key[i - 1] : c) : key[i];
      idx[i] = gt[i] ? (gt[i - 1] ? idx[i - 1] : ci) : idx[i];
    }
    key[0] = gt[0] ? c : key[0];
    idx[0] = gt[0] ? ci : idx[0];
  }
  __device__ __forceinline__ void push(float v, int e) {
    const uint32_t c = sel_float_key(v);
    bool gt[K];
#pragma unroll
    for (int i = 0; i < K; ++i) gt[i] = c > key[i];
    place(c, e, gt);
  }
  __device__ __forceinline__ void push_any(uint32_t c, int ci) {
    bool gt[K];
#pragma unroll
    for (int i = 0; i < K; ++i) gt[i] = c > key[i] || (c == key[i] && ci < idx[i]);
    place(c, ci, gt);
  }
  // the lists of the lanes lane ^ 1, lane ^ 2, ... lane ^ (parts - 1) meet: afterwards every lane of the group holds
  // the best K of the group (parts a power of two, groups aligned in the warp; all 32 lanes must call)
  __device__ __forceinline__ void merge_lanes(int parts) {
    for (int m = 1; m < parts; m <<= 1) {
      uint32_t ok_[K];
      int oi[K];
#pragma unroll
      for (int i = 0; i < K; ++i) {
        ok_[i] = __shfl_xor_sync(0xFFFFFFFFu, key[i], m);
        oi[i] = __shfl_xor_sync(0xFFFFFFFFu, idx[i], m);
      }
#pragma unroll
      for (int i = 0; i < K; ++i) push_any(ok_[i], oi[i]);
    }
  }
};
