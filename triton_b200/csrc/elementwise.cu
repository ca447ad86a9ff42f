// HBM-bound elementwise kernels: standalone SwiGLU, the masked / scaled k-way combine (reduce) and the
// row gather / scatter used around the expert-parallel exchange.
//
// SwiGLU semantics: triton_kernels swiglu_details/_swiglu.py:55-64 (gate = even columns, linear = odd
// columns; gate clamped above, linear clamped both ways; s = g / (1 + exp(-alpha g)); out = s*l + s).
// Combine semantics: triton_kernels reduce.py:1181-1214 (fp32 sum over the reduced axis of
// mask * scale * x, cast to the output type).
#include "common.cuh"

namespace {

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float swiglu_one(float g, float l, float alpha, float limit, bool has_limit) {
  if (has_limit) {
    g = fminf(g, limit);
    l = fminf(fmaxf(l, -limit), limit);
  }
  const float s = g / (1.0f + ex2_approx(-alpha * g * 1.4426950408889634f));
  return fmaf(s, l, s);
}

// thread = 8 outputs (16 interleaved inputs) on the vector path
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) swiglu_kernel(const T* __restrict__ a, int64_t ld_a, T* __restrict__ out,
                                                     int64_t ld_out, int64_t M, int64_t N, float alpha, float limit,
                                                     int has_limit, const int32_t* __restrict__ n_rows_dev) {
  if (n_rows_dev) M = min(M, (int64_t)*n_rows_dev);
  constexpr int V = VEC ? 8 : 1;
  const int64_t per_row = (N + V - 1) / V;
  const int64_t total = M * per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / per_row, c = (i - r * per_row) * V;
    const T* src = a + r * ld_a + 2 * c;
    T* dst = out + r * ld_out + c;
    if constexpr (VEC && sizeof(T) == 2) {
      uint4 v0 = *reinterpret_cast<const uint4*>(src);
      uint4 v1 = *reinterpret_cast<const uint4*>(src + 8);
      const T* e0 = reinterpret_cast<const T*>(&v0);
      const T* e1 = reinterpret_cast<const T*>(&v1);
      T o[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        o[j] = from_f32<T>(swiglu_one(to_f32<T>(e0[2 * j]), to_f32<T>(e0[2 * j + 1]), alpha, limit, has_limit));
        o[4 + j] = from_f32<T>(swiglu_one(to_f32<T>(e1[2 * j]), to_f32<T>(e1[2 * j + 1]), alpha, limit, has_limit));
      }
      *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(o);
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j)
        if (c + j < N)
          dst[j] = from_f32<T>(swiglu_one(to_f32<T>(src[2 * j]), to_f32<T>(src[2 * j + 1]), alpha, limit, has_limit));
    }
  }
}

__device__ __forceinline__ bool mask_nonzero(const void* m, int bytes, int64_t off) {
  switch (bytes) {
    case 1: return ((const uint8_t*)m)[off] != 0;
    case 2: return ((const uint16_t*)m)[off] != 0;
    case 4: return ((const uint32_t*)m)[off] != 0;
    default: return ((const unsigned long long*)m)[off] != 0;
  }
}

// y[s0, s1] = sum_r mask * scale * x[r, s0, s1]; thread = V consecutive s1 (V = 8 on the vector path)
template <typename TX, typename TY, bool VEC>
__global__ void __launch_bounds__(256) reduce_kernel(const TX* __restrict__ x, int64_t R, int64_t S0, int64_t S1,
                                                     int64_t sx_r, int64_t sx_0, int64_t sx_1, const void* __restrict__ mask,
                                                     int mask_bytes, int64_t sm_r, int64_t sm_0, int64_t sm_1,
                                                     const float* __restrict__ scale, int64_t ss_r, int64_t ss_0,
                                                     int64_t ss_1, TY* __restrict__ y, int64_t sy_0, int64_t sy_1) {
  constexpr int V = VEC ? 8 : 1;
  const int64_t per_row = (S1 + V - 1) / V;
  const int64_t total = S0 * per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t s0 = i / per_row, c = (i - s0 * per_row) * V;
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.0f;
    for (int64_t r = 0; r < R; ++r) {
      if constexpr (VEC) {
        // vector path: mask and scale do not vary along s1 (stride 0), x is contiguous along s1
        if (mask && !mask_nonzero(mask, mask_bytes, r * sm_r + s0 * sm_0)) continue;
        const float sc = scale ? scale[r * ss_r + s0 * ss_0] : 1.0f;
        uint4 raw = *reinterpret_cast<const uint4*>(x + r * sx_r + s0 * sx_0 + c);
        const TX* e = reinterpret_cast<const TX*>(&raw);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += to_f32<TX>(e[j]) * sc;
      } else {
        if (mask && !mask_nonzero(mask, mask_bytes, r * sm_r + s0 * sm_0 + c * sm_1)) continue;
        const float sc = scale ? scale[r * ss_r + s0 * ss_0 + c * ss_1] : 1.0f;
        acc[0] += to_f32<TX>(x[r * sx_r + s0 * sx_0 + c * sx_1]) * sc;
      }
    }
    if constexpr (VEC) {
      TY o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = from_f32<TY>(acc[j]);
      *reinterpret_cast<uint4*>(y + s0 * sy_0 + c) = *reinterpret_cast<const uint4*>(o);
    } else {
      y[s0 * sy_0 + c * sy_1] = from_f32<TY>(acc[0]);
    }
  }
}

// dst[i, :] = src[indx[i], :]   (indx < 0: zero row) -- 16 bytes per thread
// One block walks whole rows (no division per 16-byte element); every thread keeps two loads in flight.
__global__ void __launch_bounds__(128) gather_rows_kernel(const uint8_t* __restrict__ src, int64_t ld_src,
                                                          const int32_t* __restrict__ indx, int64_t n_out,
                                                          int64_t row_bytes, uint8_t* __restrict__ dst, int64_t ld_dst) {
  const int vec_per_row = (int)(row_bytes >> 4);
  for (int64_t r = blockIdx.x; r < n_out; r += gridDim.x) {
    const int32_t s = indx ? indx[r] : (int32_t)r;
    const uint4* in = s >= 0 ? reinterpret_cast<const uint4*>(src + (int64_t)s * ld_src) : nullptr;
    uint4* out = reinterpret_cast<uint4*>(dst + r * ld_dst);
    for (int c = threadIdx.x; c < vec_per_row; c += 256) {
      const int c2 = c + 128;
      const uint4 v0 = in ? in[c] : make_uint4(0, 0, 0, 0);
      const uint4 v1 = (in && c2 < vec_per_row) ? in[c2] : make_uint4(0, 0, 0, 0);
      out[c] = v0;
      if (c2 < vec_per_row) out[c2] = v1;
    }
  }
}

// Rows spread over several devices: global row g lives in buffer g / rows_per_peer at row g % rows_per_peer.
struct PeerBases { const uint8_t* base[MOE_MAX_PEERS]; };

// dst[r, :] = peers[indx[r] / rows_per_peer][indx[r] % rows_per_peer, :]; indx -1: zeros, indx -2: row left untouched.
// A warp takes `batch` (1 .. 32) consecutive rows at a time: their indices come with one coalesced load, so skipped
// rows (most of them, on a rank that owns 1/W of the experts) cost no round trip each; the live rows are then copied
// one after the other by the whole warp, four 16-byte loads in flight per lane.  The host picks the batch so that
// there are warps for all SMs: with a block per 32 rows a decode-sized pull (512 rows) ran on 16 blocks, each walking
// its rows one NVLink round trip after the other -- 119 us for 1.5 MB.
__global__ void __launch_bounds__(128) gather_rows_peers_kernel(PeerBases peers, int64_t rows_per_peer, int64_t ld_src,
                                                                const int32_t* __restrict__ indx, int64_t n_out,
                                                                int64_t row_bytes, uint8_t* __restrict__ dst, int64_t ld_dst,
                                                                int batch) {
  const int lane = threadIdx.x & 31;
  const int vec_per_row = (int)(row_bytes >> 4);
  const int64_t n_warps = (int64_t)gridDim.x * 4;
  for (int64_t r0 = ((int64_t)blockIdx.x * 4 + (threadIdx.x >> 5)) * batch; r0 < n_out; r0 += n_warps * batch) {
    int32_t s = -2;
    if (lane < batch && r0 + lane < n_out) s = indx[r0 + lane];
    unsigned live = __ballot_sync(0xFFFFFFFFu, s != -2);
    while (live) {
      const int j = __ffs(live) - 1;
      live &= live - 1;
      const int32_t sj = __shfl_sync(0xFFFFFFFFu, s, j);
      const uint4* src = nullptr;
      if (sj >= 0) {
        const int64_t peer = sj / rows_per_peer;
        src = reinterpret_cast<const uint4*>(peers.base[peer] + (sj - peer * rows_per_peer) * ld_src);
      }
      uint4* out = reinterpret_cast<uint4*>(dst + (r0 + j) * ld_dst);
      for (int c = lane; c < vec_per_row; c += 128) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = (src && c + 32 * u < vec_per_row) ? src[c + 32 * u] : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (c + 32 * u < vec_per_row) out[c + 32 * u] = v[u];
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// Barrier among the ranks of an expert-parallel group through peer-mapped signal words, and an all-gather of small
// per-rank slices by plain loads from the peers' buffers: the routing phase of the expert-parallel layer then holds
// no collective call, only kernels (which also makes the whole step capturable in a CUDA graph).
// Rank r owns `sig` words [W]; word s is written by rank s.  Every call bumps this rank's epoch counter (device
// memory, so that a replayed graph keeps counting), writes the epoch into its word on every peer and waits until all
// of its own words have reached it.  The wait is bounded (2 s): on expiry the kernel records a status and returns.
struct PeerSignals { uint32_t* sig[MOE_MAX_PEERS]; };

__global__ void __launch_bounds__(32) peer_barrier_kernel(PeerSignals peers, int W, int rank, uint32_t* __restrict__ epoch,
                                                          int32_t* __restrict__ status) {
  __shared__ uint32_t s_e;
  if (threadIdx.x == 0) {
    s_e = *epoch + 1u;
    *epoch = s_e;
  }
  __syncthreads();
  const uint32_t e = s_e;
  __threadfence_system();                              // everything this rank wrote before the barrier is visible first
  if ((int)threadIdx.x < W) {
    uint32_t* theirs = peers.sig[threadIdx.x] + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(e) : "memory");
    const uint32_t* mine = peers.sig[rank] + threadIdx.x;
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (;;) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if ((int32_t)(v - e) >= 0) break;
      unsigned long long t1;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
      if (t1 - t0 > 2000000000ull) {
        if (status) atomicExch(status, 901);
        break;
      }
      __nanosleep(200);
    }
  }
  __syncthreads();
  __threadfence_system();
}

// dst[r * slice_words + w] = src[r][w]: every rank's slice (32-bit words) from its own buffer into one local array
__global__ void __launch_bounds__(256) allgather_peers_kernel(PeerBases src, int W, int64_t slice_words,
                                                              uint32_t* __restrict__ dst) {
  const int64_t total = (int64_t)W * slice_words;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / slice_words;
    dst[i] = reinterpret_cast<const uint32_t*>(src.base[r])[i - r * slice_words];
  }
}

// dst[indx[i], :] = src[i, :]   (indx < 0: dropped)
__global__ void __launch_bounds__(256) scatter_rows_kernel(const uint8_t* __restrict__ src, int64_t ld_src,
                                                           const int32_t* __restrict__ indx, int64_t n_in,
                                                           int64_t row_bytes, uint8_t* __restrict__ dst, int64_t ld_dst) {
  const int64_t vec_per_row = row_bytes >> 4;
  const int64_t total = n_in * vec_per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / vec_per_row, c = i - r * vec_per_row;
    const int32_t d = indx[r];
    if (d < 0) continue;
    *reinterpret_cast<uint4*>(dst + (int64_t)d * ld_dst + c * 16) =
        *reinterpret_cast<const uint4*>(src + r * ld_src + c * 16);
  }
}

int grid_for(int64_t total, int threads) {
  int64_t blocks = cdiv64(total, threads);
  int64_t cap = (int64_t)moe_sm_count() * 16;
  if (blocks > cap) blocks = cap;
  return (int)(blocks < 1 ? 1 : blocks);
}

}  // namespace

extern "C" __attribute__((visibility("default"))) int moe_swiglu(const void* a, int64_t ld_a, void* out, int64_t ld_out, int dtype, int64_t M, int64_t N,
                          float alpha, float limit, int has_limit, const int32_t* n_rows_dev, void* stream) {
  MOE_CHECK_ARG(M >= 0 && N >= 0, "moe_swiglu: negative extent");
  if (M == 0 || N == 0) return MOE_OK;
  MOE_CHECK_ARG(a && out, "moe_swiglu: NULL pointer");
  cudaStream_t st = (cudaStream_t)stream;
  MOE_DISPATCH_FLOAT(dtype, T, {
    const bool vec = sizeof(T) == 2 && N % 8 == 0 && ld_a % 8 == 0 && ld_out % 8 == 0 && (uintptr_t)a % 16 == 0 &&
                     (uintptr_t)out % 16 == 0;
    if (vec)
      swiglu_kernel<T, true><<<grid_for(M * (N / 8), 256), 256, 0, st>>>((const T*)a, ld_a, (T*)out, ld_out, M, N, alpha,
                                                                         limit, has_limit, n_rows_dev);
    else
      swiglu_kernel<T, false><<<grid_for(M * N, 256), 256, 0, st>>>((const T*)a, ld_a, (T*)out, ld_out, M, N, alpha,
                                                                    limit, has_limit, n_rows_dev);
  });
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}

template <typename TX, typename TY>
static int launch_reduce(const void* x, int64_t R, int64_t S0, int64_t S1, int64_t sx_r, int64_t sx_0, int64_t sx_1,
                         const void* mask, int mb, int64_t sm_r, int64_t sm_0, int64_t sm_1, const float* scale,
                         int64_t ss_r, int64_t ss_0, int64_t ss_1, void* y, int64_t sy_0, int64_t sy_1,
                         cudaStream_t st) {
  if constexpr (sizeof(TX) == 2 && sizeof(TY) == 2) {
    const bool vec = sx_1 == 1 && sy_1 == 1 && S1 % 8 == 0 && sx_r % 8 == 0 && sx_0 % 8 == 0 && sy_0 % 8 == 0 &&
                     (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0 && (!mask || sm_1 == 0) && (!scale || ss_1 == 0);
    if (vec) {
      reduce_kernel<TX, TY, true><<<grid_for(S0 * (S1 / 8), 256), 256, 0, st>>>(
          (const TX*)x, R, S0, S1, sx_r, sx_0, sx_1, mask, mb, sm_r, sm_0, sm_1, scale, ss_r, ss_0, ss_1, (TY*)y, sy_0,
          sy_1);
      MOE_CHECK_LAUNCH();
      return MOE_OK;
    }
  }
  reduce_kernel<TX, TY, false><<<grid_for(S0 * S1, 256), 256, 0, st>>>(
      (const TX*)x, R, S0, S1, sx_r, sx_0, sx_1, mask, mb, sm_r, sm_0, sm_1, scale, ss_r, ss_0, ss_1, (TY*)y, sy_0, sy_1);
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}

extern "C" __attribute__((visibility("default"))) int moe_reduce(const void* x, int dtype, int64_t R, int64_t S0, int64_t S1, int64_t sx_r, int64_t sx_0,
                          int64_t sx_1, const void* mask, int mask_elem_bytes, int64_t sm_r, int64_t sm_0, int64_t sm_1,
                          const float* scale, int64_t ss_r, int64_t ss_0, int64_t ss_1, void* y, int y_dtype,
                          int64_t sy_0, int64_t sy_1, void* stream) {
  MOE_CHECK_ARG(R >= 0 && S0 >= 0 && S1 >= 0, "moe_reduce: negative extent");
  if (S0 == 0 || S1 == 0) return MOE_OK;
  MOE_CHECK_ARG(x && y, "moe_reduce: NULL pointer");
  MOE_CHECK_ARG(!mask || mask_elem_bytes == 1 || mask_elem_bytes == 2 || mask_elem_bytes == 4 || mask_elem_bytes == 8,
                "moe_reduce: mask element size %d unsupported", mask_elem_bytes);
  cudaStream_t st = (cudaStream_t)stream;
#define MOE_REDUCE_CASE(DX, TX, DY, TY)                                                                             \
  if (dtype == DX && y_dtype == DY)                                                                                 \
    return launch_reduce<TX, TY>(x, R, S0, S1, sx_r, sx_0, sx_1, mask, mask_elem_bytes, sm_r, sm_0, sm_1, scale, ss_r, \
                                 ss_0, ss_1, y, sy_0, sy_1, st);
  MOE_REDUCE_CASE(MOE_BF16, __nv_bfloat16, MOE_BF16, __nv_bfloat16)
  MOE_REDUCE_CASE(MOE_F16, __half, MOE_F16, __half)
  MOE_REDUCE_CASE(MOE_F32, float, MOE_F32, float)
  MOE_REDUCE_CASE(MOE_BF16, __nv_bfloat16, MOE_F32, float)
  MOE_REDUCE_CASE(MOE_F16, __half, MOE_F32, float)
  MOE_REDUCE_CASE(MOE_F32, float, MOE_BF16, __nv_bfloat16)
  MOE_REDUCE_CASE(MOE_F32, float, MOE_F16, __half)
#undef MOE_REDUCE_CASE
  moe_set_error("moe_reduce: dtype combination (%d -> %d) unsupported", dtype, y_dtype);
  return MOE_ERR_UNSUPPORTED;
}

extern "C" __attribute__((visibility("default"))) int moe_gather_rows(const void* src, int64_t ld_src, const int32_t* row_indx, int64_t n_rows_out,
                               int64_t row_bytes, void* dst, int64_t ld_dst, void* stream) {
  MOE_CHECK_ARG(n_rows_out >= 0 && row_bytes >= 0, "moe_gather_rows: negative extent");
  if (n_rows_out == 0 || row_bytes == 0) return MOE_OK;
  MOE_CHECK_ARG(src && dst, "moe_gather_rows: NULL pointer");
  MOE_CHECK_ARG(row_bytes % 16 == 0 && ld_src % 16 == 0 && ld_dst % 16 == 0 && (uintptr_t)src % 16 == 0 &&
                    (uintptr_t)dst % 16 == 0,
                "moe_gather_rows: rows must be 16-byte aligned multiples of 16 bytes");
  const int64_t gr_max = (int64_t)moe_sm_count() * 16;
  gather_rows_kernel<<<(int)(n_rows_out < gr_max ? n_rows_out : gr_max), 128, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)src, ld_src, row_indx, n_rows_out, row_bytes, (uint8_t*)dst, ld_dst);
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}

extern "C" __attribute__((visibility("default"))) int moe_gather_rows_peers(const void* const* src_peers, int n_peers, int64_t rows_per_peer,
                                     int64_t ld_src, const int32_t* row_indx, int64_t n_rows_out, int64_t row_bytes,
                                     void* dst, int64_t ld_dst, void* stream) {
  MOE_CHECK_ARG(n_rows_out >= 0 && row_bytes >= 0, "moe_gather_rows_peers: negative extent");
  if (n_rows_out == 0 || row_bytes == 0) return MOE_OK;
  MOE_CHECK_ARG(src_peers && dst && row_indx, "moe_gather_rows_peers: NULL pointer");
  MOE_CHECK_ARG(n_peers >= 1 && n_peers <= MOE_MAX_PEERS && rows_per_peer > 0,
                "moe_gather_rows_peers: need 1..%d peers and rows_per_peer > 0", MOE_MAX_PEERS);
  MOE_CHECK_ARG(row_bytes % 16 == 0 && ld_src % 16 == 0 && ld_dst % 16 == 0 && (uintptr_t)dst % 16 == 0,
                "moe_gather_rows_peers: rows must be 16-byte aligned multiples of 16 bytes");
  PeerBases pb;
  for (int i = 0; i < MOE_MAX_PEERS; ++i) {
    pb.base[i] = i < n_peers ? (const uint8_t*)src_peers[i] : nullptr;
    MOE_CHECK_ARG(i >= n_peers || (pb.base[i] && (uintptr_t)pb.base[i] % 16 == 0),
                  "moe_gather_rows_peers: peer buffer %d is NULL or not 16-byte aligned", i);
  }
  // rows per warp at a time: as many as leave a warp for every slot of the grid, 32 at most
  const int64_t max_blocks = (int64_t)moe_sm_count() * 16;
  int batch = 32;
  while (batch > 1 && cdiv64(n_rows_out, batch) < max_blocks * 4) batch >>= 1;
  const int64_t blocks = cdiv64(cdiv64(n_rows_out, batch), 4);
  gather_rows_peers_kernel<<<(int)(blocks < max_blocks ? blocks : max_blocks), 128, 0, (cudaStream_t)stream>>>(
      pb, rows_per_peer, ld_src, row_indx, n_rows_out, row_bytes, (uint8_t*)dst, ld_dst, batch);
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}

extern "C" __attribute__((visibility("default"))) int moe_peer_barrier(void* const* sig_peers, int n_peers, int rank, uint32_t* epoch,
                                                                       int32_t* status, void* stream) {
  MOE_CHECK_ARG(sig_peers && epoch, "moe_peer_barrier: NULL pointer");
  MOE_CHECK_ARG(n_peers >= 1 && n_peers <= MOE_MAX_PEERS && rank >= 0 && rank < n_peers, "moe_peer_barrier: bad rank / world");
  PeerSignals ps;
  for (int i = 0; i < MOE_MAX_PEERS; ++i) {
    ps.sig[i] = i < n_peers ? (uint32_t*)sig_peers[i] : nullptr;
    MOE_CHECK_ARG(i >= n_peers || ps.sig[i], "moe_peer_barrier: signal buffer %d is NULL", i);
  }
  peer_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(ps, n_peers, rank, epoch, status);
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}

extern "C" __attribute__((visibility("default"))) int moe_allgather_peers(const void* const* src_peers, int n_peers, int64_t slice_bytes,
                                                                          void* dst, void* stream) {
  MOE_CHECK_ARG(slice_bytes >= 0 && slice_bytes % 4 == 0, "moe_allgather_peers: slices must be multiples of 4 bytes");
  if (slice_bytes == 0) return MOE_OK;
  MOE_CHECK_ARG(src_peers && dst, "moe_allgather_peers: NULL pointer");
  MOE_CHECK_ARG(n_peers >= 1 && n_peers <= MOE_MAX_PEERS, "moe_allgather_peers: need 1..%d peers", MOE_MAX_PEERS);
  PeerBases pb;
  for (int i = 0; i < MOE_MAX_PEERS; ++i) {
    pb.base[i] = i < n_peers ? (const uint8_t*)src_peers[i] : nullptr;
    MOE_CHECK_ARG(i >= n_peers || (pb.base[i] && (uintptr_t)pb.base[i] % 4 == 0), "moe_allgather_peers: buffer %d is NULL or unaligned", i);
  }
  allgather_peers_kernel<<<grid_for((int64_t)n_peers * (slice_bytes / 4), 256), 256, 0, (cudaStream_t)stream>>>(
      pb, n_peers, slice_bytes / 4, (uint32_t*)dst);
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}

extern "C" __attribute__((visibility("default"))) int moe_scatter_rows(const void* src, int64_t ld_src, const int32_t* row_indx, int64_t n_rows_in,
                                int64_t row_bytes, void* dst, int64_t ld_dst, void* stream) {
  MOE_CHECK_ARG(n_rows_in >= 0 && row_bytes >= 0, "moe_scatter_rows: negative extent");
  if (n_rows_in == 0 || row_bytes == 0) return MOE_OK;
  MOE_CHECK_ARG(src && dst && row_indx, "moe_scatter_rows: NULL pointer");
  MOE_CHECK_ARG(row_bytes % 16 == 0 && ld_src % 16 == 0 && ld_dst % 16 == 0 && (uintptr_t)src % 16 == 0 &&
                    (uintptr_t)dst % 16 == 0,
                "moe_scatter_rows: rows must be 16-byte aligned multiples of 16 bytes");
  scatter_rows_kernel<<<grid_for(n_rows_in * (row_bytes / 16), 256), 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)src, ld_src, row_indx, n_rows_in, row_bytes, (uint8_t*)dst, ld_dst);
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Expert-parallel exchange keys.  For every expert-sorted position p (col_sorted[p] = flat token * k + slot, or
// -1): key[p] = source_rank * world + destination_rank, where the source rank is the home of the token and the
// destination rank the owner of the expert.  A stable sort of the positions by this key (done with the same
// counting sort as the expert sort) is the order in which rows travel in both all-to-all exchanges.
namespace {
__global__ void __launch_bounds__(256) ep_keys_kernel(const int32_t* __restrict__ col_sorted,
                                                      const int16_t* __restrict__ expt_indx,
                                                      const int32_t* __restrict__ owner, int64_t n, int entries_per_rank,
                                                      int world, int16_t* __restrict__ keys) {
  for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < n; p += (int64_t)gridDim.x * blockDim.x) {
    const int32_t flat = col_sorted[p];
    int16_t key = -1;
    if (flat >= 0) {
      const int e = expt_indx[flat];
      key = (int16_t)((flat / entries_per_rank) * world + owner[e]);
    }
    keys[p] = key;
  }
}
}  // namespace

extern "C" __attribute__((visibility("default"))) int moe_ep_keys(const int32_t* col_sorted, const int16_t* expt_indx,
                                                                  const int32_t* owner, int64_t n, int entries_per_rank,
                                                                  int world, int16_t* keys, void* stream) {
  MOE_CHECK_ARG(n >= 0 && entries_per_rank > 0 && world > 0 && world * world < 32768, "moe_ep_keys: bad extents");
  if (n == 0) return MOE_OK;
  MOE_CHECK_ARG(col_sorted && expt_indx && owner && keys, "moe_ep_keys: NULL pointer");
  ep_keys_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(col_sorted, expt_indx, owner, n, entries_per_rank,
                                                                      world, keys);
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}

// Per expert-sorted position p of the replicated routing metadata: the global token row this rank pulls for it
// (flat / k when the position's expert is local, -2 = not ours or padding) and the routing weight of that position.
namespace {
__global__ void __launch_bounds__(256) ep_pull_index_kernel(const int32_t* __restrict__ col_sorted,
                                                            const int16_t* __restrict__ expt_indx,
                                                            const float* __restrict__ vals,
                                                            const int32_t* __restrict__ local_expt, int64_t n, int k,
                                                            int32_t* __restrict__ src_row, float* __restrict__ gammas) {
  for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < n; p += (int64_t)gridDim.x * blockDim.x) {
    const int32_t flat = col_sorted[p];
    int32_t row = -2;
    float g = 0.0f;
    if (flat >= 0) {
      g = vals[flat];
      if (local_expt[expt_indx[flat]] >= 0) row = flat / k;
    }
    src_row[p] = row;
    gammas[p] = g;
  }
}
}  // namespace

extern "C" __attribute__((visibility("default"))) int moe_ep_pull_index(const int32_t* col_sorted, const int16_t* expt_indx,
                                                                        const float* vals, const int32_t* local_expt,
                                                                        int64_t n, int k, int32_t* src_row, float* gammas,
                                                                        void* stream) {
  MOE_CHECK_ARG(n >= 0 && k > 0, "moe_ep_pull_index: bad extents");
  if (n == 0) return MOE_OK;
  MOE_CHECK_ARG(col_sorted && expt_indx && vals && local_expt && src_row && gammas, "moe_ep_pull_index: NULL pointer");
  ep_pull_index_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(col_sorted, expt_indx, vals, local_expt, n, k,
                                                                            src_row, gammas);
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}

// Index of the pull combine: for the n_local flat (token, slot) entries of this rank's tokens (flat indices
// [lo, lo + n_local)), the global row of the owners' output buffers that holds the entry's expert output:
// owner[expert] * rows_per_peer + row_sorted[flat], or -1 for a dropped entry (row_sorted < 0).
namespace {
__global__ void __launch_bounds__(256) ep_combine_index_kernel(const int32_t* __restrict__ row_sorted,
                                                               const int16_t* __restrict__ expt_indx,
                                                               const int32_t* __restrict__ owner, int64_t lo, int64_t n_local,
                                                               int64_t rows_per_peer, int32_t* __restrict__ out) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_local; i += (int64_t)gridDim.x * blockDim.x) {
    const int32_t pos = row_sorted[lo + i];
    const int e = expt_indx[lo + i];
    out[i] = (pos < 0 || e < 0) ? -1 : (int32_t)((int64_t)owner[e] * rows_per_peer + pos);
  }
}
}  // namespace

extern "C" __attribute__((visibility("default"))) int moe_ep_combine_index(const int32_t* row_sorted, const int16_t* expt_indx,
                                                                           const int32_t* owner, int64_t lo, int64_t n_local,
                                                                           int64_t rows_per_peer, int32_t* out, void* stream) {
  MOE_CHECK_ARG(lo >= 0 && n_local >= 0 && rows_per_peer > 0, "moe_ep_combine_index: bad extents");
  if (n_local == 0) return MOE_OK;
  MOE_CHECK_ARG(row_sorted && expt_indx && owner && out, "moe_ep_combine_index: NULL pointer");
  ep_combine_index_kernel<<<grid_for(n_local, 256), 256, 0, (cudaStream_t)stream>>>(row_sorted, expt_indx, owner, lo, n_local,
                                                                                   rows_per_peer, out);
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}

// ---------------------------------------------------------------------------------------------------------
// y[t, :] = sum_{j < k} src[row_indx[t * k + j], :]   (row_indx < 0: skipped), fp32 accumulation, bf16 rows.
// The k-way combine of an expert-parallel layer read straight out of the receive buffer of the combine
// exchange, without first scattering the rows back into token order.
namespace {
__global__ void __launch_bounds__(256) gather_reduce_kernel(const __nv_bfloat16* __restrict__ src, int64_t ld_src,
                                                            const int32_t* __restrict__ row_indx, int64_t T, int k,
                                                            int64_t d, __nv_bfloat16* __restrict__ y, int64_t ld_y) {
  const int64_t vec_per_row = d >> 3;
  const int64_t total = T * vec_per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / vec_per_row, c = (i - t * vec_per_row) * 8;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
    for (int s = 0; s < k; ++s) {
      const int32_t r = row_indx[t * k + s];
      if (r < 0) continue;
      const uint4 raw = *reinterpret_cast<const uint4*>(src + (int64_t)r * ld_src + c);
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(e[j]);
    }
    __nv_bfloat16 o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16_rn(acc[j]);
    *reinterpret_cast<uint4*>(y + t * ld_y + c) = *reinterpret_cast<const uint4*>(o);
  }
}
}  // namespace

// The same combine over rows that live on several devices: row_indx holds global rows (buffer = index / rows_per_peer).
// All k loads of a thread are issued before the first is used, so four NVLink reads are in flight per thread.
namespace {
__global__ void __launch_bounds__(128) gather_reduce_peers_kernel(PeerBases peers, int64_t rows_per_peer, int64_t ld_src,
                                                                  const int32_t* __restrict__ row_indx, int64_t T, int k,
                                                                  int64_t d, __nv_bfloat16* __restrict__ y, int64_t ld_y) {
  const int vec_per_row = (int)(d >> 3);
  for (int64_t t = blockIdx.x; t < T; t += gridDim.x) {           // one block per token: no division per element
    for (int c = threadIdx.x; c < vec_per_row; c += 128) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
      for (int s0 = 0; s0 < k; s0 += 4) {
        uint4 raw[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          raw[u] = make_uint4(0, 0, 0, 0);
          const int32_t r = s0 + u < k ? row_indx[t * k + s0 + u] : -1;
          if (r >= 0) {
            const int64_t peer = r / rows_per_peer;
            raw[u] = reinterpret_cast<const uint4*>(peers.base[peer] + (r - peer * rows_per_peer) * ld_src * 2)[c];
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&raw[u]);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(e[j]);
        }
      }
      __nv_bfloat16 o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16_rn(acc[j]);
      reinterpret_cast<uint4*>(y + t * ld_y)[c] = *reinterpret_cast<const uint4*>(o);
    }
  }
}
}  // namespace

extern "C" __attribute__((visibility("default"))) int moe_gather_reduce_rows_peers(const void* const* src_peers, int n_peers,
                                                                                   int64_t rows_per_peer, int64_t ld_src,
                                                                                   const int32_t* row_indx, int64_t T, int k,
                                                                                   int64_t d, void* y, int64_t ld_y,
                                                                                   void* stream) {
  MOE_CHECK_ARG(T >= 0 && k > 0 && d >= 0, "moe_gather_reduce_rows_peers: bad extents");
  if (T == 0 || d == 0) return MOE_OK;
  MOE_CHECK_ARG(src_peers && row_indx && y, "moe_gather_reduce_rows_peers: NULL pointer");
  MOE_CHECK_ARG(n_peers >= 1 && n_peers <= MOE_MAX_PEERS && rows_per_peer > 0,
                "moe_gather_reduce_rows_peers: need 1..%d peers and rows_per_peer > 0", MOE_MAX_PEERS);
  MOE_CHECK_ARG(d % 8 == 0 && ld_src % 8 == 0 && ld_y % 8 == 0 && (uintptr_t)y % 16 == 0,
                "moe_gather_reduce_rows_peers: rows must be 16-byte aligned multiples of 8 bf16");
  PeerBases pb;
  for (int i = 0; i < MOE_MAX_PEERS; ++i) {
    pb.base[i] = i < n_peers ? (const uint8_t*)src_peers[i] : nullptr;
    MOE_CHECK_ARG(i >= n_peers || (pb.base[i] && (uintptr_t)pb.base[i] % 16 == 0),
                  "moe_gather_reduce_rows_peers: peer buffer %d is NULL or not 16-byte aligned", i);
  }
  const int64_t grp_max = (int64_t)moe_sm_count() * 16;
  gather_reduce_peers_kernel<<<(int)(T < grp_max ? T : grp_max), 128, 0, (cudaStream_t)stream>>>(
      pb, rows_per_peer, ld_src, row_indx, T, k, d, (__nv_bfloat16*)y, ld_y);
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}

extern "C" __attribute__((visibility("default"))) int moe_gather_reduce_rows(const void* src, int64_t ld_src,
                                                                             const int32_t* row_indx, int64_t T, int k,
                                                                             int64_t d, void* y, int64_t ld_y, void* stream) {
  MOE_CHECK_ARG(T >= 0 && k > 0 && d >= 0, "moe_gather_reduce_rows: bad extents");
  if (T == 0 || d == 0) return MOE_OK;
  MOE_CHECK_ARG(src && row_indx && y, "moe_gather_reduce_rows: NULL pointer");
  MOE_CHECK_ARG(d % 8 == 0 && ld_src % 8 == 0 && ld_y % 8 == 0 && (uintptr_t)src % 16 == 0 && (uintptr_t)y % 16 == 0,
                "moe_gather_reduce_rows: bf16 rows must be 16-byte aligned multiples of 8 elements");
  gather_reduce_kernel<<<grid_for(T * (d / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)src, ld_src, row_indx, T, k, d, (__nv_bfloat16*)y, ld_y);
  MOE_CHECK_LAUNCH();
  return MOE_OK;
}
