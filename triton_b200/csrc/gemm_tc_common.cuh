// Pieces shared by the tensor-core GEMM kernels: tile constants, PTX wrappers (mbarrier, bulk and cp.async copies,
// tcgen05 descriptors / MMA / tensor-memory loads), the in-register MXFP4 -> bf16 conversion, output stores and the
// token-tile schedule.
#pragma once
#include "gemm_common.cuh"
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_bf16.h>
#include <mutex>

namespace {

constexpr int HALF_M = 128;           // token rows of one MMA (MMA M)
constexpr int HALF_N = 128;           // weight rows of one weight tile in memory; a CTA tile spans NH of them
constexpr int BLOCK_K = 64;           // k per pipeline stage: one 128-byte swizzle row of bf16
constexpr int TILE_K = 128;           // k extent of a weight tile in global memory (two stages)
constexpr int SUBTILE_BYTES = 128 * 128;                 // 128 rows x 128 bytes (64 bf16)
constexpr int RAWV_BYTES = HALF_N * BLOCK_K / 2;        // 4 KB: half of an 8 KB weight tile ([2 groups][128 rows][16 B])
constexpr int RAWS_BYTES = HALF_N * 4;                  // 512 B: the scale tile of the whole 128-k weight tile
constexpr int TMEM_COLS = 512;                           // two accumulator buffers of MH x 128 columns (256 used when MH = 1)
constexpr int MAX_PREFIX_EXPERTS = 512;                  // experts the 256-row tile schedule can index

constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;      // a wait that lasts 2 s aborts the CTA

// ---- PTX wrappers -------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// try_wait parks the thread in hardware until the phase completes or an implementation-defined time passes
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
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
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

struct Ctl {
  volatile int* abort_flag;   // shared memory
  int32_t* status;            // global, may be null
};

// Bounded wait.  Returns false when the CTA is aborting (this wait expired, or another one did).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const Ctl& ctl, int code) {
  if (mbar_try(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (;;) {
    if (mbar_try(bar, parity)) return true;
    if (*ctl.abort_flag) return false;
    if (global_ns() - t0 > WAIT_LIMIT_NS) {
      *ctl.abort_flag = 1;
      if (ctl.status) atomicExch(ctl.status, code);
      return false;
    }
  }
}

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// arrive on `bar` once every cp.async this thread has issued so far has landed (the barrier's expected count
// already includes this arrival)
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);          // start address, 16-byte units
  d |= (uint64_t)1 << 16;                            // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                            // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                            // 128-byte swizzle
  return d;
}

// instruction descriptor: D fp32, A/B bf16, both K-major, N = 128, M = 128
__device__ __forceinline__ constexpr uint32_t make_idesc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(HALF_M >> 4) << 24);
}

__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// One box of the tensor map (64 bf16 x 128 rows) starting at column `col`, row `row`, written to `dst` in the tensor
// map's 128-byte swizzle; rows or columns outside the tensor read as zeros.  `col` * 2 bytes must be a multiple of 16.
__device__ __forceinline__ void tma_tile_2d(uint32_t dst, const CUtensorMap* tmap, int col, int row, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(tmap), "r"(col), "r"(row), "r"(bar)
      : "memory");
}

// ---- shared-memory accesses by 32-bit shared address: the shared-memory base of these kernels is an aligned-up
// generic pointer, through which the compiler can only emit generic loads and stores (address-space check on every
// access, tracked like global loads); these go straight to the shared-memory pipe
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds8(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, const uint4& v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ---- weight dequantisation ---------------------------------------------------------------------------
// `w` holds 8 e2m1 codes of one row: nibble p of the low half-word is k = 2p, of the high half-word k = 2p+1.
// The 3 magnitude bits dropped at bf16 bit 6 give value * 2^-126; one bf16x2 multiply by 2^(s-1)
// (s = e8m0 byte) gives value * 2^(s-127) exactly.  Byte 0 multiplies by 0.0 as in the reference's upcast
// (scale bits s << 7); bytes above 128 would overflow the single factor and take two multiplies.
__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// pair i of word w -> bf16x2 bit pattern of (value * 2^-126): magnitude to bits 8:6 / 24:22, sign to 15 / 31
template <int I> __device__ __forceinline__ uint32_t e2m1_pair(uint32_t w) {
  const uint32_t mag = (I < 2 ? (w << (6 - 4 * I)) : (w >> (4 * I - 6))) & 0x01C001C0u;
  const uint32_t sgn = (w << (12 - 4 * I)) & 0x80008000u;
  return mag | sgn;
}
__device__ __forceinline__ uint4 dequant8(uint32_t w, uint32_t c2) {
  return make_uint4(bf16x2_mul(e2m1_pair<0>(w), c2), bf16x2_mul(e2m1_pair<1>(w), c2),
                    bf16x2_mul(e2m1_pair<2>(w), c2), bf16x2_mul(e2m1_pair<3>(w), c2));
}
__device__ __forceinline__ uint4 dequant8_wide(uint32_t w, uint32_t sb) {      // scale bytes above 128
  const uint32_t s2 = (sb << 7) | (sb << 23);
  const uint32_t k = 0x7E807E80u;                                               // 2^126
  return make_uint4(bf16x2_mul(bf16x2_mul(e2m1_pair<0>(w), k), s2), bf16x2_mul(bf16x2_mul(e2m1_pair<1>(w), k), s2),
                    bf16x2_mul(bf16x2_mul(e2m1_pair<2>(w), k), s2), bf16x2_mul(bf16x2_mul(e2m1_pair<3>(w), k), s2));
}

// store N consecutive outputs of one row; `vec` selects 16-byte stores, `n_valid` bounds the scalar path
template <typename TY, int N> __device__ __forceinline__ void store_out(TY* dst, const float (&v)[N], bool vec, int n_valid) {
  if (vec) {
    if constexpr (sizeof(TY) == 2) {
#pragma unroll
      for (int j = 0; j < N; j += 8) {
        __nv_bfloat162 h[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) h[q] = __floats2bfloat162_rn(v[j + 2 * q], v[j + 2 * q + 1]);
        *reinterpret_cast<uint4*>(dst + j) = *reinterpret_cast<const uint4*>(h);
      }
    } else {
#pragma unroll
      for (int j = 0; j < N; j += 4)
        *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < N; ++j)
      if (j < n_valid) dst[j] = from_f32<TY>(v[j]);
  }
}

// =========================================================================================================
// Token-tile -> (expert, first row, valid rows).  MH = 1 follows the block schedule for blocks of 128 rows.
// MH = 2 pairs consecutive 128-row blocks of one expert: tile j of expert e covers rows [256 j, 256 j + 256);
// `prefix` (shared memory) holds the exclusive prefix of ceil(slice_sizes[e] / 256) over experts.
template <int MH>
__device__ __forceinline__ bool map_tile(const GemmParams& p, const int32_t* prefix, int64_t pid_m, int& e,
                                         int64_t& row0, int& rows) {
  if constexpr (MH == 1) {
    return gemm_map_block<HALF_M>(p, pid_m, e, row0, rows);
  } else {
    if (p.slice_sizes == nullptr) return gemm_map_block<2 * HALF_M>(p, pid_m, e, row0, rows);
    int lo = 0, hi = p.E;                         // largest e with prefix[e] <= pid_m
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (prefix[mid] <= pid_m) lo = mid; else hi = mid;
    }
    e = lo;
    const int j = (int)(pid_m - prefix[lo]);
    row0 = (int64_t)p.slice_offs[e] + (int64_t)j * (2 * HALF_M);
    rows = min(2 * HALF_M, p.slice_sizes[e] - j * (2 * HALF_M));
    return rows > 0;
  }
}

// Tensor map of the activation matrix: bf16 [rows_x, K], row pitch ld_x elements, boxes of 128 rows x 64 columns,
// 128-byte swizzle, out-of-range elements read as zero.
inline int make_x_map(const GemmParams& p, CUtensorMap* map) {
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
  const cuuint64_t dims[2] = {(cuuint64_t)p.K, (cuuint64_t)p.rows_x};
  const cuuint64_t strides[1] = {(cuuint64_t)p.ld_x * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BLOCK_K, (cuuint32_t)HALF_M};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(p.x), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    moe_set_error("moe_grouped_gemm: cuTensorMapEncodeTiled failed with code %d (rows %lld, K %d, pitch %lld)", (int)r,
                  (long long)p.rows_x, p.K, (long long)p.ld_x);
    return MOE_ERR_CUDA;
  }
  return MOE_OK;
}

}  // namespace
