// Tensor-pipe roof of one MMA kind, measured: every SM runs one CTA whose single issuing thread streams back-to-back
// tcgen05.mma instructions (M = 128, N = 256) over operand tiles that stay in shared memory, so nothing but the tensor
// pipe itself bounds the rate.  The benchmark divides the block-scaled kernels' throughput by these numbers instead of
// by a multiple of the bf16 figure.  (The reference quotes such peaks from a table: triton_kernels/roofline.py and
// python/tutorials/gluon/11-tcgen05-mma-scaled.py:1530-1535; here they are taken on the device at hand.)
#include "gemm_tc_common.cuh"

namespace {

constexpr int ROOF_N = 256;

__device__ __forceinline__ void roof_mma(int kind, uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                         uint32_t acc) {
  switch (kind) {
    case 0:
      asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
                   "l"(a), "l"(b), "r"(idesc), "r"(acc)
                   : "memory");
      break;
    case 1:
      asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
                   "l"(a), "l"(b), "r"(idesc), "r"(acc)
                   : "memory");
      break;
    case 2:
      asm volatile(
          "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
          "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}" ::"r"(d),
          "l"(a), "l"(b), "r"(idesc), "r"(sfa), "r"(sfb), "r"(acc)
          : "memory");
      break;
    default:
      asm volatile(
          "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
          "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%4], [%5], p;\n\t}" ::"r"(d),
          "l"(a), "l"(b), "r"(idesc), "r"(sfa), "r"(sfb), "r"(acc)
          : "memory");
      break;
  }
}

// kind 0: bf16 x bf16 (K = 16 per instruction); 1: e4m3 x e4m3 (K = 32); 2: e2m1 (byte-padded) x e4m3 with e8m0 block
// scales (K = 32); 3: e2m1 x e2m1 packed with e8m0 block scales (K = 64).  Every instruction reads 32 bytes of K per row.
__global__ void __launch_bounds__(128, 1) tensor_roof_kernel(int kind, int iters, int32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  const int warp = threadIdx.x >> 5;
  // A: 128 rows x 128 B, B: 256 rows x 128 B (128-byte swizzle, K-major); zeros are as good as any data for the rate
  for (int i = threadIdx.x; i < (128 + ROOF_N) * 128 / 16; i += blockDim.x) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;
  // scale columns (256 ..): all-zero e8m0 bytes = 2^-127, finite
  {
    const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16) + 256u;
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(taddr),
                 "r"(0u)
                 : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (threadIdx.x == 0) {
    Ctl ctl{&s_abort, status};
    uint32_t idesc;
    if (kind == 0) idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(ROOF_N >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    else if (kind == 1) idesc = (1u << 4) | ((uint32_t)(ROOF_N >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    else if (kind == 2) idesc = (5u << 7) | ((uint32_t)(ROOF_N >> 3) << 17) | (1u << 23) | (1u << 27);
    else idesc = (1u << 7) | (1u << 10) | ((uint32_t)(ROOF_N >> 3) << 17) | (1u << 23) | (1u << 27);
    const uint64_t adesc = make_desc(sbase), bdesc = make_desc(sbase + 128 * 128);
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        uint32_t id = idesc;
        if (kind == 2) id |= ((uint32_t)kk << 4) | ((uint32_t)kk << 29);           // scale byte of this k group
        if (kind == 3) id |= ((uint32_t)(kk & 1) * 2u << 4) | ((uint32_t)(kk & 1) * 2u << 29);
        roof_mma(kind, tmem, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), id, tmem + 256u, tmem + 260u, (it | kk) ? 1u : 0u);
      }
    }
    mma_commit(smem_u32(&bar));
    mbar_wait(smem_u32(&bar), 0, ctl, 701);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
}

}  // namespace

// Runs the loop on `stream` with one CTA per SM; the caller times it (CUDA events) and converts with
// *flop_out = SMs x iters x 4 x 2 x 128 x 256 x K(kind).
extern "C" __attribute__((visibility("default"))) int moe_tensor_roof(int kind, int iters, double* flop_out, int32_t* status,
                                                                      void* stream) {
  MOE_CHECK_ARG(kind >= 0 && kind <= 3 && iters > 0 && iters <= (1 << 20), "moe_tensor_roof: kind 0..3, 1 <= iters <= 2^20");
  const int smem = (128 + ROOF_N) * 128 + 1024;
  MOE_CHECK_CUDA(cudaFuncSetAttribute(tensor_roof_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  const int sms = moe_sm_count();
  tensor_roof_kernel<<<sms, 128, smem, (cudaStream_t)stream>>>(kind, iters, status);
  MOE_CHECK_LAUNCH();
  static const int k_per[4] = {16, 32, 32, 64};
  if (flop_out) *flop_out = (double)sms * iters * 4.0 * 2.0 * 128.0 * ROOF_N * k_per[kind];
  return MOE_OK;
}
