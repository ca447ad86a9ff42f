// Error reporting, version and device facts of the C ABI.
#include "common.cuh"
#include <stdarg.h>
#include <atomic>

static thread_local char g_err[512] = "";

void moe_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int moe_sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

static std::atomic<uint64_t> g_launches{0};
void moe_count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
extern "C" __attribute__((visibility("default"))) uint64_t moe_launch_count(void) { return g_launches.load(); }

extern "C" __attribute__((visibility("default"))) const char* moe_last_error(void) { return g_err; }
extern "C" __attribute__((visibility("default"))) int moe_abi_version(void) { return 1; }

extern "C" __attribute__((visibility("default"))) int moe_device_info(int device, MoeDeviceInfo* out) {
  MOE_CHECK_ARG(out != nullptr, "moe_device_info: out is NULL");
  cudaDeviceProp p;
  MOE_CHECK_CUDA(cudaGetDeviceProperties(&p, device));
  out->sm_count = p.multiProcessorCount;
  out->cc_major = p.major;
  out->cc_minor = p.minor;
  out->smem_per_block_optin = p.sharedMemPerBlockOptin;
  out->l2_bytes = (size_t)p.l2CacheSize;
  out->total_mem = p.totalGlobalMem;
  return MOE_OK;
}
