// Shared helpers for the sm_100a kernels of libmoe_b200.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include "../../include/moe_b200.h"

// per-thread error message, set by every failing entry point
void moe_set_error(const char* fmt, ...);

#define MOE_CHECK_ARG(cond, ...)                 \
  do {                                           \
    if (!(cond)) {                               \
      moe_set_error(__VA_ARGS__);                \
      return MOE_ERR_ARG;                        \
    }                                            \
  } while (0)

#define MOE_CHECK_CUDA(expr)                                                              \
  do {                                                                                    \
    cudaError_t _e = (expr);                                                              \
    if (_e != cudaSuccess) {                                                              \
      moe_set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
      return MOE_ERR_CUDA;                                                                \
    }                                                                                     \
  } while (0)

void moe_count_launch();   // one kernel launch (api.cu keeps the process-wide counter)
#define MOE_CHECK_LAUNCH()              \
  do {                                  \
    moe_count_launch();                 \
    MOE_CHECK_CUDA(cudaGetLastError()); \
  } while (0)

static inline int64_t cdiv64(int64_t a, int64_t b) { return (a + b - 1) / b; }

int moe_sm_count();  // SMs of the current device (cached per device)

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Dispatch a generic lambda on one of the three float element types.
#define MOE_DISPATCH_FLOAT(dtype, T, ...)                                   \
  switch (dtype) {                                                          \
    case MOE_F32: { using T = float; __VA_ARGS__; break; }                  \
    case MOE_F16: { using T = __half; __VA_ARGS__; break; }                 \
    case MOE_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }         \
    default: moe_set_error("unsupported dtype %d", (int)(dtype)); return MOE_ERR_ARG; \
  }
