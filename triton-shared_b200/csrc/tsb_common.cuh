// Shared host/device helpers for the tsb200 library (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include "tsb200.h"

namespace tsb {

// Per-thread error text behind tsb_last_error().
void set_error(const char *fmt, ...);
int fail(int code, const char *fmt, ...);

#define TSB_CUDA_OK(expr)                                                                  \
  do {                                                                                     \
    cudaError_t e__ = (expr);                                                              \
    if (e__ != cudaSuccess)                                                                \
      return ::tsb::fail(TSB_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), \
                         __FILE__, __LINE__);                                              \
  } while (0)

// Launch check that does not synchronise: reports configuration errors only.
#define TSB_LAUNCH_OK(what)                                                                \
  do {                                                                                     \
    cudaError_t e__ = cudaGetLastError();                                                  \
    if (e__ != cudaSuccess)                                                                \
      return ::tsb::fail(TSB_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e__)); \
  } while (0)

int sm_count();

__host__ __device__ inline int dtype_size(int dt) {
  switch (dt) {
    case TSB_F32: case TSB_I32: case TSB_U32: return 4;
    case TSB_F16: case TSB_BF16: case TSB_I16: case TSB_U16: return 2;
    case TSB_I8: case TSB_I1: case TSB_U8: return 1;
    case TSB_I64: case TSB_F64: return 8;
  }
  return 0;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace tsb
