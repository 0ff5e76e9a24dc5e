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
// Current device ordinal clamped to [0, 64): index for per-device host-side caches.
int device_slot();
// Whether kernels are launched with programmatic stream serialization (default on; the
// environment variable TSB_PDL=0 turns it off).
bool pdl_enabled();

// Raise a kernel's dynamic shared-memory limit.  The attribute belongs to the (function, device)
// pair, so the high-water mark already set is remembered per device ordinal: a second device
// used by the same process gets its own call.  A race between host threads at worst repeats it.
struct SmemLimit {
  int set[64];
};
template <typename K>
inline cudaError_t allow_dynamic_smem(K kernel, size_t bytes, SmemLimit &st) {
  if (bytes <= 48 * 1024) return cudaSuccess;
  const int d = device_slot();
  if (st.set[d] >= (int)bytes) return cudaSuccess;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e == cudaSuccess) st.set[d] = (int)bytes;
  return e;
}

// Programmatic dependent launch: a kernel launched through launch_pdl may become resident while
// the kernel before it on the stream is still draining.  It must call grid_dependency_wait()
// before its first access to global memory (the wait returns once the preceding kernel has
// completed and its writes are visible) and calls grid_launch_dependents() once its own CTAs
// no longer compete for SM slots.  Both are no-ops for a kernel launched the ordinary way, and a
// preceding kernel that never signals simply releases its dependents when it completes.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                              Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

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
