// Flat-addressing VM kernel of the structured-access engine (see tsb_ew.cuh for the addressing and
// tsb_elementwise.cu for the reference semantics), in a translation unit of its own so that it
// compiles beside the blocked kernels.
#include "tsb_vm_exec.cuh"

namespace tsb {

__global__ void __launch_bounds__(256) ew_flat_vm_kernel(const __grid_constant__ FlatParams P) {
  extern __shared__ __align__(16) unsigned vm_smem[];
  const VmRegs<4, FLAT_VM_U> R{vm_smem, (int)blockDim.x, (int)threadIdx.x};
  const long long n_vec = (P.g_hi - P.g_lo) >> 2;
  const long long step = (long long)gridDim.x * blockDim.x * FLAT_VM_U;
  for (long long v0 = (long long)blockIdx.x * blockDim.x * FLAT_VM_U + threadIdx.x; v0 < n_vec; v0 += step) {
    vm_exec<4, FLAT_VM_U, false, true>(
        P.ops, P.n_ops, R,
        [&](int a, unsigned(&r)[FLAT_VM_U][4]) {
#pragma unroll
          for (int u = 0; u < FLAT_VM_U; ++u) {
            const long long v = v0 + (long long)u * blockDim.x;
            if (v < n_vec) {
              flat_load(P.acc[a], P.g_lo + v * 4, r[u]);
            } else {
              r[u][0] = r[u][1] = r[u][2] = r[u][3] = 0u;
            }
          }
        },
        [&](int a, const unsigned(&r)[FLAT_VM_U][4]) {
#pragma unroll
          for (int u = 0; u < FLAT_VM_U; ++u) {
            const long long v = v0 + (long long)u * blockDim.x;
            if (v < n_vec) flat_store(P.acc[a], P.g_lo + v * 4, r[u]);
          }
        },
        [&](int, int, unsigned, const unsigned(&)[4], const unsigned(&)[4], unsigned(&)[4]) {},
        [&](int, int, unsigned, const unsigned(&)[4], const unsigned(&)[4], const unsigned(&)[4]) {});
  }
}

int launch_flat_vm(const FlatParams &F, unsigned ctas, int threads, size_t smem, cudaStream_t s) {
  static SmemLimit lim_flat;
  if (smem > 48 * 1024) TSB_CUDA_OK(allow_dynamic_smem(ew_flat_vm_kernel, 200 * 1024, lim_flat));
  ew_flat_vm_kernel<<<ctas, threads, smem, s>>>(F);
  TSB_LAUNCH_OK("ew_flat_vm_kernel");
  return TSB_OK;
}

}  // namespace tsb
