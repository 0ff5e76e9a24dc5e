// Kernel template of the packed VM form (see tsb_ew_packed.cu); instantiated in several translation
// units so that they compile side by side.
#pragma once
#include "tsb_vm_exec.cuh"

namespace tsb {

constexpr int PACKED_STATES = 256;
constexpr int PACKED_LEAN_U = 4;  // (program, access) states a CTA holds at a time

// MODE: which accessors the body needs; the smaller sets cost fewer registers and instructions
//   PACKED_LEAN      every access is lean (lean_ok)
//   PACKED_GENERAL   probes, wrap terms, strided or unaligned inner dims
//   PACKED_INDIRECT  PACKED_GENERAL plus data-dependent accesses
enum { PACKED_LEAN = 0, PACKED_GENERAL = 1, PACKED_INDIRECT = 2 };

// U lane-vectors per thread and 1024 / U threads per CTA.  U = 8 (32 lanes per decoded op, 128
// registers per thread) measured slower than U = 4 on every body tried: the halved warp count
// costs more than the shared decode saves.
template <bool LOOPS, int MODE, int U>
__global__ void __launch_bounds__(1024 / U, MODE == PACKED_LEAN ? 3 : 4)
    ew_vm_packed_kernel(const __grid_constant__ EwParams P, int lg_g, int per_pass, int rounds) {
  constexpr int VEC = 4;
  extern __shared__ __align__(16) unsigned vm_smem[];
  __shared__ ProgState shared_state[PACKED_STATES];
  // the op list and the compact access descriptors, read from shared memory in the body: indexed
  // reads of kernel parameters (constant bank) are far slower than shared-memory reads
  __shared__ __align__(16) tsb_op s_ops[TSB_MAX_OPS];
  __shared__ __align__(16) LeanAcc s_lean[TSB_MAX_ACCESSES];
  for (int k = (int)threadIdx.x; k < P.n_ops; k += (int)blockDim.x) s_ops[k] = P.ops[k];
  if (MODE == PACKED_LEAN && (int)threadIdx.x < P.n_acc) make_lean(P.acc[threadIdx.x], P.size, s_lean[threadIdx.x]);
  const VmRegs<VEC, U> R{vm_smem, (int)blockDim.x, (int)threadIdx.x};
  const int G = 1 << lg_g;
  const int sh1 = P.lg[2], sh0 = P.lg[2] + P.lg[1];
  const int slot = (int)threadIdx.x >> lg_g;   // which program of a set this thread works on
  const int within = (int)threadIdx.x & (G - 1);
  const bool member = slot < per_pass;         // threads beyond the last whole program of a set idle
  const long long n_prog = P.pid_hi - P.pid_lo;
  const int per_cta = per_pass * rounds;       // programs per CTA iteration
  const int n_states = per_cta * P.n_acc;
  // lane coordinates of this thread's sub-items do not depend on the program
  int c0[U], c1[U], c2[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int l = (within + u * G) * VEC;
    c0[u] = l >> sh0;
    c1[u] = (l >> sh1) & (P.size[1] - 1);
    c2[u] = l & (P.size[2] - 1);
  }
  grid_dependency_wait();
  grid_launch_dependents();
  for (long long first = (long long)blockIdx.x * per_cta; first < n_prog; first += (long long)gridDim.x * per_cta) {
    for (long long q = 0; q < (LOOPS ? P.total_trips : 1); ++q) {
      // later iterations of a program see the stores of earlier ones (same CTA); the previous
      // iteration's states are no longer read
      if (LOOPS) __threadfence_block();
      __syncthreads();
      for (int t = (int)threadIdx.x; t < n_states; t += (int)blockDim.x) {
        const int sl = t / P.n_acc, a = t - sl * P.n_acc;
        if (first + sl < n_prog) {
          long long qx, qy, qz;
          split_pid(P.grid, P.order, P.pid_lo + first + sl, qx, qy, qz);
          if (LOOPS) {
            int it[TSB_MAX_LOOPS];
            loop_counters(P, q, it);
            program_state_loops(P.acc[a], P.size, qx, qy, qz, it, shared_state[t]);
          } else {
            program_state(P.acc[a], P.size, qx, qy, qz, shared_state[t]);
          }
        }
      }
      __syncthreads();
      if (!member) continue;
      for (int r = 0; r < rounds; ++r) {
        const int sl = r * per_pass + slot;
        if (first + sl >= n_prog) break;
        const ProgState *S = shared_state + sl * P.n_acc;
        vm_exec<VEC, U, MODE == PACKED_INDIRECT, MODE == PACKED_LEAN>(
            s_ops, P.n_ops, R,
            [&](int a, unsigned(&v)[U][VEC]) {
              if (MODE == PACKED_LEAN) {
                lean_load<U>(s_lean[a], S[a], c0, c1, c2, v);
              } else {
#pragma unroll
                for (int u = 0; u < U; ++u) load_vec<VEC>(P.acc[a], S[a], c0[u], c1[u], c2[u], v[u]);
              }
            },
            [&](int a, const unsigned(&v)[U][VEC]) {
              if (MODE == PACKED_LEAN) {
                lean_store<U>(s_lean[a], S[a], c0, c1, c2, v);
              } else {
#pragma unroll
                for (int u = 0; u < U; ++u) store_vec<VEC>(P.acc[a], S[a], c0[u], c1[u], c2[u], v[u]);
              }
            },
            [&](int a, int u, unsigned flags, const unsigned(&ix)[VEC], const unsigned(&mk)[VEC], unsigned(&v)[VEC]) {
              load_vec_indirect<VEC>(P.acc[a], S[a], c0[u], c1[u], c2[u], flags & MEM_INDEX, flags & MEM_MASK, ix, mk, v);
            },
            [&](int a, int u, unsigned flags, const unsigned(&ix)[VEC], const unsigned(&mk)[VEC],
                const unsigned(&v)[VEC]) {
              store_vec_indirect<VEC>(P.acc[a], S[a], c0[u], c1[u], c2[u], flags & MEM_INDEX, flags & MEM_MASK, ix, mk, v);
            });
      }
    }
  }
}

template <bool LOOPS, int MODE, int U>
inline int launch_packed_instance(const EwParams &P, dim3 grid, size_t smem, cudaStream_t s, int lg_g, int per_pass,
                                  int rounds) {
  static SmemLimit lim;
  TSB_CUDA_OK(allow_dynamic_smem(ew_vm_packed_kernel<LOOPS, MODE, U>, 200 * 1024, lim));
  TSB_CUDA_OK(launch_pdl(ew_vm_packed_kernel<LOOPS, MODE, U>, grid, dim3(1024 / U), smem, s, P, lg_g, per_pass, rounds));
  return TSB_OK;
}

// one per translation unit
int launch_packed_lean(const EwParams &P, dim3 grid, size_t smem, cudaStream_t s, int lg_g, int per_pass, int rounds);
int launch_packed_lean_loops(const EwParams &P, dim3 grid, size_t smem, cudaStream_t s, int lg_g, int per_pass, int rounds);
int launch_packed_general(const EwParams &P, bool indirect, dim3 grid, size_t smem, cudaStream_t s, int lg_g,
                          int per_pass, int rounds);

}  // namespace tsb
