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

// Barrier over the `threads` threads (a multiple of 32) of group `slot` (0..3) of a CTA: a named
// barrier per group, with the ids written out so that the kernel reserves five barriers, not all 16.
__device__ __forceinline__ void group_barrier(int slot, int threads) {
  switch (slot) {
    case 0: asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory"); break;
    case 1: asm volatile("bar.sync 2, %0;" ::"r"(threads) : "memory"); break;
    case 2: asm volatile("bar.sync 3, %0;" ::"r"(threads) : "memory"); break;
    default: asm volatile("bar.sync 4, %0;" ::"r"(threads) : "memory"); break;
  }
}

// One combination of a fold with the combiner known at compile time; NARROW: the type is less than
// 32 bits wide and every partial result is rounded / wrapped to it.
template <int COMB, bool NARROW>
__device__ __forceinline__ unsigned fold2(int ty, unsigned a, unsigned b) {
  if constexpr (COMB >= TSB_OP_ADDF && COMB < TSB_OP_EXP) {
    const float r = binf(COMB, __uint_as_float(a), __uint_as_float(b));
    return __float_as_uint(NARROW ? round_to(r, ty) : r);
  } else {
    const unsigned r = bini(COMB, a, b);
    return NARROW ? wrap_to(r, ty) : r;
  }
}

// TSB_OP_REDUCE in the packed kernel: every lane of v := the fold of v over all lanes of the program.
// This thread's lanes in order, then the G threads of the program: shuffles inside a warp, one
// partial per warp through shared memory behind a barrier that only the program's own warps join.
template <int COMB, bool NARROW, int U>
__device__ __forceinline__ void fold_group(unsigned (&v)[U][4], int ty, int G, int lg_g, int slot, unsigned *s_red) {
  unsigned r = v[0][0];
#pragma unroll
  for (int u = 0; u < U; ++u)
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (u | k) r = fold2<COMB, NARROW>(ty, r, v[u][k]);
  const int lane = (int)threadIdx.x & 31;
  const int span = G < 32 ? G : 32;  // threads of this program inside the warp
  const unsigned peers = span == 32 ? 0xffffffffu : (((1u << span) - 1u) << (lane & ~(span - 1)));
  for (int s2 = span >> 1; s2 > 0; s2 >>= 1) r = fold2<COMB, NARROW>(ty, r, __shfl_xor_sync(peers, r, s2));
  if (G > 32) {
    const int warp = (int)threadIdx.x >> 5, first_warp = (slot << lg_g) >> 5, n_warps = G >> 5;
    if (lane == 0) s_red[warp] = r;
    group_barrier(slot, G);
    r = s_red[first_warp];
    for (int w = 1; w < n_warps; ++w) r = fold2<COMB, NARROW>(ty, r, s_red[first_warp + w]);
    group_barrier(slot, G);  // partials read before reuse
  }
#pragma unroll
  for (int u = 0; u < U; ++u)
#pragma unroll
    for (int k = 0; k < 4; ++k) v[u][k] = r;
}

// U lane-vectors per thread and 1024 / U threads per CTA.  U = 8 (32 lanes per decoded op, 128
// registers per thread) measured slower than U = 4 on every body tried: the halved warp count
// costs more than the shared decode saves.
template <bool LOOPS, int MODE, int U>
__global__ void __launch_bounds__(1024 / U, 3)
    ew_vm_packed_kernel(const __grid_constant__ EwParams P, int lg_g, int per_pass, int rounds) {
  constexpr int VEC = 4;
  extern __shared__ __align__(16) unsigned vm_smem[];
  __shared__ ProgState shared_state[PACKED_STATES];
  // the op list and the compact access descriptors, read from shared memory in the body: indexed
  // reads of kernel parameters (constant bank) are far slower than shared-memory reads
  __shared__ unsigned s_red[32];  // one partial per warp of the CTA (TSB_OP_REDUCE across warps)
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
            },
            [&](const tsb_op &op, unsigned(&v)[U][VEC]) {
              const bool narrow = dtype_size(op.type) != 4;
              switch ((int)op.imm) {  // one decision per op: the fold itself is straight-line code
#define TSB_FOLD_CASE(C)                                                                   \
  case C:                                                                                  \
    if (narrow) fold_group<C, true, U>(v, op.type, G, lg_g, slot, s_red);                  \
    else fold_group<C, false, U>(v, op.type, G, lg_g, slot, s_red);                        \
    break;
                TSB_FOLD_CASE(TSB_OP_ADDF) TSB_FOLD_CASE(TSB_OP_MULF) TSB_FOLD_CASE(TSB_OP_MAXNUMF)
                TSB_FOLD_CASE(TSB_OP_MINNUMF) TSB_FOLD_CASE(TSB_OP_MAXIMUMF) TSB_FOLD_CASE(TSB_OP_MINIMUMF)
                TSB_FOLD_CASE(TSB_OP_ADDI) TSB_FOLD_CASE(TSB_OP_MULI) TSB_FOLD_CASE(TSB_OP_MINSI)
                TSB_FOLD_CASE(TSB_OP_MAXSI) TSB_FOLD_CASE(TSB_OP_MINUI) TSB_FOLD_CASE(TSB_OP_MAXUI)
                TSB_FOLD_CASE(TSB_OP_ANDI) TSB_FOLD_CASE(TSB_OP_ORI) TSB_FOLD_CASE(TSB_OP_XORI)
#undef TSB_FOLD_CASE
                default: break;
              }
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
