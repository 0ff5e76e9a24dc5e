// Packed form of the blocked VM kernel of the structured-access engine, for programs of at most
// 1024 lane-vectors (see tsb_elementwise.cu for the reference semantics of the accesses).
//
// A program of `items` lane-vectors is shared by G = items / U consecutive threads, each carrying U
// vectors G apart (consecutive threads touch consecutive vectors); programs are dealt to thread
// groups in the walk order of the launch, so a CTA of 256 threads works on 256 / G programs at once
// and small blocks still fill it.  A CTA takes `rounds` such sets of programs at a time: the access
// state (offset, wrap offsets, mask extents) of all of them is derived once per (program, access),
// one per thread, into shared memory, and read from there when the body reaches the load or store:
// one barrier pair per `rounds` sets, no per-thread program bookkeeping in registers.
#include "tsb_vm_exec.cuh"

namespace tsb {

constexpr int PACKED_STATES = 256;  // (program, access) states a CTA holds at a time

// MODE: which accessors the body needs; the smaller sets cost fewer registers and instructions
//   PACKED_LEAN      every access is lean (lean_ok)
//   PACKED_GENERAL   probes, wrap terms, strided or unaligned inner dims
//   PACKED_INDIRECT  PACKED_GENERAL plus data-dependent accesses
enum { PACKED_LEAN = 0, PACKED_GENERAL = 1, PACKED_INDIRECT = 2 };

template <bool LOOPS, int MODE>
__global__ void __launch_bounds__(256, 4)
    ew_vm_packed_kernel(const __grid_constant__ EwParams P, int lg_g, int per_pass, int rounds) {
  constexpr int VEC = 4, U = 4;
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
        vm_exec<VEC, U, MODE == PACKED_INDIRECT>(
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

// Launch the packed kernel for blocks of `items` lane-vectors (4 <= items <= 1024, a power of two).
// Returns TSB_ERR_UNSUPPORTED without reporting when the body's registers do not fit shared memory.
int launch_ew_packed(const EwParams &P, int items, int regs_used, cudaStream_t s) {
  int lg_g = 0;
  while ((4 << (lg_g + 1)) <= items) ++lg_g;  // G = items / 4 threads per program, at most 256
  const size_t smem = (size_t)regs_used * 4 * 4 * 256 * sizeof(unsigned);
  if (smem > 200 * 1024) return TSB_ERR_UNSUPPORTED;
  const long long n_prog = P.pid_hi - P.pid_lo;
  // programs of one set: as many as the thread groups of a CTA, bounded by the states a CTA holds
  int per_pass = 256 >> lg_g;
  if (per_pass * P.n_acc > PACKED_STATES) per_pass = PACKED_STATES / P.n_acc;
  // sets per CTA iteration: fill the state table, but keep every SM busy with several CTAs
  int rounds = PACKED_STATES / (per_pass * P.n_acc);
  const long long want_ctas = (long long)sm_count() * 4 * 2;
  while (rounds > 1 && (n_prog + (long long)per_pass * rounds - 1) / ((long long)per_pass * rounds) < want_ctas) --rounds;
  const long long per_cta = (long long)per_pass * rounds;
  long long ctas = (n_prog + per_cta - 1) / per_cta;
  const long long cap = (long long)sm_count() * 4 * 8;
  if (ctas > cap) ctas = cap;
  const dim3 grid((unsigned)ctas), block(256);
#define TSB_PACKED_LAUNCH(L, M)                                                                       \
  {                                                                                                   \
    static SmemLimit lim;                                                                             \
    TSB_CUDA_OK(allow_dynamic_smem(ew_vm_packed_kernel<L, M>, 200 * 1024, lim));                      \
    TSB_CUDA_OK(launch_pdl(ew_vm_packed_kernel<L, M>, grid, block, smem, s, P, lg_g, per_pass, rounds)); \
  }
  bool lean = !P.indirect;
  for (int a = 0; a < P.n_acc && lean; ++a) lean = lean_ok(P.acc[a], P.size);
  const int mode = P.indirect ? PACKED_INDIRECT : (lean ? PACKED_LEAN : PACKED_GENERAL);
  if (P.n_loops) {
    if (mode == PACKED_LEAN) TSB_PACKED_LAUNCH(true, PACKED_LEAN)
    else if (mode == PACKED_GENERAL) TSB_PACKED_LAUNCH(true, PACKED_GENERAL)
    else TSB_PACKED_LAUNCH(true, PACKED_INDIRECT)
  } else {
    if (mode == PACKED_LEAN) TSB_PACKED_LAUNCH(false, PACKED_LEAN)
    else if (mode == PACKED_GENERAL) TSB_PACKED_LAUNCH(false, PACKED_GENERAL)
    else TSB_PACKED_LAUNCH(false, PACKED_INDIRECT)
  }
#undef TSB_PACKED_LAUNCH
  return TSB_OK;
}

}  // namespace tsb
