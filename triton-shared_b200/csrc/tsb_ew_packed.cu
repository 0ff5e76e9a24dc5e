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
#include "tsb_ew_packed.cuh"

namespace tsb {

// Launch the packed kernel for blocks of `items` lane-vectors (4 <= items <= 1024, a power of two).
// Returns TSB_ERR_UNSUPPORTED without reporting when the body's registers do not fit shared memory.
int launch_ew_packed(const EwParams &P, int items, int regs_used, cudaStream_t s) {
  bool lean = !P.indirect && items >= PACKED_LEAN_U;
  for (int a = 0; a < P.n_acc && lean; ++a) lean = lean_ok(P.acc[a], P.size);
  const int U = lean ? PACKED_LEAN_U : 4, threads = 1024 / U;
  int lg_g = 0;
  while ((U << (lg_g + 1)) <= items) ++lg_g;  // G = items / U threads per program, at most `threads`
  const size_t smem = (size_t)regs_used * 4 * 1024 * sizeof(unsigned);  // U * threads = 1024 lane-vectors
  if (smem > 200 * 1024) return TSB_ERR_UNSUPPORTED;
  const long long n_prog = P.pid_hi - P.pid_lo;
  // programs of one set: as many as the thread groups of a CTA, bounded by the states a CTA holds
  int per_pass = threads >> lg_g;
  if (per_pass * P.n_acc > PACKED_STATES) per_pass = PACKED_STATES / P.n_acc;
  // sets per CTA iteration: fill the state table, but keep every SM busy with several CTAs
  int rounds = PACKED_STATES / (per_pass * P.n_acc);
  const long long want_ctas = (long long)sm_count() * 4 * 2;
  while (rounds > 1 && (n_prog + (long long)per_pass * rounds - 1) / ((long long)per_pass * rounds) < want_ctas) --rounds;
  const long long per_cta = (long long)per_pass * rounds;
  long long ctas = (n_prog + per_cta - 1) / per_cta;
  const long long cap = (long long)sm_count() * 4 * 8;
  if (ctas > cap) ctas = cap;
  const dim3 grid((unsigned)ctas);
  if (!lean) return launch_packed_general(P, P.indirect != 0, grid, smem, s, lg_g, per_pass, rounds);
  if (P.n_loops) return launch_packed_lean_loops(P, grid, smem, s, lg_g, per_pass, rounds);
  return launch_packed_lean(P, grid, smem, s, lg_g, per_pass, rounds);
}

int launch_packed_lean(const EwParams &P, dim3 grid, size_t smem, cudaStream_t s, int lg_g, int per_pass, int rounds) {
  return launch_packed_instance<false, PACKED_LEAN, PACKED_LEAN_U>(P, grid, smem, s, lg_g, per_pass, rounds);
}

}  // namespace tsb
