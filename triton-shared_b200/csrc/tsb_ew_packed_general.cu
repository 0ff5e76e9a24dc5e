// Packed VM kernel (tsb_ew_packed.cuh) for bodies with general accesses (probes, wrap terms, strided
// or unaligned inner dims) and with data-dependent accesses.
#include "tsb_ew_packed.cuh"

namespace tsb {

int launch_packed_general(const EwParams &P, bool indirect, dim3 grid, size_t smem, cudaStream_t s, int lg_g,
                          int per_pass, int rounds) {
  if (P.n_loops) {
    if (indirect) return launch_packed_instance<true, PACKED_INDIRECT, 4>(P, grid, smem, s, lg_g, per_pass, rounds);
    return launch_packed_instance<true, PACKED_GENERAL, 4>(P, grid, smem, s, lg_g, per_pass, rounds);
  }
  if (indirect) return launch_packed_instance<false, PACKED_INDIRECT, 4>(P, grid, smem, s, lg_g, per_pass, rounds);
  return launch_packed_instance<false, PACKED_GENERAL, 4>(P, grid, smem, s, lg_g, per_pass, rounds);
}

}  // namespace tsb
