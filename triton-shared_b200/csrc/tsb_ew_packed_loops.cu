// Packed VM kernel (tsb_ew_packed.cuh) for bodies inside a device-side loop nest, lean accesses.
#include "tsb_ew_packed.cuh"

namespace tsb {

int launch_packed_lean_loops(const EwParams &P, dim3 grid, size_t smem, cudaStream_t s, int lg_g, int per_pass,
                             int rounds) {
  return launch_packed_instance<true, PACKED_LEAN, PACKED_LEAN_U>(P, grid, smem, s, lg_g, per_pass, rounds);
}

}  // namespace tsb
