// Parameter blocks and addressing helpers of the structured-access engine (tsb_elementwise.cu).
#pragma once
#include "tsb_vm.cuh"

namespace tsb {

struct EwParams {
  DAcc acc[TSB_MAX_ACCESSES];
  tsb_op ops[TSB_MAX_OPS];
  int n_acc, n_ops;
  int size[3];
  int lg[3];      // log2 of sizes (Triton block shapes are powers of two)
  int lanes;      // size[0]*size[1]*size[2]
  int grid[3];
  int order[3];   // grid axes from fastest to slowest in the order programs are walked
  long long pid_lo, pid_hi;
  int n_loops;               // perfect loop nest around the whole body (outermost first)
  int trip[TSB_MAX_LOOPS];
  long long total_trips;     // product of the trip counts
  int indirect;              // some load/store takes a per-lane index or mask operand
  int has_reduce;            // some op folds a value over all lanes of its program (TSB_OP_REDUCE)
};

// flags in the imm field of TSB_OP_LOAD / TSB_OP_STORE
constexpr unsigned MEM_INDEX = 1u, MEM_MASK = 2u;

// Decode the flat iteration number q of a perfect loop nest into per-level counters.
__device__ __forceinline__ void loop_counters(const EwParams &P, long long q, int it[TSB_MAX_LOOPS]) {
#pragma unroll
  for (int l = TSB_MAX_LOOPS - 1; l >= 0; --l) {
    if (l < P.n_loops) {
      it[l] = (int)(q % P.trip[l]);
      q /= P.trip[l];
    } else {
      it[l] = 0;
    }
  }
}

// ---- flat addressing ------------------------------------------------------------
// When every access is a unit-stride 1-D block whose offset and mask start advance
// by exactly the block size per program (the "pid * BLOCK + arange(BLOCK)" idiom on a
// 1-D grid), lane l of program p is element g = p*BLOCK + l of one flat range: it
// lives at base + shift + g and is accessible iff g < limit.  The kernels below walk
// that range with no per-program bookkeeping; results are identical to the blocked
// kernels.
struct FlatAcc {  // 40 bytes: the whole parameter block stays below 4 KB (see the static_assert)
  char *base;
  long long shift;
  long long limit;
  unsigned other;
  unsigned char dtype, esize, vec_ok, has_other;
  unsigned char kind, pad_[7];
};
struct FlatParams {
  FlatAcc acc[TSB_MAX_ACCESSES];
  tsb_op ops[TSB_MAX_OPS];
  int n_acc, n_ops;
  long long g_lo, g_hi;
};
// kernel parameters beyond 4 KB are passed another way; the flat VM kernel measured 20 % slower
// when this block grew past that size
static_assert(sizeof(FlatParams) <= 4096, "FlatParams must fit the classic 4 KB kernel-parameter space");

__device__ __forceinline__ void flat_load(const FlatAcc &A, long long g, unsigned (&out)[4]) {
  const long long e = A.shift + g;
  if (A.kind >= 2) {
#pragma unroll
    for (int k = 0; k < 4; ++k) out[k] = A.kind == 2 ? ((g + k) < A.limit ? 1u : 0u) : (unsigned)(e + k);
    return;
  }
  const char *p = A.base + e * A.esize;
  if (A.vec_ok && g + 4 <= A.limit) {
    if (A.esize == 4) {
      const uint4 v = __ldcs(reinterpret_cast<const uint4 *>(p));
      out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    } else if (A.esize == 2) {
      const uint2 v = __ldcs(reinterpret_cast<const uint2 *>(p));
      out[0] = v.x & 0xffffu; out[1] = v.x >> 16; out[2] = v.y & 0xffffu; out[3] = v.y >> 16;
      raw_to_reg<4>(A.dtype, out);
    } else {
      const unsigned v = __ldcs(reinterpret_cast<const unsigned *>(p));
#pragma unroll
      for (int k = 0; k < 4; ++k) out[k] = (v >> (8 * k)) & 0xffu;
      raw_to_reg<4>(A.dtype, out);
    }
    return;
  }
  const unsigned fill = A.has_other ? A.other : 0u;
#pragma unroll
  for (int k = 0; k < 4; ++k) out[k] = (g + k) < A.limit ? ld_elem(p + k * A.esize, A.dtype) : fill;
}

__device__ __forceinline__ void flat_store(const FlatAcc &A, long long g, const unsigned (&in)[4]) {
  char *p = A.base + (A.shift + g) * A.esize;
  if (A.vec_ok && g + 4 <= A.limit) {
    if (A.esize == 4) {
      __stcs(reinterpret_cast<uint4 *>(p), make_uint4(in[0], in[1], in[2], in[3]));
    } else if (A.esize == 2) {
      unsigned h[4] = {in[0], in[1], in[2], in[3]};
      reg_to_raw<4>(A.dtype, h);
      __stcs(reinterpret_cast<uint2 *>(p), make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16)));
    } else {
      unsigned h[4] = {in[0], in[1], in[2], in[3]};
      reg_to_raw<4>(A.dtype, h);
      __stcs(reinterpret_cast<unsigned *>(p), h[0] | (h[1] << 8) | (h[2] << 16) | (h[3] << 24));
    }
    return;
  }
#pragma unroll
  for (int k = 0; k < 4; ++k)
    if (g + k < A.limit) st_elem(p + k * A.esize, A.dtype, in[k]);
}

// tsb_ew_packed.cu
int launch_ew_packed(const EwParams &P, int items, int regs_used, cudaStream_t s);

constexpr int FLAT_VM_U = 4;  // lane-vectors per thread of the flat VM kernel

// tsb_ew_flat.cu
int launch_flat_vm(const FlatParams &F, unsigned ctas, int threads, size_t smem, cudaStream_t s);

}  // namespace tsb
