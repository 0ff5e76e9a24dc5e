// Block programs: bodies that mix structured loads/stores, elementwise ops and reductions
// over whole blocks (tt.reduce along an axis), one Triton program per CTA.
//
// Reference semantics (paths inside microsoft/triton-shared): tt.reduce becomes a transpose
// plus linalg.reduce with a single-op combiner folded from the combiner's identity
// (ReduceConverter, ConversionPatterns.hpp:1203-1440); the surrounding ops are the same
// linalg.generic / memref.copy forms as in tsb_elementwise.cu.  The CPU backend keeps every
// intermediate block in a malloc'ed buffer; here every intermediate lives in shared memory
// for the lifetime of the program and never touches HBM.
//
// Values ("registers") are indexed by the coordinates of one iteration space of rank <= 3; a
// register extends along a subset of the dims (its mask) and is broadcast along the others,
// which is how splat / expand_dims / broadcast and keep-dim reduction results are expressed.
// Ops run one after another over the whole block with a barrier between them.  This is the
// general path: the dedicated softmax / LayerNorm / reduction kernels are faster where they apply.
#include "tsb_vm.cuh"

namespace tsb {

constexpr int BP_MAX_REGS = 24;
constexpr int BP_THREADS = 256;

struct BpParams {
  DAcc acc[TSB_MAX_ACCESSES];
  tsb_op ops[TSB_MAX_OPS];
  int n_acc, n_ops, n_regs;
  int size[3];
  int lg[3];  // log2 of size
  int grid[3];
  int order[3];   // grid axes from fastest to slowest in the order programs are walked
  long long pid_lo, pid_hi;
  int reg_mask[BP_MAX_REGS];  // bit d set: the register extends along dim d
  int reg_off[BP_MAX_REGS];   // offset (32-bit words) in dynamic shared memory
  int reg_n[BP_MAX_REGS];     // number of elements
};

// Block sizes are powers of two, so coordinates come from shifts and masks.
// coordinates of element e of a register with mask m (row-major over its present dims)
__device__ __forceinline__ void reg_coords(const int lg[3], int m, int e, int &i0, int &i1, int &i2) {
  const int l2 = (m & 4) ? lg[2] : 0, l1 = (m & 2) ? lg[1] : 0;
  i2 = e & ((1 << l2) - 1);
  e >>= l2;
  i1 = e & ((1 << l1) - 1);
  i0 = e >> l1;
}
// element index of coordinates (i0,i1,i2) in a register with mask m (absent dims are broadcast)
__device__ __forceinline__ int reg_index(const int lg[3], int m, int i0, int i1, int i2) {
  const int l2 = (m & 4) ? lg[2] : 0, l1 = (m & 2) ? lg[1] : 0;
  return (((((m & 1) ? i0 : 0) << l1) + ((m & 2) ? i1 : 0)) << l2) + ((m & 4) ? i2 : 0);
}

// dst[e] = OPC(a, b, c) for this thread's elements; operands with the destination's mask are read
// at the same index, scalars at 0, anything else through its coordinates
template <int OPC>
__device__ __forceinline__ void ew_loop(const tsb_op &op, const int lg[3], unsigned *dst, int n, int md,
                                        const unsigned *ra, int ma, const unsigned *rb, int mb,
                                        const unsigned *rc, int mc) {
  constexpr int AR = alu_arity<OPC>();
  const bool sa = ma == md || ma == 0, sb = AR < 2 || mb == md || mb == 0, sc = AR < 3 || mc == md || mc == 0;
  if (sa && sb && sc && (n & 3) == 0) {
    // four consecutive elements per thread and step: one 16-byte access per full-size operand,
    // scalars (mask 0) read once
    const uint4 *pa = reinterpret_cast<const uint4 *>(ra), *pb = reinterpret_cast<const uint4 *>(rb),
                *pc = reinterpret_cast<const uint4 *>(rc);
    const unsigned a0 = ra[0], b0 = AR >= 2 ? rb[0] : 0u, c0 = AR >= 3 ? rc[0] : 0u;
    for (int e = threadIdx.x; e < (n >> 2); e += blockDim.x) {
      const uint4 A = ma == md ? pa[e] : make_uint4(a0, a0, a0, a0);
      const uint4 B = (AR >= 2 && mb == md) ? pb[e] : make_uint4(b0, b0, b0, b0);
      const uint4 C = (AR >= 3 && mc == md) ? pc[e] : make_uint4(c0, c0, c0, c0);
      uint4 r;
      r.x = alu_op<OPC, false>(op, A.x, B.x, C.x);
      r.y = alu_op<OPC, false>(op, A.y, B.y, C.y);
      r.z = alu_op<OPC, false>(op, A.z, B.z, C.z);
      r.w = alu_op<OPC, false>(op, A.w, B.w, C.w);
      if (alu_rounds<OPC>() && op.type != TSB_F32) {  // 16-bit float op: re-round, decided once per vector
        r.x = __float_as_uint(round_to(__uint_as_float(r.x), op.type));
        r.y = __float_as_uint(round_to(__uint_as_float(r.y), op.type));
        r.z = __float_as_uint(round_to(__uint_as_float(r.z), op.type));
        r.w = __float_as_uint(round_to(__uint_as_float(r.w), op.type));
      }
      reinterpret_cast<uint4 *>(dst)[e] = r;
    }
  } else if (sa && sb && sc) {
    const int ka = ma == md ? 1 : 0, kb = (AR >= 2 && mb == md) ? 1 : 0, kc = (AR >= 3 && mc == md) ? 1 : 0;
    for (int e = threadIdx.x; e < n; e += blockDim.x) dst[e] = alu_op<OPC>(op, ra[e * ka], rb[e * kb], rc[e * kc]);
  } else {
    for (int e = threadIdx.x; e < n; e += blockDim.x) {
      int i0, i1, i2;
      reg_coords(lg, md, e, i0, i1, i2);
      dst[e] = alu_op<OPC>(op, ra[reg_index(lg, ma, i0, i1, i2)], rb[reg_index(lg, mb, i0, i1, i2)],
                           rc[reg_index(lg, mc, i0, i1, i2)]);
    }
  }
}

__global__ void __launch_bounds__(BP_THREADS) block_program_kernel(const __grid_constant__ BpParams P) {
  extern __shared__ __align__(16) unsigned bp_smem[];
  __shared__ unsigned red[BP_THREADS / 32];
  // The op list and the register tables are read once per op by every thread: from shared memory
  // (indexed reads of kernel parameters were the busiest pipe of this kernel).
  __shared__ __align__(16) tsb_op s_ops[TSB_MAX_OPS];
  __shared__ int s_mask[BP_MAX_REGS], s_off[BP_MAX_REGS], s_n[BP_MAX_REGS];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int k = tid; k < P.n_ops; k += BP_THREADS) s_ops[k] = P.ops[k];
  if (tid < BP_MAX_REGS) {
    s_mask[tid] = P.reg_mask[tid];
    s_off[tid] = P.reg_off[tid];
    s_n[tid] = P.reg_n[tid];
  }
  __syncthreads();
  for (long long prog = P.pid_lo + blockIdx.x; prog < P.pid_hi; prog += gridDim.x) {
    long long px, py, pz;
    split_pid(P.grid, P.order, prog, px, py, pz);
    // loop state in registers: the slot is selected by comparison, never by indexing
    int it[TSB_MAX_LOOPS] = {0, 0, 0, 0}, trip[TSB_MAX_LOOPS] = {0, 0, 0, 0}, begin[TSB_MAX_LOOPS] = {0, 0, 0, 0};
    for (int k = 0; k < P.n_ops;) {
      const tsb_op op = s_ops[k];
      // loops: uniform control flow, the same for every thread of the CTA
      if (op.opcode == TSB_OP_LOOP_BEGIN) {
        int next = k + 1;
#pragma unroll
        for (int l = 0; l < TSB_MAX_LOOPS; ++l)
          if (l == op.a) {
            it[l] = 0;
            trip[l] = (int)op.imm;
            begin[l] = k + 1;
            if (trip[l] <= 0) next = op.b;
          }
        k = next;
        continue;
      }
      if (op.opcode == TSB_OP_LOOP_END) {
        int next = k + 1;
#pragma unroll
        for (int l = 0; l < TSB_MAX_LOOPS; ++l)
          if (l == op.a && ++it[l] < trip[l]) next = begin[l];
        k = next;
        continue;
      }
      ++k;
      __syncthreads();  // every op may read what other threads wrote in the previous one
      if (op.opcode == TSB_OP_LOAD) {
        const DAcc &A = P.acc[op.a];
        ProgState st;
        program_state_loops(A, P.size, px, py, pz, it, st);
        const int m = s_mask[op.dst];
        unsigned *dst = bp_smem + s_off[op.dst];
        if (op.imm2 & 3u) {
          // data-dependent access (flags in imm2: 1 = per-lane index in register b, 2 = per-lane mask
          // in register c): one element per thread and step
          const bool hi = op.imm2 & 1u, hm = op.imm2 & 2u;
          const unsigned *ri = bp_smem + s_off[hi ? op.b : 0], *rm = bp_smem + s_off[hm ? op.c : 0];
          const int mi = s_mask[hi ? op.b : 0], mm = s_mask[hm ? op.c : 0];
          for (int e = tid; e < s_n[op.dst]; e += BP_THREADS) {
            int i0, i1, i2;
            reg_coords(P.lg, m, e, i0, i1, i2);
            const unsigned ix[1] = {hi ? ri[reg_index(P.lg, mi, i0, i1, i2)] : 0u};
            const unsigned mk[1] = {hm ? rm[reg_index(P.lg, mm, i0, i1, i2)] : 1u};
            unsigned v[1];
            load_vec_indirect<1>(A, st, i0, i1, i2, hi, hm, ix, mk, v);
            dst[e] = v[0];
          }
        } else if ((m & 4) && (P.size[2] & 3) == 0) {
          // 4-lane vectors along the innermost dim, four independent loads in flight per thread
          const int n4 = s_n[op.dst] >> 2;
          for (int e0 = tid; e0 < n4; e0 += BP_THREADS * 4) {
            unsigned v[4][4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int e4 = e0 + u * BP_THREADS;
              if (e4 < n4) {
                int i0, i1, i2;
                reg_coords(P.lg, m, e4 * 4, i0, i1, i2);
                load_vec<4>(A, st, i0, i1, i2, v[u]);
              }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int e4 = e0 + u * BP_THREADS;
              if (e4 < n4) reinterpret_cast<uint4 *>(dst)[e4] = make_uint4(v[u][0], v[u][1], v[u][2], v[u][3]);
            }
          }
        } else {
          for (int e = tid; e < s_n[op.dst]; e += BP_THREADS) {
            int i0, i1, i2;
            reg_coords(P.lg, m, e, i0, i1, i2);
            unsigned v[1];
            load_vec<1>(A, st, i0, i1, i2, v);
            dst[e] = v[0];
          }
        }
      } else if (op.opcode == TSB_OP_STORE) {
        const DAcc &A = P.acc[op.a];
        ProgState st;
        program_state_loops(A, P.size, px, py, pz, it, st);
        const int m = (int)op.imm;  // dims the store extends along
        const int ms = s_mask[op.b];
        const unsigned *src = bp_smem + s_off[op.b];
        const int n = ((m & 1) ? P.size[0] : 1) * ((m & 2) ? P.size[1] : 1) * ((m & 4) ? P.size[2] : 1);
        if (op.imm2 & 3u) {
          // data-dependent store: per-lane index in register c, per-lane mask in register dst
          const bool hi = op.imm2 & 1u, hm = op.imm2 & 2u;
          const unsigned *ri = bp_smem + s_off[hi ? op.c : 0], *rm = bp_smem + s_off[hm ? op.dst : 0];
          const int mi = s_mask[hi ? op.c : 0], mm = s_mask[hm ? op.dst : 0];
          for (int e = tid; e < n; e += BP_THREADS) {
            int i0, i1, i2;
            reg_coords(P.lg, m, e, i0, i1, i2);
            const unsigned ix[1] = {hi ? ri[reg_index(P.lg, mi, i0, i1, i2)] : 0u};
            const unsigned mk[1] = {hm ? rm[reg_index(P.lg, mm, i0, i1, i2)] : 1u};
            const unsigned v[1] = {src[reg_index(P.lg, ms, i0, i1, i2)]};
            store_vec_indirect<1>(A, st, i0, i1, i2, hi, hm, ix, mk, v);
          }
        } else if ((m & 4) && ms == m && (P.size[2] & 3) == 0) {
          for (int e4 = tid; e4 < (n >> 2); e4 += BP_THREADS) {
            int i0, i1, i2;
            reg_coords(P.lg, m, e4 * 4, i0, i1, i2);
            const uint4 q = reinterpret_cast<const uint4 *>(src)[e4];
            const unsigned v[4] = {q.x, q.y, q.z, q.w};
            store_vec<4>(A, st, i0, i1, i2, v);
          }
        } else {
          for (int e = tid; e < n; e += BP_THREADS) {
            int i0, i1, i2;
            reg_coords(P.lg, m, e, i0, i1, i2);
            unsigned v[1] = {src[reg_index(P.lg, ms, i0, i1, i2)]};
            store_vec<1>(A, st, i0, i1, i2, v);
          }
        }
      } else if (op.opcode == TSB_OP_ARGREDUCE) {
        // (dst, c) = (value, index) of the extreme element along dim imm2; one warp per output
        const int d = (int)op.imm2;
        const bool want_max = op.imm != 0;
        const int mv = s_mask[op.a], mi = s_mask[op.b], md = s_mask[op.dst];
        const unsigned *vsrc = bp_smem + s_off[op.a], *isrc = bp_smem + s_off[op.b];
        unsigned *vdst = bp_smem + s_off[op.dst], *idst = bp_smem + s_off[op.c];
        const int len = P.size[d];
        // a over b iff a is strictly better, or equal with the smaller index (the region of tl.argmax / tl.argmin)
        auto better = [&](float va, int ia, float vb, int ib) {
          return (want_max ? va > vb : va < vb) || (va == vb && ia < ib);
        };
        for (int o = warp; o < s_n[op.dst]; o += BP_THREADS / 32) {
          int c[3];
          reg_coords(P.lg, md, o, c[0], c[1], c[2]);
          // the reference folds from (-inf | +inf, -1): an element replaces the running pair only if it is
          // strictly better or ties with a smaller index, so NaNs never win and a line without any
          // winner keeps index -1 (ConversionPatterns.hpp:1569-1672, 1734, 1765)
          float bv = __uint_as_float(want_max ? 0xff800000u : 0x7f800000u);
          int bi = -1;
          for (int j = lane; j < len; j += 32) {
            c[d] = j;
            const float v = __uint_as_float(vsrc[reg_index(P.lg, mv, c[0], c[1], c[2])]);
            const int ix = (int)isrc[reg_index(P.lg, mi, c[0], c[1], c[2])];
            if (better(v, ix, bv, bi)) { bv = v; bi = ix; }
          }
#pragma unroll
          for (int s = 16; s > 0; s >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, s);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, s);
            if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
          }
          if (lane == 0) {
            vdst[o] = __float_as_uint(bv);
            idst[o] = (unsigned)bi;
          }
        }
      } else if (op.opcode == TSB_OP_SCAN) {
        // dst = inclusive running combination of src along dim imm2 (cumulative sum): one warp per
        // line, 32 elements per step with a shuffle scan, the running total carried between steps
        const int d = (int)op.imm2, comb = (int)op.imm;
        const int m = s_mask[op.a];
        const unsigned *src = bp_smem + s_off[op.a];
        unsigned *dst = bp_smem + s_off[op.dst];
        const int len = (m & (1 << d)) ? P.size[d] : 1;
        const int lines = s_n[op.a] / len;
        const int md = m & ~(1 << d);  // coordinates of a line: the register's dims without the scanned one
        for (int o = warp; o < lines; o += BP_THREADS / 32) {
          int c[3];
          reg_coords(P.lg, md, o, c[0], c[1], c[2]);
          unsigned carry = combine_identity(comb);
          for (int j0 = 0; j0 < len; j0 += 32) {
            const int j = j0 + lane;
            c[d] = j < len ? j : 0;
            const int at = reg_index(P.lg, m, c[0], c[1], c[2]);
            unsigned v = j < len ? src[at] : combine_identity(comb);
#pragma unroll
            for (int s = 1; s < 32; s <<= 1) {
              const unsigned up = __shfl_up_sync(0xffffffffu, v, s);
              if (lane >= s) v = combine(comb, op.type, up, v);
            }
            v = combine(comb, op.type, carry, v);
            if (j < len) dst[at] = v;
            carry = __shfl_sync(0xffffffffu, v, 31);
          }
        }
      } else if (op.opcode == TSB_OP_REDUCE) {
        // dst = fold of src along dim imm2 with combiner imm; one warp per output element
        const int d = (int)op.imm2, comb = (int)op.imm;
        const int ms = s_mask[op.a], md = s_mask[op.dst];
        const unsigned *src = bp_smem + s_off[op.a];
        unsigned *dst = bp_smem + s_off[op.dst];
        const int len = P.size[d];
        const int n_out = s_n[op.dst];
        if (n_out < BP_THREADS / 32) {
          // few outputs (a 1-D block folded to a scalar): the whole CTA works on each of them
          for (int o = 0; o < n_out; ++o) {
            int c[3];
            reg_coords(P.lg, md, o, c[0], c[1], c[2]);
            unsigned acc = combine_identity(comb);
            for (int j = tid; j < len; j += BP_THREADS) {
              c[d] = j;
              acc = combine(comb, op.type, src[reg_index(P.lg, ms, c[0], c[1], c[2])], acc);
            }
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) acc = combine(comb, op.type, __shfl_xor_sync(0xffffffffu, acc, s), acc);
            if (lane == 0) red[warp] = acc;
            __syncthreads();
            if (tid == 0) {
              unsigned r = red[0];
              for (int w = 1; w < BP_THREADS / 32; ++w) r = combine(comb, op.type, red[w], r);
              dst[o] = r;
            }
            __syncthreads();
          }
        } else {
          for (int o = warp; o < n_out; o += BP_THREADS / 32) {
            int c[3];
            reg_coords(P.lg, md, o, c[0], c[1], c[2]);
            unsigned acc = combine_identity(comb);
            for (int j = lane; j < len; j += 32) {
              c[d] = j;
              acc = combine(comb, op.type, src[reg_index(P.lg, ms, c[0], c[1], c[2])], acc);
            }
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) acc = combine(comb, op.type, __shfl_xor_sync(0xffffffffu, acc, s), acc);
            if (lane == 0) dst[o] = acc;
          }
        }
      } else {
        const int md = s_mask[op.dst];
        unsigned *dst = bp_smem + s_off[op.dst];
        // operand fields an op does not use may hold anything: keep the table reads in range
        const int qa = (unsigned)op.a < BP_MAX_REGS ? op.a : 0, qb = (unsigned)op.b < BP_MAX_REGS ? op.b : 0,
                  qc = (unsigned)op.c < BP_MAX_REGS ? op.c : 0;
        const int ma = s_mask[qa], mb = s_mask[qb], mc = s_mask[qc];
        const unsigned *ra = bp_smem + s_off[qa], *rb = bp_smem + s_off[qb], *rc = bp_smem + s_off[qc];
        const int n = s_n[op.dst];
        if (op.opcode == TSB_OP_CONST) {
          for (int e = tid; e < n; e += BP_THREADS) dst[e] = op.imm;
        } else {
          switch (op.opcode) {
#define TSB_BP_CASE(O) \
  case O: ew_loop<O>(op, P.lg, dst, n, md, ra, ma, rb, mb, rc, mc); break;
            TSB_ALU_OPCODES(TSB_BP_CASE)
#undef TSB_BP_CASE
            default: break;
          }
        }
      }
    }
    __syncthreads();  // the next program reuses the registers
  }
}

}  // namespace tsb

using namespace tsb;

extern "C" int tsb_block_program(const tsb_access *acc, int n_acc, const tsb_op *ops, int n_ops,
                                 const int32_t *reg_masks, int n_regs, const int32_t grid[3],
                                 int64_t pid_lo, int64_t pid_hi, void *stream) {
  if (!acc || !ops || !reg_masks || !grid) return fail(TSB_ERR_INVALID, "tsb_block_program: null argument");
  if (n_acc < 1 || n_acc > TSB_MAX_ACCESSES || n_ops < 1 || n_ops > TSB_MAX_OPS || n_regs < 1 || n_regs > BP_MAX_REGS)
    return fail(TSB_ERR_UNSUPPORTED, "tsb_block_program: %d accesses / %d ops / %d registers (max %d / %d / %d)", n_acc,
                n_ops, n_regs, TSB_MAX_ACCESSES, TSB_MAX_OPS, BP_MAX_REGS);
  const long long total = (long long)grid[0] * grid[1] * grid[2];
  if (pid_lo < 0 || pid_hi > total || pid_lo > pid_hi)
    return fail(TSB_ERR_INVALID, "tsb_block_program: program range [%lld,%lld) outside grid of %lld",
                (long long)pid_lo, (long long)pid_hi, total);
  static thread_local BpParams P;
  memset(&P, 0, sizeof(P));
  const int rank = acc[0].rank;
  if (rank < 1 || rank > TSB_MAX_RANK) return fail(TSB_ERR_UNSUPPORTED, "tsb_block_program: rank %d", rank);
  P.size[0] = P.size[1] = P.size[2] = 1;
  for (int d = 0; d < rank; ++d) {
    if (acc[0].sizes[d] < 1 || acc[0].sizes[d] > (1 << 20)) return fail(TSB_ERR_INVALID, "tsb_block_program: bad block size");
    P.size[3 - rank + d] = (int)acc[0].sizes[d];
  }
  for (int d = 0; d < 3; ++d) {
    P.lg[d] = ilog2_exact(P.size[d]);
    if (P.lg[d] < 0) return fail(TSB_ERR_INVALID, "tsb_block_program: block size %d is not a power of two", P.size[d]);
  }
  for (int a = 0; a < n_acc; ++a) {
    int rc = convert_access(acc, a, rank, P.size, grid, (P.size[2] % 4 == 0) ? 4 : 1, P.acc[a]);
    if (rc != TSB_OK) return rc;
  }
  long long words = 0;
  for (int r = 0; r < n_regs; ++r) {
    const int m = reg_masks[r];
    if (m < 0 || m > 7) return fail(TSB_ERR_INVALID, "tsb_block_program: register %d has mask %d", r, m);
    // masks are given over the access rank; shift to the padded rank-3 space
    const int pm = m << (3 - rank);
    long long n = 1;
    for (int d = 0; d < 3; ++d)
      if (pm & (1 << d)) n *= P.size[d];
    P.reg_mask[r] = pm;
    P.reg_off[r] = (int)words;
    P.reg_n[r] = (int)n;
    words += (n + 3) & ~3ll;  // 16-byte aligned registers
  }
  const long long smem = words * 4;
  if (smem > 200 * 1024)
    return fail(TSB_ERR_UNSUPPORTED, "tsb_block_program: %lld bytes of block values exceed the 200 KB on-chip budget", smem);
  for (int k = 0; k < n_ops; ++k) {
    tsb_op o = ops[k];
    const bool mem = o.opcode == TSB_OP_LOAD || o.opcode == TSB_OP_STORE;
    if (mem && (o.a < 0 || o.a >= n_acc)) return fail(TSB_ERR_INVALID, "tsb_block_program: op %d names access %d", k, o.a);
    if (o.opcode == TSB_OP_LOAD && acc[o.a].is_store == 1) return fail(TSB_ERR_INVALID, "tsb_block_program: op %d loads from a store access", k);
    if (o.opcode == TSB_OP_STORE && acc[o.a].is_store != 1) return fail(TSB_ERR_INVALID, "tsb_block_program: op %d stores to a load access", k);
    if (o.opcode == TSB_OP_STORE) o.imm = o.imm << (3 - rank);
    if (o.opcode == TSB_OP_SCAN && o.imm != TSB_OP_ADDF && o.imm != TSB_OP_ADDI)
      return fail(TSB_ERR_UNSUPPORTED, "tsb_block_program: op %d scans with combiner %u (only sums)", k, o.imm);
    if (o.opcode == TSB_OP_REDUCE || o.opcode == TSB_OP_ARGREDUCE || o.opcode == TSB_OP_SCAN) {
      if (o.imm2 >= (unsigned)rank) return fail(TSB_ERR_INVALID, "tsb_block_program: op %d reduces dim %u of rank %d", k, o.imm2, rank);
      o.imm2 += 3 - rank;
    }
    if (o.opcode == TSB_OP_LOOP_BEGIN || o.opcode == TSB_OP_LOOP_END) {
      if (o.a < 0 || o.a >= TSB_MAX_LOOPS) return fail(TSB_ERR_INVALID, "tsb_block_program: op %d uses loop slot %d", k, o.a);
      if (o.opcode == TSB_OP_LOOP_BEGIN && (o.b <= k || o.b > n_ops || ops[o.b - 1].opcode != TSB_OP_LOOP_END || ops[o.b - 1].a != o.a))
        return fail(TSB_ERR_INVALID, "tsb_block_program: op %d does not name its matching loop end", k);
      P.ops[k] = o;
      continue;
    }
    if (mem && (o.imm2 & ~3u)) return fail(TSB_ERR_INVALID, "tsb_block_program: op %d has memory flags %u", k, o.imm2);
    // operands of a load: index in b, mask in c; of a store: value in b, index in c, mask in dst (each only when flagged)
    const bool ld = o.opcode == TSB_OP_LOAD, stn = o.opcode == TSB_OP_STORE;
    const int regs[4] = {stn ? ((o.imm2 & 2u) ? o.dst : 0) : o.dst, mem || o.opcode == TSB_OP_CONST ? 0 : o.a,
                         (ld ? ((o.imm2 & 1u) ? o.b : 0) : (o.opcode == TSB_OP_CONST ? 0 : o.b)),
                         mem ? (((ld ? o.imm2 & 2u : o.imm2 & 1u)) ? o.c : 0) : o.c};
    for (int r = 0; r < 4; ++r)
      if (regs[r] < 0 || regs[r] >= n_regs) return fail(TSB_ERR_INVALID, "tsb_block_program: op %d register %d out of range", k, regs[r]);
    P.ops[k] = o;
  }
  P.n_acc = n_acc; P.n_ops = n_ops; P.n_regs = n_regs;
  for (int k = 0; k < 3; ++k) P.grid[k] = grid[k] > 0 ? grid[k] : 1;
  P.pid_lo = pid_lo; P.pid_hi = pid_hi;
  choose_program_order(P.acc, n_acc, P.grid, pid_lo, pid_hi, P.order);
  if (pid_hi == pid_lo) return TSB_OK;
  static SmemLimit smem_limit;
  if (smem > 48 * 1024) TSB_CUDA_OK(allow_dynamic_smem(block_program_kernel, 200 * 1024, smem_limit));
  long long per_sm = smem > 0 ? (220 * 1024) / (smem + 1024) : 8;
  if (per_sm > 8) per_sm = 8;
  if (per_sm < 1) per_sm = 1;
  long long ctas = (long long)sm_count() * per_sm;
  if (ctas > pid_hi - pid_lo) ctas = pid_hi - pid_lo;
  block_program_kernel<<<(unsigned)ctas, BP_THREADS, (size_t)smem, (cudaStream_t)stream>>>(P);
  TSB_LAUNCH_OK("block_program_kernel");
  return TSB_OK;
}
