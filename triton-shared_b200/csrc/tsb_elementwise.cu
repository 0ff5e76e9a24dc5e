// Structured-access engine: masked strided block loads/stores around an
// elementwise body, one Triton program per CTA iteration.
//
// Reference semantics implemented here (paths inside microsoft/triton-shared):
//   block view      lib/Conversion/StructuredToMemref/StructuredToMemref.cpp:528-551
//   masked load     same file :794-853 (+ fillWithValue :192-224)
//   masked store    same file :1163-1196
//   mask dims       lib/Analysis/MaskAnalysis.cpp:583-585
//   element copy    backend/include/ExecutionEngine/CRunnerUtils.cpp:58-113
//   elementwise op  lib/Conversion/TritonArithToLinalg/TritonArithToLinalg.cpp:104
// The CPU backend materialises every block in a malloc'ed buffer and runs one
// scalar loop per op; here a lane's values stay in registers from load to store.
#include "tsb_vm_exec.cuh"
#include <stdlib.h>

namespace tsb {

template <int VEC, int U>
__global__ void __launch_bounds__(256) ew_vm_kernel(const __grid_constant__ EwParams P) {
  extern __shared__ __align__(16) unsigned vm_smem[];
  __shared__ ProgState st[TSB_MAX_ACCESSES];
  const VmRegs<VEC, U> R{vm_smem, (int)blockDim.x, (int)threadIdx.x};
  const int items = P.lanes / VEC;
  const int sh1 = P.lg[2], sh0 = P.lg[2] + P.lg[1];
  grid_dependency_wait();
  grid_launch_dependents();
  for (long long prog = P.pid_lo + blockIdx.x; prog < P.pid_hi; prog += gridDim.x) {
    long long px, py, pz;
    split_pid(P.grid, P.order, prog, px, py, pz);
    // a loop nest around the body runs here, in order, one iteration after the other: a later
    // iteration sees what an earlier one of the same program stored
    for (long long q = 0; q < P.total_trips; ++q) {
      int it[TSB_MAX_LOOPS];
      loop_counters(P, q, it);
      __threadfence_block();
      __syncthreads();  // the previous program's (iteration's) state is no longer read
      if (threadIdx.x < P.n_acc) program_state_loops(P.acc[threadIdx.x], P.size, px, py, pz, it, st[threadIdx.x]);
      __syncthreads();
      for (int it0 = threadIdx.x; it0 < items; it0 += blockDim.x * U) {
        auto coords = [&](int u, int &i0, int &i1, int &i2) {
          const int itm = it0 + u * (int)blockDim.x;
          const int l = itm * VEC;
          i2 = l & (P.size[2] - 1);
          i1 = (l >> sh1) & (P.size[1] - 1);
          i0 = l >> sh0;
          return itm < items;
        };
        vm_exec<VEC, U, true, false>(
            P.ops, P.n_ops, R,
            [&](int a, unsigned(&r)[U][VEC]) {
#pragma unroll
              for (int u = 0; u < U; ++u) {
                int i0, i1, i2;
                if (coords(u, i0, i1, i2)) {
                  load_vec<VEC>(P.acc[a], st[a], i0, i1, i2, r[u]);
                } else {
#pragma unroll
                  for (int v = 0; v < VEC; ++v) r[u][v] = 0u;
                }
              }
            },
            [&](int a, const unsigned(&r)[U][VEC]) {
#pragma unroll
              for (int u = 0; u < U; ++u) {
                int i0, i1, i2;
                if (coords(u, i0, i1, i2)) store_vec<VEC>(P.acc[a], st[a], i0, i1, i2, r[u]);
              }
            },
            [&](int a, int u, unsigned flags, const unsigned(&ix)[VEC], const unsigned(&mk)[VEC], unsigned(&r)[VEC]) {
              int i0, i1, i2;
              if (coords(u, i0, i1, i2)) {
                load_vec_indirect<VEC>(P.acc[a], st[a], i0, i1, i2, flags & MEM_INDEX, flags & MEM_MASK, ix, mk, r);
              } else {
#pragma unroll
                for (int v = 0; v < VEC; ++v) r[v] = 0u;
              }
            },
            [&](int a, int u, unsigned flags, const unsigned(&ix)[VEC], const unsigned(&mk)[VEC],
                const unsigned(&r)[VEC]) {
              int i0, i1, i2;
              if (coords(u, i0, i1, i2))
                store_vec_indirect<VEC>(P.acc[a], st[a], i0, i1, i2, flags & MEM_INDEX, flags & MEM_MASK, ix, mk, r);
            });
      }
    }
  }
}


// ---- fast body: out = binop(load0, load1), all fp32 ---------------------------
// Two programs per CTA iteration so that each thread has four 16-byte loads in
// flight before the first use.
template <int VEC>
__global__ void __launch_bounds__(256) ew_binary_f32_kernel(const __grid_constant__ EwParams P) {
  const int items = P.lanes / VEC;
  const int sh1 = P.lg[2], sh0 = P.lg[2] + P.lg[1];
  const int opc = P.ops[2].opcode;
  const DAcc &A0 = P.acc[P.ops[0].a];
  const DAcc &A1 = P.acc[P.ops[1].a];
  const DAcc &AS = P.acc[P.ops[3].a];
  constexpr int U = 2;
  for (long long prog0 = P.pid_lo + (long long)blockIdx.x * U; prog0 < P.pid_hi;
       prog0 += (long long)gridDim.x * U) {
    ProgState s0[U], s1[U], ss[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      long long prog = prog0 + u;
      if (prog >= P.pid_hi) prog = P.pid_hi - 1;  // duplicate work is skipped below
      long long px, py, pz;
      split_pid(P.grid, P.order, prog, px, py, pz);
      program_state(A0, P.size, px, py, pz, s0[u]);
      program_state(A1, P.size, px, py, pz, s1[u]);
      program_state(AS, P.size, px, py, pz, ss[u]);
    }
    for (int it = threadIdx.x; it < items; it += blockDim.x) {
      const int l = it * VEC;
      const int i2 = l & (P.size[2] - 1);
      const int i1 = (l >> sh1) & (P.size[1] - 1);
      const int i0 = l >> sh0;
      unsigned a[U][VEC], b[U][VEC];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        load_vec<VEC>(A0, s0[u], i0, i1, i2, a[u]);
        load_vec<VEC>(A1, s1[u], i0, i1, i2, b[u]);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (prog0 + u >= P.pid_hi) break;
        unsigned r[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v)
          r[v] = __float_as_uint(binf(opc, __uint_as_float(a[u][v]), __uint_as_float(b[u][v])));
        store_vec<VEC>(AS, ss[u], i0, i1, i2, r);
      }
    }
  }
}

// ---- copy body: store(load) with one element type ------------------------------------------
// The B200 counterpart of memrefCopy (CRunnerUtils.cpp:58-113) for masked strided blocks of any
// rank <= 3: 16-byte (or 8 / 4-byte for narrow types) accesses along the unit-stride dim, four
// independent vectors in flight per thread, no VM.
template <int VEC>
__global__ void __launch_bounds__(256) ew_copy_kernel(const __grid_constant__ EwParams P) {
  const int items = P.lanes / VEC;
  const int sh1 = P.lg[2], sh0 = P.lg[2] + P.lg[1];
  const DAcc &AL = P.acc[P.ops[0].a];
  const DAcc &AS = P.acc[P.ops[1].a];
  constexpr int U = 4;
  for (long long prog = P.pid_lo + blockIdx.x; prog < P.pid_hi; prog += gridDim.x) {
    long long px, py, pz;
    split_pid(P.grid, P.order, prog, px, py, pz);
    ProgState sl, ss;
    program_state(AL, P.size, px, py, pz, sl);
    program_state(AS, P.size, px, py, pz, ss);
    for (int it0 = threadIdx.x; it0 < items; it0 += blockDim.x * U) {
      unsigned v[U][VEC];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int it = it0 + u * (int)blockDim.x;
        if (it < items) {
          const int l = it * VEC;
          load_vec<VEC>(AL, sl, l >> sh0, (l >> sh1) & (P.size[1] - 1), l & (P.size[2] - 1), v[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int it = it0 + u * (int)blockDim.x;
        if (it < items) {
          const int l = it * VEC;
          store_vec<VEC>(AS, ss, l >> sh0, (l >> sh1) & (P.size[1] - 1), l & (P.size[2] - 1), v[u]);
        }
      }
    }
  }
}

// Lean form of the copy for rank <= 2 blocks whose rows are 16-byte aligned on both sides and
// whose load and store masks are the same: raw 16-byte vectors, addresses by pointer arithmetic.
__global__ void __launch_bounds__(256) ew_copy2d_kernel(const __grid_constant__ EwParams P) {
  const DAcc &AL = P.acc[P.ops[0].a];
  const DAcc &AS = P.acc[P.ops[1].a];
  const int es = AL.esize;
  const int epv_lg = es == 4 ? 2 : (es == 2 ? 3 : 4);  // elements per 16-byte vector
  const int vr_lg = P.lg[2] - epv_lg;                  // vectors per row
  const int n_vec = P.size[1] << vr_lg;
  const long long pitch_l = AL.stride[1] * es, pitch_s = AS.stride[1] * es;
  constexpr int U = 4;
  for (long long prog = P.pid_lo + blockIdx.x; prog < P.pid_hi; prog += gridDim.x) {
    long long px, py, pz;
    split_pid(P.grid, P.order, prog, px, py, pz);
    ProgState sl, ss;
    program_state(AL, P.size, px, py, pz, sl);
    program_state(AS, P.size, px, py, pz, ss);
    const char *lb = AL.base + sl.off * es;
    char *sb = AS.base + ss.off * es;
    const int rows = ss.dim[1], cols = ss.dim[2];
    for (int v0 = threadIdx.x; v0 < n_vec; v0 += blockDim.x * U) {
      uint4 q[U];
      int row[U], col[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int v = v0 + u * (int)blockDim.x;
        row[u] = v >> vr_lg;
        col[u] = (v & ((1 << vr_lg) - 1)) << epv_lg;
        if (v < n_vec && row[u] < rows && col[u] + (1 << epv_lg) <= cols)
          q[u] = __ldcs(reinterpret_cast<const uint4 *>(lb + row[u] * pitch_l + (long long)col[u] * es));
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int v = v0 + u * (int)blockDim.x;
        if (v >= n_vec || row[u] >= rows) continue;
        if (col[u] + (1 << epv_lg) <= cols) {
          __stcs(reinterpret_cast<uint4 *>(sb + row[u] * pitch_s + (long long)col[u] * es), q[u]);
        } else {
          // ragged right edge: element by element
          for (int e = col[u]; e < cols; ++e) {
            const char *ps = lb + row[u] * pitch_l + (long long)e * es;
            char *pd = sb + row[u] * pitch_s + (long long)e * es;
            st_raw(pd, es, ld_raw(ps, es));
          }
        }
      }
    }
  }
}

constexpr int FLAT_UNROLL = 4;

// out = OPC(in0, in1) over the flat range.  The leading `interior` vectors lie below
// every access's limit and all three accesses are aligned fp32, so they run as a bare
// 16-byte load/load/op/store stream with FLAT_UNROLL independent vectors per thread;
// the ragged remainder (and any unaligned or narrow access) takes the checked path.
template <int OPC>
__device__ __forceinline__ void flat_binary_body(const FlatParams &P) {
  const FlatAcc &A0 = P.acc[P.ops[0].a];
  const FlatAcc &A1 = P.acc[P.ops[1].a];
  const FlatAcc &AS = P.acc[P.ops[3].a];
  const long long n_vec = (P.g_hi - P.g_lo) >> 2;
  long long interior = 0;
  if (A0.vec_ok && A1.vec_ok && AS.vec_ok && A0.esize == 4 && A1.esize == 4 && AS.esize == 4) {
    long long lim = A0.limit < A1.limit ? A0.limit : A1.limit;
    lim = lim < AS.limit ? lim : AS.limit;
    interior = (lim - P.g_lo) >> 2;
    interior = interior < 0 ? 0 : (interior > n_vec ? n_vec : interior);
  }
  const long long tid = (long long)blockIdx.x * blockDim.x * FLAT_UNROLL + threadIdx.x;
  const long long step = (long long)gridDim.x * blockDim.x * FLAT_UNROLL;
  {
    const float4 *pa = reinterpret_cast<const float4 *>(A0.base + (A0.shift + P.g_lo) * 4);
    const float4 *pb = reinterpret_cast<const float4 *>(A1.base + (A1.shift + P.g_lo) * 4);
    float4 *pc = reinterpret_cast<float4 *>(AS.base + (AS.shift + P.g_lo) * 4);
    long long v0 = tid;
    for (; v0 + (FLAT_UNROLL - 1) * (long long)blockDim.x < interior; v0 += step) {
      float4 a[FLAT_UNROLL], b[FLAT_UNROLL];
#pragma unroll
      for (int u = 0; u < FLAT_UNROLL; ++u) {
        a[u] = __ldcs(pa + v0 + u * blockDim.x);
        b[u] = __ldcs(pb + v0 + u * blockDim.x);
      }
#pragma unroll
      for (int u = 0; u < FLAT_UNROLL; ++u) {
        float4 r;
        r.x = binf(OPC, a[u].x, b[u].x);
        r.y = binf(OPC, a[u].y, b[u].y);
        r.z = binf(OPC, a[u].z, b[u].z);
        r.w = binf(OPC, a[u].w, b[u].w);
        __stcs(pc + v0 + u * blockDim.x, r);
      }
    }
    // this thread's leftover interior vectors of its last, partial group
    for (int u = 0; u < FLAT_UNROLL; ++u) {
      const long long v = v0 + u * (long long)blockDim.x;
      if (v < interior) {
        const float4 x = __ldcs(pa + v), y = __ldcs(pb + v);
        float4 r;
        r.x = binf(OPC, x.x, y.x);
        r.y = binf(OPC, x.y, y.y);
        r.z = binf(OPC, x.z, y.z);
        r.w = binf(OPC, x.w, y.w);
        __stcs(pc + v, r);
      }
    }
  }
  // checked path for everything at or beyond `interior`
  const long long gstep = (long long)gridDim.x * blockDim.x;
  for (long long v = interior + (long long)blockIdx.x * blockDim.x + threadIdx.x; v < n_vec; v += gstep) {
    unsigned a[4], b[4], r[4];
    flat_load(A0, P.g_lo + v * 4, a);
    flat_load(A1, P.g_lo + v * 4, b);
#pragma unroll
    for (int k = 0; k < 4; ++k) r[k] = __float_as_uint(binf(OPC, __uint_as_float(a[k]), __uint_as_float(b[k])));
    flat_store(AS, P.g_lo + v * 4, r);
  }
}

__global__ void __launch_bounds__(256) ew_flat_binary_f32_kernel(const __grid_constant__ FlatParams P) {
  switch (P.ops[2].opcode) {
    case TSB_OP_ADDF: flat_binary_body<TSB_OP_ADDF>(P); break;
    case TSB_OP_SUBF: flat_binary_body<TSB_OP_SUBF>(P); break;
    case TSB_OP_MULF: flat_binary_body<TSB_OP_MULF>(P); break;
    case TSB_OP_DIVF: flat_binary_body<TSB_OP_DIVF>(P); break;
    case TSB_OP_MAXNUMF: flat_binary_body<TSB_OP_MAXNUMF>(P); break;
    case TSB_OP_MINNUMF: flat_binary_body<TSB_OP_MINNUMF>(P); break;
    case TSB_OP_MAXIMUMF: flat_binary_body<TSB_OP_MAXIMUMF>(P); break;
    case TSB_OP_MINIMUMF: flat_binary_body<TSB_OP_MINIMUMF>(P); break;
  }
}


static int build_params(const tsb_access *acc, int n_acc, const tsb_op *ops, int n_ops,
                        const int32_t grid[3], int64_t pid_lo, int64_t pid_hi, EwParams &P,
                        int &vec) {  // on return P.ops / P.n_ops hold the body without its loop ops
  if (!acc || !ops || !grid) return fail(TSB_ERR_INVALID, "tsb_elementwise: null argument");
  if (n_acc < 1 || n_acc > TSB_MAX_ACCESSES)
    return fail(TSB_ERR_UNSUPPORTED, "tsb_elementwise: %d accesses (max %d)", n_acc, TSB_MAX_ACCESSES);
  if (n_ops < 1 || n_ops > TSB_MAX_OPS)
    return fail(TSB_ERR_UNSUPPORTED, "tsb_elementwise: %d ops (max %d)", n_ops, TSB_MAX_OPS);
  long long total = (long long)grid[0] * grid[1] * grid[2];
  if (grid[0] < 0 || grid[1] < 0 || grid[2] < 0 || pid_lo < 0 || pid_hi > total || pid_lo > pid_hi)
    return fail(TSB_ERR_INVALID, "tsb_elementwise: program range [%lld,%lld) outside grid of %lld",
                (long long)pid_lo, (long long)pid_hi, total);
  memset(&P, 0, sizeof(P));
  const int rank = acc[0].rank;
  if (rank < 1 || rank > TSB_MAX_RANK) return fail(TSB_ERR_UNSUPPORTED, "tsb_elementwise: rank %d", rank);
  // iteration space, padded to rank 3 with leading unit dims
  long long sz[3] = {1, 1, 1};
  for (int d = 0; d < rank; ++d) sz[3 - rank + d] = acc[0].sizes[d];
  long long lanes = 1;
  for (int d = 0; d < 3; ++d) {
    int lg = ilog2_exact(sz[d]);
    if (lg < 0) return fail(TSB_ERR_INVALID, "tsb_elementwise: block size %lld is not a power of two", sz[d]);
    P.size[d] = (int)sz[d];
    P.lg[d] = lg;
    lanes *= sz[d];
  }
  if (lanes > (1ll << 24)) return fail(TSB_ERR_UNSUPPORTED, "tsb_elementwise: block of %lld lanes", lanes);
  P.lanes = (int)lanes;
  vec = (sz[2] % 4 == 0) ? 4 : 1;
  for (int a = 0; a < n_acc; ++a) {
    int rc = convert_access(acc, a, rank, P.size, grid, vec, P.acc[a]);
    if (rc != TSB_OK) return rc;
  }
  // a perfect loop nest around the whole body: leading LOOP_BEGINs (slot = nesting depth, imm =
  // trip count) matched by trailing LOOP_ENDs
  int n_loops = 0;
  while (n_loops < n_ops && ops[n_loops].opcode == TSB_OP_LOOP_BEGIN) ++n_loops;
  if (n_loops > TSB_MAX_LOOPS) return fail(TSB_ERR_UNSUPPORTED, "tsb_elementwise: loops nested %d deep (max %d)", n_loops, TSB_MAX_LOOPS);
  if (n_ops < 2 * n_loops + 1) return fail(TSB_ERR_INVALID, "tsb_elementwise: loop ops without a body");
  P.total_trips = 1;
  for (int l = 0; l < n_loops; ++l) {
    const tsb_op &b = ops[l], &e = ops[n_ops - 1 - l];
    if (b.a != l || e.opcode != TSB_OP_LOOP_END || e.a != l)
      return fail(TSB_ERR_UNSUPPORTED, "tsb_elementwise: loops must form one perfect nest around the whole body");
    P.trip[l] = (int)b.imm;
    if ((long long)b.imm > 0x7fffffffll) return fail(TSB_ERR_INVALID, "tsb_elementwise: trip count %u", b.imm);
    P.total_trips *= (long long)b.imm;
    if (P.total_trips > (1ll << 40)) return fail(TSB_ERR_UNSUPPORTED, "tsb_elementwise: loop nest of more than 2^40 iterations");
  }
  P.n_loops = n_loops;
  ops += n_loops;
  n_ops -= 2 * n_loops;
  for (int a = 0; a < n_acc; ++a)
    for (int l = n_loops; l < TSB_MAX_LOOPS; ++l) {
      P.acc[a].off_loop[l] = 0;
      for (int d = 0; d < 3; ++d) P.acc[a].mstart_loop[d][l] = 0;
    }
  auto reg_ok = [](int r) { return r >= TSB_REG_IMM && r < TSB_NUM_REGS; };
  for (int k = 0; k < n_ops; ++k) {
    const tsb_op &o = ops[k];
    P.ops[k] = o;
    const bool is_mem = o.opcode == TSB_OP_LOAD || o.opcode == TSB_OP_STORE;
    if (o.opcode == TSB_OP_LOOP_BEGIN || o.opcode == TSB_OP_LOOP_END || o.opcode == TSB_OP_ARGREDUCE ||
        o.opcode == TSB_OP_SCAN)
      return fail(TSB_ERR_UNSUPPORTED, "tsb_elementwise: op %d (opcode %d) is not an elementwise op", k, o.opcode);
    if (is_mem && (o.a < 0 || o.a >= n_acc))
      return fail(TSB_ERR_INVALID, "tsb_elementwise: op %d names access %d of %d", k, o.a, n_acc);
    if (o.opcode == TSB_OP_LOAD && acc[o.a].is_store == 1)
      return fail(TSB_ERR_INVALID, "tsb_elementwise: op %d loads from a store access", k);
    if (o.opcode == TSB_OP_STORE && acc[o.a].is_store != 1)
      return fail(TSB_ERR_INVALID, "tsb_elementwise: op %d stores to a load access", k);
    if (o.opcode != TSB_OP_STORE && (o.dst < TSB_REG_ACC || o.dst >= TSB_NUM_REGS))
      return fail(TSB_ERR_INVALID, "tsb_elementwise: op %d register %d out of range", k, o.dst);
    if (is_mem) {
      if (o.imm & ~(MEM_INDEX | MEM_MASK)) return fail(TSB_ERR_INVALID, "tsb_elementwise: op %d has memory flags %u", k, o.imm);
      if (o.imm) P.indirect = 1;
      const int ix = o.opcode == TSB_OP_LOAD ? o.b : o.c, mk = o.opcode == TSB_OP_LOAD ? o.c : o.dst;
      if (((o.imm & MEM_INDEX) && (!reg_ok(ix) || ix == TSB_REG_IMM)) || ((o.imm & MEM_MASK) && (!reg_ok(mk) || mk == TSB_REG_IMM)))
        return fail(TSB_ERR_INVALID, "tsb_elementwise: op %d index or mask operand out of range", k);
      if (o.opcode == TSB_OP_STORE && !reg_ok(o.b))
        return fail(TSB_ERR_INVALID, "tsb_elementwise: op %d register %d out of range", k, o.b);
      continue;
    }
    if (o.opcode == TSB_OP_REDUCE) {
      const int c = (int)o.imm;
      const bool known = (c >= TSB_OP_ADDF && c <= TSB_OP_MINIMUMF && c != TSB_OP_SUBF && c != TSB_OP_DIVF) ||
                         c == TSB_OP_ADDI || c == TSB_OP_MULI || (c >= TSB_OP_MINSI && c <= TSB_OP_XORI);
      if (!known) return fail(TSB_ERR_UNSUPPORTED, "tsb_elementwise: op %d folds with opcode %d", k, c);
      if (!reg_ok(o.a) || o.a == TSB_REG_IMM || (o.a == TSB_REG_ACC && k == 0))
        return fail(TSB_ERR_INVALID, "tsb_elementwise: op %d register %d out of range", k, o.a);
      P.has_reduce = 1;
      continue;
    }
    const int regs[3] = {o.opcode == TSB_OP_CONST ? 0 : o.a, o.opcode == TSB_OP_CONST ? 0 : o.b,
                         (o.opcode == TSB_OP_SELECT || o.opcode == TSB_OP_FMA) ? o.c : 0};
    for (int r = 0; r < 3; ++r) {
      if (!reg_ok(regs[r]))
        return fail(TSB_ERR_INVALID, "tsb_elementwise: op %d register %d out of range", k, regs[r]);
      if (regs[r] == TSB_REG_IMM && o.opcode == TSB_OP_CAST)
        return fail(TSB_ERR_INVALID, "tsb_elementwise: op %d: a cast cannot take an immediate operand", k);
      if (regs[r] == TSB_REG_ACC && k == 0)
        return fail(TSB_ERR_INVALID, "tsb_elementwise: op 0 reads the accumulator");
    }
  }
  P.n_acc = n_acc;
  P.n_ops = n_ops;
  for (int k = 0; k < 3; ++k) P.grid[k] = grid[k] > 0 ? grid[k] : 1;
  choose_program_order(P.acc, n_acc, P.grid, pid_lo, pid_hi, P.order);
  P.pid_lo = pid_lo;
  P.pid_hi = pid_hi;
  return TSB_OK;
}

// Flat form of a launch, when every access follows the pid*BLOCK + lane idiom on a 1-D grid.
static bool build_flat(const EwParams &P, int vec, FlatParams &F) {
  if (vec != 4 || P.size[0] != 1 || P.size[1] != 1 || P.grid[1] != 1 || P.grid[2] != 1) return false;
  const long long B = P.size[2];
  for (int a = 0; a < P.n_acc; ++a) {
    const DAcc &d = P.acc[a];
    if (d.masked & 3) return false;
    if (d.n_wrap) return false;
    if (d.kind != 2 && (d.stride[2] != 1 || d.off_pid[0] != B)) return false;
    if ((d.masked & 4) && d.mstart_pid[2][0] != B) return false;
    FlatAcc &f = F.acc[a];
    f.base = d.base;
    f.shift = d.off0;
    f.limit = (d.masked & 4) ? d.bound[2] - d.mstart0[2] : 0x7fffffffffffffffll;
    f.dtype = d.dtype; f.esize = d.esize; f.has_other = d.has_other; f.kind = d.kind; f.other = d.other;
    f.vec_ok = d.kind < 2 && d.esize <= 4 && ((uintptr_t)d.base % (4ull * d.esize)) == 0 && d.off0 % 4 == 0;
  }
  memcpy(F.ops, P.ops, sizeof(tsb_op) * P.n_ops);
  F.n_acc = P.n_acc;
  F.n_ops = P.n_ops;
  F.g_lo = P.pid_lo * B;
  F.g_hi = P.pid_hi * B;
  return true;
}

// Registers the body touches (highest register number + 1): sizes the VM's shared-memory file.
static int vm_regs_used(const tsb_op *ops, int n_ops) {
  int hi = 0;
  for (int k = 0; k < n_ops; ++k) {
    const tsb_op &o = ops[k];
    if (o.opcode != TSB_OP_STORE && o.dst > hi) hi = o.dst;
    if (o.opcode == TSB_OP_STORE && o.b > hi) hi = o.b;
    if (o.opcode != TSB_OP_LOAD && o.opcode != TSB_OP_STORE && o.opcode != TSB_OP_CONST) {
      if (o.a > hi) hi = o.a;
      if (o.b > hi) hi = o.b;
      if (o.c > hi) hi = o.c;
    }
  }
  return hi + 1;
}

static bool is_copy(const tsb_access *acc, const tsb_op *ops, int n_ops) {
  return n_ops == 2 && ops[0].opcode == TSB_OP_LOAD && ops[1].opcode == TSB_OP_STORE &&
         (ops[1].b == TSB_REG_ACC || ops[1].b == ops[0].dst) && acc[ops[0].a].is_store == 0 &&
         acc[ops[0].a].dtype == acc[ops[1].a].dtype && acc[ops[0].a].dtype != TSB_I64;
}

// ew_copy2d_kernel applies when both sides are plain memory accesses of rank <= 2 with unit inner
// stride, every row start is 16-byte aligned and the two masks are the same descriptor.
static bool copy2d_ok(const EwParams &P, const int32_t grid[3]) {
  const DAcc &l = P.acc[P.ops[0].a], &st = P.acc[P.ops[1].a];
  if (P.size[0] != 1 || l.kind != 0 || st.kind != 1 || l.n_wrap || st.n_wrap) return false;
  if ((long long)P.size[2] * l.esize % 16 != 0) return false;
  if (l.masked != st.masked) return false;
  for (int d = 1; d < 3; ++d) {
    if (!(l.masked & (1 << d))) continue;
    if (l.mstart0[d] != st.mstart0[d] || l.bound[d] != st.bound[d]) return false;
    for (int k = 0; k < 3; ++k)
      if (l.mstart_pid[d][k] != st.mstart_pid[d][k]) return false;
  }
  const DAcc *both[2] = {&l, &st};
  for (const DAcc *d : both) {
    const long long es = d->esize;
    if (d->stride[2] != 1 || ((uintptr_t)d->base + d->off0 * es) % 16 != 0) return false;
    for (int k = 0; k < 3; ++k)
      if (grid[k] > 1 && (d->off_pid[k] * es) % 16 != 0) return false;
    if (P.size[1] > 1 && (d->stride[1] * es) % 16 != 0) return false;
  }
  return true;
}

// out = binop(load, load) on fp32, written with registers or with the accumulator forms.
// swapped: operand a of the binop comes from the second load.
static bool is_fast_binary(const tsb_access *acc, const tsb_op *ops, int n_ops, bool &swapped) {
  swapped = false;
  if (n_ops != 4) return false;
  if (ops[0].opcode != TSB_OP_LOAD || ops[1].opcode != TSB_OP_LOAD || ops[3].opcode != TSB_OP_STORE)
    return false;
  const int o = ops[2].opcode;
  if (o < TSB_OP_ADDF || o > TSB_OP_MINIMUMF || ops[2].type != TSB_F32) return false;
  auto source = [&](int x) {  // which load produced operand x of ops[2]
    if (x == TSB_REG_ACC) return 1;
    if (x >= 0 && x == ops[1].dst) return 1;
    if (x >= 0 && x == ops[0].dst) return 0;
    return -1;
  };
  const int sa = source(ops[2].a), sb = source(ops[2].b);
  if (sa < 0 || sb < 0 || sa == sb) return false;
  if (!(ops[3].b == TSB_REG_ACC || (ops[3].b >= 0 && ops[3].b == ops[2].dst))) return false;
  swapped = sa == 1;
  return acc[ops[0].a].dtype == TSB_F32 && acc[ops[1].a].dtype == TSB_F32 &&
         acc[ops[3].a].dtype == TSB_F32;
}

}  // namespace tsb

using namespace tsb;

extern "C" int tsb_elementwise(const tsb_access *acc, int n_acc, const tsb_op *ops_in, int n_ops_in,
                               const int32_t grid[3], int64_t pid_lo, int64_t pid_hi, void *stream) {
  static thread_local EwParams P;
  int vec = 1;
  int rc = build_params(acc, n_acc, ops_in, n_ops_in, grid, pid_lo, pid_hi, P, vec);
  if (rc != TSB_OK) return rc;
  const tsb_op *ops = P.ops;  // the body without its loop ops
  const int n_ops = P.n_ops;
  const long long n_prog = pid_hi - pid_lo;
  if (n_prog == 0 || P.total_trips == 0) return TSB_OK;
  const int items = P.lanes / vec;
  int threads = items >= 256 ? 256 : (items >= 128 ? 128 : (items >= 64 ? 64 : 32));
  const long long max_ctas = (long long)sm_count() * (2048 / threads) * 4;
  cudaStream_t s = (cudaStream_t)stream;
  // eligible for the flat and the dedicated kernels
  const bool plain = P.n_loops == 0 && !P.indirect && !P.has_reduce;
  bool swapped = false;
  const bool fast_binary = plain && is_fast_binary(acc, ops, n_ops, swapped);
  if (fast_binary && swapped) {  // the fast kernels take ops[0] as the load of operand a
    const int t = P.ops[0].a;
    P.ops[0].a = P.ops[1].a;
    P.ops[1].a = t;
  }
  const int regs_used = vm_regs_used(ops, n_ops);
  static thread_local FlatParams F;
  if (plain && build_flat(P, vec, F)) {
    const long long n_vec = (F.g_hi - F.g_lo) / 4;
    const bool fast = fast_binary;
    // the VM's register file lives in shared memory: fewer threads per CTA when the body uses many registers
    int flat_threads = 256;
    const size_t regs_bytes = (size_t)regs_used * FLAT_VM_U * 4 * sizeof(unsigned);
    while (!fast && regs_bytes * flat_threads > 96 * 1024 && flat_threads > 32) flat_threads /= 2;
    const long long per_cta = fast ? 256ll * FLAT_UNROLL : (long long)flat_threads * FLAT_VM_U;
    long long ctas = (n_vec + per_cta - 1) / per_cta;
    const long long cap = (long long)sm_count() * 8 * 4;
    if (ctas > cap) ctas = cap;
    if (fast) {
      ew_flat_binary_f32_kernel<<<(unsigned)ctas, 256, 0, s>>>(F);
    } else {
      rc = launch_flat_vm(F, (unsigned)ctas, flat_threads, regs_bytes * flat_threads, s);
      if (rc != TSB_OK) return rc;
    }
    TSB_LAUNCH_OK("ew_flat_kernel");
    return TSB_OK;
  }
  // the blocked binary kernel derives its access state per thread: worth it only when a thread
  // then moves several vectors per program; smaller blocks go to the packed kernel below
  if (fast_binary && (items > 256 || vec != 4)) {
    long long ctas = (n_prog + 1) / 2;
    if (ctas > max_ctas) ctas = max_ctas;
    if (vec == 4) ew_binary_f32_kernel<4><<<(unsigned)ctas, threads, 0, s>>>(P);
    else ew_binary_f32_kernel<1><<<(unsigned)ctas, threads, 0, s>>>(P);
    TSB_LAUNCH_OK("ew_binary_f32_kernel");
    return TSB_OK;
  }
  if (plain && is_copy(acc, ops, n_ops)) {
    long long ctas = n_prog < max_ctas ? n_prog : max_ctas;
    if (copy2d_ok(P, grid)) {
      ew_copy2d_kernel<<<(unsigned)ctas, 256, 0, s>>>(P);
      TSB_LAUNCH_OK("ew_copy2d_kernel");
      return TSB_OK;
    }
    if (vec == 4) ew_copy_kernel<4><<<(unsigned)ctas, threads, 0, s>>>(P);
    else ew_copy_kernel<1><<<(unsigned)ctas, threads, 0, s>>>(P);
    TSB_LAUNCH_OK("ew_copy_kernel");
    return TSB_OK;
  }
  if (vec == 4 && items >= 4 && items <= 1024) {
    // packed form: items / 4 threads per program, several programs per CTA
    rc = launch_ew_packed(P, items, regs_used, s);
    if (rc != TSB_ERR_UNSUPPORTED) return rc;
  }
  if (P.has_reduce)  // only the packed kernel's threads know the other threads of their program
    return fail(TSB_ERR_UNSUPPORTED, "tsb_elementwise: a body with a fold needs blocks of 16 to 4096 lanes, a multiple of 4, and at most 12 live registers");
  // four lane-vectors per thread when the block is large enough to keep at least a warp busy
  const int U = (vec == 4 && items >= 128) ? 4 : 1;
  if (U == 4) {
    threads = items / 4 >= 256 ? 256 : (items / 4 >= 128 ? 128 : (items / 4 >= 64 ? 64 : 32));
  }
  while ((size_t)regs_used * U * vec * threads * sizeof(unsigned) > 96 * 1024 && threads > 32) threads /= 2;
  long long ctas = n_prog < max_ctas ? n_prog : max_ctas;
  const size_t smem = (size_t)regs_used * U * vec * threads * sizeof(unsigned);
  static SmemLimit lim44, lim41;
  if (smem > 48 * 1024) {
    TSB_CUDA_OK(allow_dynamic_smem(ew_vm_kernel<4, 4>, 200 * 1024, lim44));
    TSB_CUDA_OK(allow_dynamic_smem(ew_vm_kernel<4, 1>, 200 * 1024, lim41));
  }
  if (U == 4) ew_vm_kernel<4, 4><<<(unsigned)ctas, threads, smem, s>>>(P);
  else if (vec == 4) ew_vm_kernel<4, 1><<<(unsigned)ctas, threads, smem, s>>>(P);
  else ew_vm_kernel<1, 1><<<(unsigned)ctas, threads, smem, s>>>(P);
  TSB_LAUNCH_OK("ew_vm_kernel");
  return TSB_OK;
}

extern "C" int tsb_block_copy(const tsb_access *src, const tsb_access *dst, const int32_t grid[3],
                              int64_t pid_lo, int64_t pid_hi, void *stream) {
  if (!src || !dst) return fail(TSB_ERR_INVALID, "tsb_block_copy: null access");
  if (src->dtype != dst->dtype)
    return fail(TSB_ERR_INVALID, "tsb_block_copy: source and destination element types differ");
  tsb_access acc[2] = {*src, *dst};
  acc[0].is_store = 0;
  acc[1].is_store = 1;
  tsb_op ops[2];
  memset(ops, 0, sizeof(ops));
  ops[0].opcode = TSB_OP_LOAD; ops[0].type = src->dtype; ops[0].dst = 0; ops[0].a = 0;
  ops[1].opcode = TSB_OP_STORE; ops[1].type = dst->dtype; ops[1].a = 1; ops[1].b = 0;
  return tsb_elementwise(acc, 2, ops, 2, grid, pid_lo, pid_hi, stream);
}
