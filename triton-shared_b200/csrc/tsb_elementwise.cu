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
#include "tsb_common.cuh"
#include <math.h>
#include <string.h>

namespace tsb {

struct DAcc {
  char *base;
  long long off0;
  long long off_pid[3];
  long long stride[3];
  long long mstart0[3];
  long long mstart_pid[3][3];
  long long bound[3];
  int masked;     // bit d set: dim d carries a mask
  int dtype;
  int esize;
  int vec_ok;     // innermost dim contiguous and every vector 16B/8B/4B aligned
  int has_other;
  unsigned other; // fill value in register representation
  int kind;       // 0 memory load, 1 memory store, 2 mask probe, 3 index probe
  int n_wrap;     // wrap-around (modulo) terms
  int wrap_inner; // some wrap term is on the innermost dim (lanes of a vector differ non-linearly)
  struct {
    int dim;
    long long off0, off_pid[3], stride, modulus, scale;
  } wrap[2];
};

struct EwParams {
  DAcc acc[TSB_MAX_ACCESSES];
  tsb_op ops[TSB_MAX_OPS];
  int n_acc, n_ops;
  int size[3];
  int lg[3];      // log2 of sizes (Triton block shapes are powers of two)
  int lanes;      // size[0]*size[1]*size[2]
  int grid[3];
  long long pid_lo, pid_hi;
};

// ---- register representation -------------------------------------------------
// Every VM lane is 32 bits: f32 bits for all float types (f16/bf16 values are
// held exactly widened and re-rounded after each op), sign/zero-extended ints.

__device__ __forceinline__ unsigned ld_elem(const char *p, int dt) {
  switch (dt) {
    case TSB_F32: case TSB_I32: case TSB_U32: return *reinterpret_cast<const unsigned *>(p);
    case TSB_F16: return __float_as_uint(__half2float(*reinterpret_cast<const __half *>(p)));
    case TSB_BF16: return __float_as_uint(__bfloat162float(*reinterpret_cast<const __nv_bfloat16 *>(p)));
    case TSB_I16: return (unsigned)(int)*reinterpret_cast<const short *>(p);
    case TSB_U16: return (unsigned)*reinterpret_cast<const unsigned short *>(p);
    case TSB_I8: return (unsigned)(int)*reinterpret_cast<const signed char *>(p);
    case TSB_U8: case TSB_I1: return (unsigned)*reinterpret_cast<const unsigned char *>(p);
  }
  return 0u;
}
__device__ __forceinline__ void st_elem(char *p, int dt, unsigned v) {
  switch (dt) {
    case TSB_F32: case TSB_I32: case TSB_U32: *reinterpret_cast<unsigned *>(p) = v; break;
    case TSB_F16: *reinterpret_cast<__half *>(p) = __float2half_rn(__uint_as_float(v)); break;
    case TSB_BF16: *reinterpret_cast<__nv_bfloat16 *>(p) = __float2bfloat16_rn(__uint_as_float(v)); break;
    case TSB_I16: case TSB_U16: *reinterpret_cast<unsigned short *>(p) = (unsigned short)v; break;
    case TSB_I8: case TSB_U8: *reinterpret_cast<unsigned char *>(p) = (unsigned char)v; break;
    case TSB_I1: *reinterpret_cast<unsigned char *>(p) = (unsigned char)(v & 1u); break;
  }
}

// Round an fp32 result to the value set of `dt` (identity for f32).
__device__ __forceinline__ float round_to(float x, int dt) {
  if (dt == TSB_F16) return __half2float(__float2half_rn(x));
  if (dt == TSB_BF16) return __bfloat162float(__float2bfloat16_rn(x));
  return x;
}
// Wrap an integer result to the width of `dt`.
__device__ __forceinline__ unsigned wrap_to(unsigned x, int dt) {
  switch (dt) {
    case TSB_I16: return (unsigned)(int)(short)x;
    case TSB_U16: return x & 0xffffu;
    case TSB_I8: return (unsigned)(int)(signed char)x;
    case TSB_U8: return x & 0xffu;
    case TSB_I1: return x & 1u;
  }
  return x;
}

__device__ __forceinline__ float maximumf_(float a, float b) {
  return (a != a || b != b) ? __uint_as_float(0x7fc00000u) : fmaxf(a, b);
}
__device__ __forceinline__ float minimumf_(float a, float b) {
  return (a != a || b != b) ? __uint_as_float(0x7fc00000u) : fminf(a, b);
}

__device__ __forceinline__ float binf(int opc, float a, float b) {
  switch (opc) {
    case TSB_OP_ADDF: return a + b;
    case TSB_OP_SUBF: return a - b;
    case TSB_OP_MULF: return a * b;
    case TSB_OP_DIVF: return a / b;
    case TSB_OP_MAXNUMF: return fmaxf(a, b);
    case TSB_OP_MINNUMF: return fminf(a, b);
    case TSB_OP_MAXIMUMF: return maximumf_(a, b);
    case TSB_OP_MINIMUMF: return minimumf_(a, b);
    case TSB_OP_REMF: return fmodf(a, b);
  }
  return 0.f;
}
__device__ __forceinline__ float unf(int opc, float a) {
  switch (opc) {
    case TSB_OP_EXP: return expf(a);
    case TSB_OP_EXP2: return exp2f(a);
    case TSB_OP_LOG: return logf(a);
    case TSB_OP_LOG2: return log2f(a);
    case TSB_OP_SQRT: return sqrtf(a);
    case TSB_OP_RSQRT: return 1.0f / sqrtf(a);
    case TSB_OP_SIN: return sinf(a);
    case TSB_OP_COS: return cosf(a);
    case TSB_OP_TANH: return tanhf(a);
    case TSB_OP_ERF: return erff(a);
    case TSB_OP_ABSF: return fabsf(a);
    case TSB_OP_NEGF: return -a;
    case TSB_OP_FLOOR: return floorf(a);
    case TSB_OP_CEIL: return ceilf(a);
  }
  return 0.f;
}
__device__ __forceinline__ unsigned bini(int opc, unsigned ua, unsigned ub) {
  int a = (int)ua, b = (int)ub;
  switch (opc) {
    case TSB_OP_ADDI: return ua + ub;
    case TSB_OP_SUBI: return ua - ub;
    case TSB_OP_MULI: return ua * ub;
    case TSB_OP_DIVSI: return b == 0 ? 0u : (b == -1 ? (unsigned)(0u - ua) : (unsigned)(a / b));
    case TSB_OP_REMSI: return (b == 0 || b == -1) ? 0u : (unsigned)(a % b);
    case TSB_OP_DIVUI: return ub == 0 ? 0u : ua / ub;
    case TSB_OP_REMUI: return ub == 0 ? 0u : ua % ub;
    case TSB_OP_MINSI: return (unsigned)min(a, b);
    case TSB_OP_MAXSI: return (unsigned)max(a, b);
    case TSB_OP_MINUI: return min(ua, ub);
    case TSB_OP_MAXUI: return max(ua, ub);
    case TSB_OP_ANDI: return ua & ub;
    case TSB_OP_ORI: return ua | ub;
    case TSB_OP_XORI: return ua ^ ub;
    case TSB_OP_SHLI: return ub >= 32 ? 0u : ua << ub;
    case TSB_OP_SHRSI: return (unsigned)(a >> (ub >= 32 ? 31 : ub));
    case TSB_OP_SHRUI: return ub >= 32 ? 0u : ua >> ub;
  }
  return 0u;
}
__device__ __forceinline__ unsigned cmpf_(unsigned pred, float a, float b) {
  bool un = (a != a) || (b != b);
  switch (pred) {
    case TSB_CMPF_OEQ: return !un && a == b;
    case TSB_CMPF_OGT: return !un && a > b;
    case TSB_CMPF_OGE: return !un && a >= b;
    case TSB_CMPF_OLT: return !un && a < b;
    case TSB_CMPF_OLE: return !un && a <= b;
    case TSB_CMPF_ONE: return !un && a != b;
    case TSB_CMPF_ORD: return !un;
    case TSB_CMPF_UEQ: return un || a == b;
    case TSB_CMPF_UGT: return un || a > b;
    case TSB_CMPF_UGE: return un || a >= b;
    case TSB_CMPF_ULT: return un || a < b;
    case TSB_CMPF_ULE: return un || a <= b;
    case TSB_CMPF_UNE: return un || a != b;
    case TSB_CMPF_UNO: return un;
  }
  return 0u;
}
__device__ __forceinline__ unsigned cmpi_(unsigned pred, unsigned ua, unsigned ub) {
  int a = (int)ua, b = (int)ub;
  switch (pred) {
    case TSB_CMPI_EQ: return ua == ub;
    case TSB_CMPI_NE: return ua != ub;
    case TSB_CMPI_SLT: return a < b;
    case TSB_CMPI_SLE: return a <= b;
    case TSB_CMPI_SGT: return a > b;
    case TSB_CMPI_SGE: return a >= b;
    case TSB_CMPI_ULT: return ua < ub;
    case TSB_CMPI_ULE: return ua <= ub;
    case TSB_CMPI_UGT: return ua > ub;
    case TSB_CMPI_UGE: return ua >= ub;
  }
  return 0u;
}
__device__ __forceinline__ bool is_float_dt(int dt) {
  return dt == TSB_F32 || dt == TSB_F16 || dt == TSB_BF16;
}
__device__ __forceinline__ bool is_unsigned_dt(int dt) {
  return dt == TSB_U32 || dt == TSB_U16 || dt == TSB_U8 || dt == TSB_I1;
}
// arith.extf/truncf/sitofp/uitofp/fptosi/fptoui/extsi/extui/trunci between
// register representations.
__device__ __forceinline__ unsigned cast_(unsigned v, int from, int to, unsigned mode) {
  bool ff = is_float_dt(from), tf = is_float_dt(to);
  if (ff && tf) return __float_as_uint(round_to(__uint_as_float(v), to));
  if (!ff && tf) {
    // mode 1: treat the source as unsigned (uitofp)
    float f = (mode == 1u || is_unsigned_dt(from)) ? __uint2float_rn(v) : __int2float_rn((int)v);
    return __float_as_uint(round_to(f, to));
  }
  if (ff && !tf) {
    float f = __uint_as_float(v);
    unsigned r = (mode == 1u || is_unsigned_dt(to)) ? __float2uint_rz(f) : (unsigned)__float2int_rz(f);
    return wrap_to(r, to);
  }
  // int -> int: mode 1 = zero extension of the source width (extui)
  if (mode == 1u) {
    int fs = dtype_size(from);
    if (fs == 1) v &= (from == TSB_I1 ? 1u : 0xffu);
    else if (fs == 2) v &= 0xffffu;
  }
  return wrap_to(v, to);
}

struct ProgState {
  long long off;
  long long woff[2];
  int dim[3];
};

// scale * ((offset + i*stride) mod modulus) summed over the access's wrap terms
__device__ __forceinline__ long long wrap_addend(const DAcc &A, const ProgState &s, int i0, int i1, int i2) {
  long long add = 0;
  for (int w = 0; w < A.n_wrap; ++w) {
    const int id = A.wrap[w].dim == 0 ? i0 : (A.wrap[w].dim == 1 ? i1 : i2);
    add += A.wrap[w].scale * ((s.woff[w] + id * A.wrap[w].stride) % A.wrap[w].modulus);
  }
  return add;
}

__device__ __forceinline__ void program_state(const DAcc &A, const int size[3], long long px,
                                              long long py, long long pz, ProgState &s) {
  s.off = A.off0 + A.off_pid[0] * px + A.off_pid[1] * py + A.off_pid[2] * pz;
  for (int w = 0; w < A.n_wrap; ++w)
    s.woff[w] = A.wrap[w].off0 + A.wrap[w].off_pid[0] * px + A.wrap[w].off_pid[1] * py + A.wrap[w].off_pid[2] * pz;
#pragma unroll
  for (int d = 0; d < 3; ++d) {
    int dim = size[d];
    if (A.masked & (1 << d)) {
      long long st = A.mstart0[d] + A.mstart_pid[d][0] * px + A.mstart_pid[d][1] * py +
                     A.mstart_pid[d][2] * pz;
      long long en = st + size[d];
      long long m = en < A.bound[d] ? en : A.bound[d];
      m = m > st ? m : st;
      dim = (int)(m - st);
    }
    s.dim[d] = dim;
  }
}

template <int VEC>
__device__ __forceinline__ void load_vec(const DAcc &A, const ProgState &s, int i0, int i1, int i2,
                                         unsigned out[VEC]) {
  const bool outer = i0 < s.dim[0] && i1 < s.dim[1];
  long long e = s.off + i0 * A.stride[0] + i1 * A.stride[1] + i2 * A.stride[2];
  const unsigned fill = A.has_other ? A.other : 0u;
  if (A.n_wrap) {
    if (A.wrap_inner) {
      // lanes of the vector wrap independently: one scalar access per lane
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        const bool ok = outer && (i2 + k) < s.dim[2];
        const long long ek = e + k * A.stride[2] + wrap_addend(A, s, i0, i1, i2 + k);
        out[k] = A.kind == 2 ? (ok ? 1u : 0u)
                             : (A.kind == 3 ? (unsigned)ek : (ok ? ld_elem(A.base + ek * A.esize, A.dtype) : fill));
      }
      return;
    }
    e += wrap_addend(A, s, i0, i1, i2);
  }
  if (A.kind >= 2) {
    // probes read no memory: 2 yields the lane's mask bit, 3 its linear index
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      const bool ok = outer && (i2 + k) < s.dim[2];
      out[k] = A.kind == 2 ? (ok ? 1u : 0u) : (unsigned)(e + k * A.stride[2]);
    }
    return;
  }
  if (VEC == 4 && A.vec_ok && outer && i2 + VEC <= s.dim[2]) {
    const char *p = A.base + e * A.esize;
    if (A.esize == 4) {
      uint4 v = __ldg(reinterpret_cast<const uint4 *>(p));
      out[0] = v.x; out[1 % VEC] = v.y; out[2 % VEC] = v.z; out[3 % VEC] = v.w;
    } else if (A.esize == 2) {
      uint2 v = __ldg(reinterpret_cast<const uint2 *>(p));
      unsigned short h[4] = {(unsigned short)(v.x & 0xffff), (unsigned short)(v.x >> 16),
                             (unsigned short)(v.y & 0xffff), (unsigned short)(v.y >> 16)};
#pragma unroll
      for (int k = 0; k < VEC; ++k) out[k] = ld_elem(reinterpret_cast<const char *>(&h[k]), A.dtype);
    } else {
      unsigned v = __ldg(reinterpret_cast<const unsigned *>(p));
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        unsigned char b = (unsigned char)(v >> (8 * k));
        out[k] = ld_elem(reinterpret_cast<const char *>(&b), A.dtype);
      }
    }
    return;
  }
#pragma unroll
  for (int k = 0; k < VEC; ++k) {
    bool ok = outer && (i2 + k) < s.dim[2];
    out[k] = ok ? ld_elem(A.base + (e + k * A.stride[2]) * A.esize, A.dtype) : fill;
  }
}

template <int VEC>
__device__ __forceinline__ void store_vec(const DAcc &A, const ProgState &s, int i0, int i1, int i2,
                                          const unsigned in[VEC]) {
  const bool outer = i0 < s.dim[0] && i1 < s.dim[1];
  if (!outer) return;
  long long e = s.off + i0 * A.stride[0] + i1 * A.stride[1] + i2 * A.stride[2];
  if (A.n_wrap) {
    if (A.wrap_inner) {
#pragma unroll
      for (int k = 0; k < VEC; ++k)
        if (i2 + k < s.dim[2])
          st_elem(A.base + (e + k * A.stride[2] + wrap_addend(A, s, i0, i1, i2 + k)) * A.esize, A.dtype, in[k]);
      return;
    }
    e += wrap_addend(A, s, i0, i1, i2);
  }
  if (VEC == 4 && A.vec_ok && i2 + VEC <= s.dim[2]) {
    char *p = A.base + e * A.esize;
    if (A.esize == 4) {
      *reinterpret_cast<uint4 *>(p) = make_uint4(in[0], in[1 % VEC], in[2 % VEC], in[3 % VEC]);
    } else if (A.esize == 2) {
      unsigned short h[4];
#pragma unroll
      for (int k = 0; k < VEC; ++k) st_elem(reinterpret_cast<char *>(&h[k]), A.dtype, in[k]);
      *reinterpret_cast<uint2 *>(p) =
          make_uint2((unsigned)h[0] | ((unsigned)h[1] << 16), (unsigned)h[2] | ((unsigned)h[3] << 16));
    } else {
      unsigned v = 0;
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        unsigned char b;
        st_elem(reinterpret_cast<char *>(&b), A.dtype, in[k]);
        v |= (unsigned)b << (8 * k);
      }
      *reinterpret_cast<unsigned *>(p) = v;
    }
    return;
  }
#pragma unroll
  for (int k = 0; k < VEC; ++k)
    if (i2 + k < s.dim[2]) st_elem(A.base + (e + k * A.stride[2]) * A.esize, A.dtype, in[k]);
}

// ---- general body: a small register VM ----------------------------------------
// One pass over the op list for VEC lanes; `ld(access, regs)` and `st(access, regs)`
// are supplied by the kernel (blocked or flat addressing).
template <int VEC, typename LoadFn, typename StoreFn>
__device__ __forceinline__ void vm_exec(const tsb_op *ops, int n_ops, LoadFn ld, StoreFn st) {
  unsigned R[TSB_NUM_REGS][VEC];
  for (int k = 0; k < n_ops; ++k) {
    const tsb_op &op = ops[k];
    const int opc = op.opcode;
    if (opc == TSB_OP_LOAD) {
      ld(op.a, R[op.dst]);
    } else if (opc == TSB_OP_STORE) {
      st(op.a, R[op.b]);
    } else if (opc == TSB_OP_CONST) {
#pragma unroll
      for (int v = 0; v < VEC; ++v) R[op.dst][v] = op.imm;
    } else if (opc == TSB_OP_MOV) {
#pragma unroll
      for (int v = 0; v < VEC; ++v) R[op.dst][v] = R[op.a][v];
    } else if (opc >= TSB_OP_ADDF && opc < TSB_OP_EXP) {
#pragma unroll
      for (int v = 0; v < VEC; ++v)
        R[op.dst][v] = __float_as_uint(round_to(
            binf(opc, __uint_as_float(R[op.a][v]), __uint_as_float(R[op.b][v])), op.type));
    } else if (opc >= TSB_OP_EXP && opc < TSB_OP_ADDI) {
#pragma unroll
      for (int v = 0; v < VEC; ++v)
        R[op.dst][v] = __float_as_uint(round_to(unf(opc, __uint_as_float(R[op.a][v])), op.type));
    } else if (opc == TSB_OP_ABSI) {
#pragma unroll
      for (int v = 0; v < VEC; ++v) R[op.dst][v] = wrap_to((unsigned)abs((int)R[op.a][v]), op.type);
    } else if (opc >= TSB_OP_ADDI && opc < TSB_OP_CMPF) {
#pragma unroll
      for (int v = 0; v < VEC; ++v) R[op.dst][v] = wrap_to(bini(opc, R[op.a][v], R[op.b][v]), op.type);
    } else if (opc == TSB_OP_CMPF) {
#pragma unroll
      for (int v = 0; v < VEC; ++v)
        R[op.dst][v] = cmpf_(op.imm, __uint_as_float(R[op.a][v]), __uint_as_float(R[op.b][v]));
    } else if (opc == TSB_OP_CMPI) {
#pragma unroll
      for (int v = 0; v < VEC; ++v) R[op.dst][v] = cmpi_(op.imm, R[op.a][v], R[op.b][v]);
    } else if (opc == TSB_OP_SELECT) {
#pragma unroll
      for (int v = 0; v < VEC; ++v) R[op.dst][v] = (R[op.a][v] & 1u) ? R[op.b][v] : R[op.c][v];
    } else if (opc == TSB_OP_CAST) {
#pragma unroll
      for (int v = 0; v < VEC; ++v) R[op.dst][v] = cast_(R[op.a][v], (int)op.imm, op.type, op.imm2);
    } else if (opc == TSB_OP_BITCAST) {
      // only 32-bit <-> 32-bit bitcasts keep their bits in this representation
#pragma unroll
      for (int v = 0; v < VEC; ++v) R[op.dst][v] = R[op.a][v];
    } else if (opc == TSB_OP_FMA) {
#pragma unroll
      for (int v = 0; v < VEC; ++v)
        R[op.dst][v] = __float_as_uint(round_to(
            fmaf(__uint_as_float(R[op.a][v]), __uint_as_float(R[op.b][v]), __uint_as_float(R[op.c][v])),
            op.type));
    }
  }
}

// Program id of a linearised program index (x fastest). 1-D grids skip the divisions.
__device__ __forceinline__ void split_pid(const int grid[3], long long prog, long long &px, long long &py,
                                          long long &pz) {
  if (grid[1] == 1 && grid[2] == 1) {
    px = prog; py = 0; pz = 0;
    return;
  }
  const unsigned long long gx = (unsigned long long)grid[0], gy = (unsigned long long)grid[1];
  const unsigned long long q = (unsigned long long)prog / gx;
  px = (long long)((unsigned long long)prog - q * gx);
  py = (long long)(q % gy);
  pz = (long long)(q / gy);
}

template <int VEC>
__global__ void __launch_bounds__(256) ew_vm_kernel(const __grid_constant__ EwParams P) {
  const int items = P.lanes / VEC;
  const int sh1 = P.lg[2], sh0 = P.lg[2] + P.lg[1];
  for (long long prog = P.pid_lo + blockIdx.x; prog < P.pid_hi; prog += gridDim.x) {
    long long px, py, pz;
    split_pid(P.grid, prog, px, py, pz);
    ProgState st[TSB_MAX_ACCESSES];
    for (int a = 0; a < P.n_acc; ++a) program_state(P.acc[a], P.size, px, py, pz, st[a]);
    for (int it = threadIdx.x; it < items; it += blockDim.x) {
      const int l = it * VEC;
      const int i2 = l & (P.size[2] - 1);
      const int i1 = (l >> sh1) & (P.size[1] - 1);
      const int i0 = l >> sh0;
      vm_exec<VEC>(
          P.ops, P.n_ops,
          [&](int a, unsigned(&r)[VEC]) { load_vec<VEC>(P.acc[a], st[a], i0, i1, i2, r); },
          [&](int a, const unsigned(&r)[VEC]) { store_vec<VEC>(P.acc[a], st[a], i0, i1, i2, r); });
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
      split_pid(P.grid, prog, px, py, pz);
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

// ---- flat addressing ------------------------------------------------------------
// When every access is a unit-stride 1-D block whose offset and mask start advance
// by exactly the block size per program (the "pid * BLOCK + arange(BLOCK)" idiom on a
// 1-D grid), lane l of program p is element g = p*BLOCK + l of one flat range: it
// lives at base + shift + g and is accessible iff g < limit.  The kernels below walk
// that range with no per-program bookkeeping; results are identical to the blocked
// kernels.
struct FlatAcc {
  char *base;
  long long shift;
  long long limit;
  int dtype, esize, vec_ok, has_other, kind;
  unsigned other;
};
struct FlatParams {
  FlatAcc acc[TSB_MAX_ACCESSES];
  tsb_op ops[TSB_MAX_OPS];
  int n_acc, n_ops;
  long long g_lo, g_hi;
};

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
      unsigned short h[4] = {(unsigned short)(v.x & 0xffff), (unsigned short)(v.x >> 16),
                             (unsigned short)(v.y & 0xffff), (unsigned short)(v.y >> 16)};
#pragma unroll
      for (int k = 0; k < 4; ++k) out[k] = ld_elem(reinterpret_cast<const char *>(&h[k]), A.dtype);
    } else {
      const unsigned v = __ldcs(reinterpret_cast<const unsigned *>(p));
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        unsigned char b = (unsigned char)(v >> (8 * k));
        out[k] = ld_elem(reinterpret_cast<const char *>(&b), A.dtype);
      }
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
      unsigned short h[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) st_elem(reinterpret_cast<char *>(&h[k]), A.dtype, in[k]);
      __stcs(reinterpret_cast<uint2 *>(p),
             make_uint2((unsigned)h[0] | ((unsigned)h[1] << 16), (unsigned)h[2] | ((unsigned)h[3] << 16)));
    } else {
      unsigned v = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        unsigned char b;
        st_elem(reinterpret_cast<char *>(&b), A.dtype, in[k]);
        v |= (unsigned)b << (8 * k);
      }
      __stcs(reinterpret_cast<unsigned *>(p), v);
    }
    return;
  }
#pragma unroll
  for (int k = 0; k < 4; ++k)
    if (g + k < A.limit) st_elem(p + k * A.esize, A.dtype, in[k]);
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

__global__ void __launch_bounds__(256) ew_flat_vm_kernel(const __grid_constant__ FlatParams P) {
  const long long n_vec = (P.g_hi - P.g_lo) >> 2;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < n_vec; v += step) {
    const long long g = P.g_lo + v * 4;
    vm_exec<4>(
        P.ops, P.n_ops, [&](int a, unsigned(&r)[4]) { flat_load(P.acc[a], g, r); },
        [&](int a, const unsigned(&r)[4]) { flat_store(P.acc[a], g, r); });
  }
}

static unsigned other_to_reg(uint64_t bits, int dt) {
  switch (dt) {
    case TSB_F32: case TSB_I32: case TSB_U32: return (unsigned)bits;
    case TSB_F16: {
      __half_raw hr; hr.x = (unsigned short)bits;
      float f = __half2float(__half(hr));
      unsigned u; memcpy(&u, &f, 4); return u;
    }
    case TSB_BF16: return ((unsigned)(bits & 0xffffu)) << 16;
    case TSB_I16: return (unsigned)(int)(short)bits;
    case TSB_U16: return (unsigned)(bits & 0xffffu);
    case TSB_I8: return (unsigned)(int)(signed char)bits;
    case TSB_U8: return (unsigned)(bits & 0xffu);
    case TSB_I1: return (unsigned)(bits & 1u);
  }
  return 0u;
}

static int ilog2_exact(long long v) {
  int l = 0;
  while ((1ll << l) < v) ++l;
  return ((1ll << l) == v) ? l : -1;
}

static int build_params(const tsb_access *acc, int n_acc, const tsb_op *ops, int n_ops,
                        const int32_t grid[3], int64_t pid_lo, int64_t pid_hi, EwParams &P,
                        int &vec) {
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
    const tsb_access &s = acc[a];
    DAcc &d = P.acc[a];
    if (s.rank != rank) return fail(TSB_ERR_INVALID, "tsb_elementwise: access %d has rank %d, expected %d", a, s.rank, rank);
    const int es = dtype_size(s.dtype);
    if (es == 0 || es == 8)
      return fail(TSB_ERR_UNSUPPORTED, "tsb_elementwise: access %d has unsupported dtype %d", a, s.dtype);
    if (s.is_store < 0 || s.is_store > 3)
      return fail(TSB_ERR_INVALID, "tsb_elementwise: access %d has kind %d", a, s.is_store);
    if (!s.base && s.is_store < 2)
      return fail(TSB_ERR_INVALID, "tsb_elementwise: access %d has a null base pointer", a);
    d.kind = s.is_store;
    d.base = (char *)s.base;
    d.dtype = s.dtype;
    d.esize = es;
    d.off0 = s.offset0;
    for (int k = 0; k < 3; ++k) d.off_pid[k] = s.offset_pid[k];
    d.has_other = s.has_other;
    d.other = other_to_reg(s.other_bits, s.dtype);
    for (int k = 0; k < 3; ++k) { d.stride[k] = 0; d.bound[k] = 0; }
    for (int k = 0; k < rank; ++k) {
      const int o = 3 - rank + k;
      if (s.sizes[k] != acc[0].sizes[k])
        return fail(TSB_ERR_INVALID, "tsb_elementwise: access %d block shape differs in dim %d", a, k);
      d.stride[o] = s.strides[k];
      if (s.masked[k]) {
        d.masked |= 1 << o;
        d.mstart0[o] = s.mask_start0[k];
        for (int j = 0; j < 3; ++j) d.mstart_pid[o][j] = s.mask_start_pid[k][j];
        d.bound[o] = s.mask_bound[k];
      }
    }
    if (s.n_wrap < 0 || s.n_wrap > 2) return fail(TSB_ERR_INVALID, "tsb_elementwise: access %d has %d wrap terms", a, s.n_wrap);
    d.n_wrap = s.n_wrap;
    d.wrap_inner = 0;
    bool wrap_unaligned = false;
    for (int w = 0; w < s.n_wrap; ++w) {
      const tsb_wrap &sw = s.wrap[w];
      if (sw.dim < 0 || sw.dim >= rank) return fail(TSB_ERR_INVALID, "tsb_elementwise: access %d wraps dim %d of rank %d", a, sw.dim, rank);
      if (sw.modulus <= 0) return fail(TSB_ERR_INVALID, "tsb_elementwise: access %d has wrap modulus %lld", a, (long long)sw.modulus);
      d.wrap[w].dim = 3 - rank + sw.dim;
      d.wrap[w].off0 = sw.offset0;
      for (int j = 0; j < 3; ++j) d.wrap[w].off_pid[j] = sw.offset_pid[j];
      d.wrap[w].stride = sw.stride;
      d.wrap[w].modulus = sw.modulus;
      d.wrap[w].scale = sw.scale;
      if (d.wrap[w].dim == 2) d.wrap_inner = 1;
      if (sw.scale % 4 != 0) wrap_unaligned = true;
    }
    // 4-lane vectors need: unit inner stride, vector-aligned base and offsets
    const long long vb = 4ll * es;
    bool ok = vec == 4 && d.stride[2] == 1 && ((uintptr_t)d.base % vb) == 0 && d.off0 % 4 == 0;
    for (int k = 0; k < 3; ++k) ok = ok && (grid[k] <= 1 || d.off_pid[k] % 4 == 0);
    ok = ok && (P.size[1] <= 1 || d.stride[1] % 4 == 0) && (P.size[0] <= 1 || d.stride[0] % 4 == 0);
    ok = ok && !d.wrap_inner && !wrap_unaligned;
    d.vec_ok = ok ? 1 : 0;
  }
  for (int k = 0; k < n_ops; ++k) {
    const tsb_op &o = ops[k];
    P.ops[k] = o;
    const bool is_mem = o.opcode == TSB_OP_LOAD || o.opcode == TSB_OP_STORE;
    if (is_mem && (o.a < 0 || o.a >= n_acc))
      return fail(TSB_ERR_INVALID, "tsb_elementwise: op %d names access %d of %d", k, o.a, n_acc);
    if (o.opcode == TSB_OP_LOAD && acc[o.a].is_store == 1)
      return fail(TSB_ERR_INVALID, "tsb_elementwise: op %d loads from a store access", k);
    if (o.opcode == TSB_OP_STORE && acc[o.a].is_store != 1)
      return fail(TSB_ERR_INVALID, "tsb_elementwise: op %d stores to a load access", k);
    if (o.opcode != TSB_OP_STORE && (o.dst < 0 || o.dst >= TSB_NUM_REGS))
      return fail(TSB_ERR_INVALID, "tsb_elementwise: op %d register %d out of range", k, o.dst);
    const int regs[3] = {is_mem || o.opcode == TSB_OP_CONST ? 0 : o.a,
                         o.opcode == TSB_OP_LOAD || o.opcode == TSB_OP_CONST ? 0 : o.b,
                         (o.opcode == TSB_OP_SELECT || o.opcode == TSB_OP_FMA) ? o.c : 0};
    for (int r = 0; r < 3; ++r)
      if (regs[r] < 0 || regs[r] >= TSB_NUM_REGS)
        return fail(TSB_ERR_INVALID, "tsb_elementwise: op %d register %d out of range", k, regs[r]);
  }
  P.n_acc = n_acc;
  P.n_ops = n_ops;
  for (int k = 0; k < 3; ++k) P.grid[k] = grid[k] > 0 ? grid[k] : 1;
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
    f.vec_ok = d.kind < 2 && ((uintptr_t)d.base % (4ull * d.esize)) == 0 && d.off0 % 4 == 0;
  }
  memcpy(F.ops, P.ops, sizeof(tsb_op) * P.n_ops);
  F.n_acc = P.n_acc;
  F.n_ops = P.n_ops;
  F.g_lo = P.pid_lo * B;
  F.g_hi = P.pid_hi * B;
  return true;
}

static bool is_fast_binary(const tsb_access *acc, const tsb_op *ops, int n_ops) {
  if (n_ops != 4) return false;
  if (ops[0].opcode != TSB_OP_LOAD || ops[1].opcode != TSB_OP_LOAD || ops[3].opcode != TSB_OP_STORE)
    return false;
  const int o = ops[2].opcode;
  if (o < TSB_OP_ADDF || o > TSB_OP_MINIMUMF || ops[2].type != TSB_F32) return false;
  if (ops[2].a != ops[0].dst || ops[2].b != ops[1].dst || ops[3].b != ops[2].dst) return false;
  if (ops[0].dst == ops[1].dst) return false;
  return acc[ops[0].a].dtype == TSB_F32 && acc[ops[1].a].dtype == TSB_F32 &&
         acc[ops[3].a].dtype == TSB_F32;
}

}  // namespace tsb

using namespace tsb;

extern "C" int tsb_elementwise(const tsb_access *acc, int n_acc, const tsb_op *ops, int n_ops,
                               const int32_t grid[3], int64_t pid_lo, int64_t pid_hi, void *stream) {
  static thread_local EwParams P;
  int vec = 1;
  int rc = build_params(acc, n_acc, ops, n_ops, grid, pid_lo, pid_hi, P, vec);
  if (rc != TSB_OK) return rc;
  const long long n_prog = pid_hi - pid_lo;
  if (n_prog == 0) return TSB_OK;
  const int items = P.lanes / vec;
  int threads = items >= 256 ? 256 : (items >= 128 ? 128 : (items >= 64 ? 64 : 32));
  const long long max_ctas = (long long)sm_count() * (2048 / threads) * 4;
  cudaStream_t s = (cudaStream_t)stream;
  static thread_local FlatParams F;
  if (build_flat(P, vec, F)) {
    const long long n_vec = (F.g_hi - F.g_lo) / 4;
    const bool fast = is_fast_binary(acc, ops, n_ops);
    const long long per_cta = 256ll * (fast ? FLAT_UNROLL : 1);
    long long ctas = (n_vec + per_cta - 1) / per_cta;
    const long long cap = (long long)sm_count() * 8 * 4;
    if (ctas > cap) ctas = cap;
    if (fast) ew_flat_binary_f32_kernel<<<(unsigned)ctas, 256, 0, s>>>(F);
    else ew_flat_vm_kernel<<<(unsigned)ctas, 256, 0, s>>>(F);
    TSB_LAUNCH_OK("ew_flat_kernel");
    return TSB_OK;
  }
  if (is_fast_binary(acc, ops, n_ops)) {
    long long ctas = (n_prog + 1) / 2;
    if (ctas > max_ctas) ctas = max_ctas;
    if (vec == 4) ew_binary_f32_kernel<4><<<(unsigned)ctas, threads, 0, s>>>(P);
    else ew_binary_f32_kernel<1><<<(unsigned)ctas, threads, 0, s>>>(P);
    TSB_LAUNCH_OK("ew_binary_f32_kernel");
    return TSB_OK;
  }
  long long ctas = n_prog < max_ctas ? n_prog : max_ctas;
  if (vec == 4) ew_vm_kernel<4><<<(unsigned)ctas, threads, 0, s>>>(P);
  else ew_vm_kernel<1><<<(unsigned)ctas, threads, 0, s>>>(P);
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
