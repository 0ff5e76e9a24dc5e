// Shared pieces of the structured-access engine: the device form of an access, the 32-bit
// register representation and its arithmetic, per-program access state, and lane-vector
// loads/stores.  Used by the elementwise kernels and by the block-program kernel.
#pragma once
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
  long long off_loop[TSB_MAX_LOOPS];        // block programs: advance per iteration of loop slot l
  long long mstart_loop[3][TSB_MAX_LOOPS];
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


// ---- register representation -------------------------------------------------
// Every VM lane is 32 bits: f32 bits for all float types (f16/bf16 values are
// held exactly widened and re-rounded after each op), sign/zero-extended ints.

// raw element bits (zero-extended) <-> register representation, for VEC lanes with ONE switch on
// the element type (the conversions stay in registers; nothing is punned through memory)
template <int VEC>
__device__ __forceinline__ void raw_to_reg(int dt, unsigned (&x)[VEC]) {
  switch (dt) {
    case TSB_F16:
#pragma unroll
      for (int k = 0; k < VEC; ++k) x[k] = __float_as_uint(__half2float(__ushort_as_half((unsigned short)x[k])));
      break;
    case TSB_BF16:
#pragma unroll
      for (int k = 0; k < VEC; ++k) x[k] = x[k] << 16;
      break;
    case TSB_I16:
#pragma unroll
      for (int k = 0; k < VEC; ++k) x[k] = (unsigned)(int)(short)x[k];
      break;
    case TSB_I8:
#pragma unroll
      for (int k = 0; k < VEC; ++k) x[k] = (unsigned)(int)(signed char)x[k];
      break;
    default: break;  // 32-bit types and unsigned narrow types are already in place
  }
}
template <int VEC>
__device__ __forceinline__ void reg_to_raw(int dt, unsigned (&x)[VEC]) {
  switch (dt) {
    case TSB_F16:
#pragma unroll
      for (int k = 0; k < VEC; ++k) x[k] = __half_as_ushort(__float2half_rn(__uint_as_float(x[k])));
      break;
    case TSB_BF16:
#pragma unroll
      for (int k = 0; k < VEC; ++k) x[k] = __bfloat16_as_ushort(__float2bfloat16_rn(__uint_as_float(x[k])));
      break;
    case TSB_I16: case TSB_U16:
#pragma unroll
      for (int k = 0; k < VEC; ++k) x[k] &= 0xffffu;
      break;
    case TSB_I8: case TSB_U8:
#pragma unroll
      for (int k = 0; k < VEC; ++k) x[k] &= 0xffu;
      break;
    case TSB_I1:
#pragma unroll
      for (int k = 0; k < VEC; ++k) x[k] &= 1u;
      break;
    default: break;
  }
}
// 64-bit integers (index tensors) are held as their low 32 bits and stored sign-extended
__device__ __forceinline__ unsigned ld_raw(const char *p, int esize) {
  if (esize == 8) return (unsigned)*reinterpret_cast<const unsigned long long *>(p);
  if (esize == 4) return *reinterpret_cast<const unsigned *>(p);
  if (esize == 2) return *reinterpret_cast<const unsigned short *>(p);
  return *reinterpret_cast<const unsigned char *>(p);
}
__device__ __forceinline__ void st_raw(char *p, int esize, unsigned v) {
  if (esize == 8) *reinterpret_cast<long long *>(p) = (long long)(int)v;
  else if (esize == 4) *reinterpret_cast<unsigned *>(p) = v;
  else if (esize == 2) *reinterpret_cast<unsigned short *>(p) = (unsigned short)v;
  else *reinterpret_cast<unsigned char *>(p) = (unsigned char)v;
}
__device__ __forceinline__ unsigned ld_elem(const char *p, int dt) {
  unsigned x[1] = {ld_raw(p, dtype_size(dt))};
  raw_to_reg<1>(dt, x);
  return x[0];
}
__device__ __forceinline__ void st_elem(char *p, int dt, unsigned v) {
  unsigned x[1] = {v};
  reg_to_raw<1>(dt, x);
  st_raw(p, dtype_size(dt), x[0]);
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

// program_state inside loops: iteration it[l] of loop slot l shifts the offset and the mask starts
__device__ __forceinline__ void program_state_loops(const DAcc &A, const int size[3], long long px, long long py,
                                                    long long pz, const int it[TSB_MAX_LOOPS], ProgState &s) {
  long long extra = 0, mextra[3] = {0, 0, 0};
#pragma unroll
  for (int l = 0; l < TSB_MAX_LOOPS; ++l) {
    extra += A.off_loop[l] * it[l];
#pragma unroll
    for (int d = 0; d < 3; ++d) mextra[d] += A.mstart_loop[d][l] * it[l];
  }
  s.off = A.off0 + A.off_pid[0] * px + A.off_pid[1] * py + A.off_pid[2] * pz + extra;
  for (int w = 0; w < A.n_wrap; ++w)
    s.woff[w] = A.wrap[w].off0 + A.wrap[w].off_pid[0] * px + A.wrap[w].off_pid[1] * py + A.wrap[w].off_pid[2] * pz;
#pragma unroll
  for (int d = 0; d < 3; ++d) {
    int dim = size[d];
    if (A.masked & (1 << d)) {
      long long st = A.mstart0[d] + A.mstart_pid[d][0] * px + A.mstart_pid[d][1] * py +
                     A.mstart_pid[d][2] * pz + mextra[d];
      long long en = st + size[d];
      long long m = en < A.bound[d] ? en : A.bound[d];
      m = m > st ? m : st;
      dim = (int)(m - st);
    }
    s.dim[d] = dim;
  }
}

// Plain (coherent) loads: a later loop iteration, or a later op of the same body, may read what an
// earlier one stored.
template <int VEC>
__device__ __forceinline__ void load_vec(const DAcc &A, const ProgState &s, int i0, int i1, int i2,
                                         unsigned (&out)[VEC]) {
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
      uint4 v = *reinterpret_cast<const uint4 *>(p);
      out[0] = v.x; out[1 % VEC] = v.y; out[2 % VEC] = v.z; out[3 % VEC] = v.w;
    } else if (A.esize == 2) {
      uint2 v = *reinterpret_cast<const uint2 *>(p);
      out[0] = v.x & 0xffffu; out[1 % VEC] = v.x >> 16; out[2 % VEC] = v.y & 0xffffu; out[3 % VEC] = v.y >> 16;
      raw_to_reg<VEC>(A.dtype, out);
    } else {
      unsigned v = *reinterpret_cast<const unsigned *>(p);
#pragma unroll
      for (int k = 0; k < VEC; ++k) out[k] = (v >> (8 * k)) & 0xffu;
      raw_to_reg<VEC>(A.dtype, out);
    }
    return;
  }
  bool okk[VEC];
#pragma unroll
  for (int k = 0; k < VEC; ++k) {
    okk[k] = outer && (i2 + k) < s.dim[2];
    out[k] = okk[k] ? ld_raw(A.base + (e + k * A.stride[2]) * A.esize, A.esize) : 0u;
  }
  raw_to_reg<VEC>(A.dtype, out);
#pragma unroll
  for (int k = 0; k < VEC; ++k)
    if (!okk[k]) out[k] = fill;
}

template <int VEC>
__device__ __forceinline__ void store_vec(const DAcc &A, const ProgState &s, int i0, int i1, int i2,
                                          const unsigned (&in)[VEC]) {
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
      unsigned h[VEC];
#pragma unroll
      for (int k = 0; k < VEC; ++k) h[k] = in[k];
      reg_to_raw<VEC>(A.dtype, h);
      *reinterpret_cast<uint2 *>(p) = make_uint2(h[0] | (h[1 % VEC] << 16), h[2 % VEC] | (h[3 % VEC] << 16));
    } else {
      unsigned h[VEC];
#pragma unroll
      for (int k = 0; k < VEC; ++k) h[k] = in[k];
      reg_to_raw<VEC>(A.dtype, h);
      unsigned v = 0;
#pragma unroll
      for (int k = 0; k < VEC; ++k) v |= h[k] << (8 * k);
      *reinterpret_cast<unsigned *>(p) = v;
    }
    return;
  }
  unsigned h[VEC];
#pragma unroll
  for (int k = 0; k < VEC; ++k) h[k] = in[k];
  reg_to_raw<VEC>(A.dtype, h);
#pragma unroll
  for (int k = 0; k < VEC; ++k)
    if (i2 + k < s.dim[2]) st_raw(A.base + (e + k * A.stride[2]) * A.esize, A.esize, h[k]);
}


// Data-dependent accesses (gather / scatter): lane k of the vector reads or writes element
//   structured address + (int)index[k]        (when has_index)
// and takes part only if the structured mask admits it and mask[k] & 1 (when has_mask).
// One scalar access per lane; lanes of a warp that address neighbouring elements still coalesce.
template <int VEC>
__device__ __forceinline__ void load_vec_indirect(const DAcc &A, const ProgState &s, int i0, int i1, int i2,
                                                  bool has_index, bool has_mask, const unsigned (&index)[VEC],
                                                  const unsigned (&mask)[VEC], unsigned (&out)[VEC]) {
  const bool outer = i0 < s.dim[0] && i1 < s.dim[1];
  const long long e = s.off + i0 * A.stride[0] + i1 * A.stride[1] + i2 * A.stride[2];
  const unsigned fill = A.has_other ? A.other : 0u;
  if (VEC == 4 && A.kind == 0 && !A.n_wrap && A.stride[2] == 1 && A.esize >= 2 && A.esize <= 4 && outer &&
      i2 + VEC <= s.dim[2]) {
    // row gather: the four lanes of the vector share one index (the index varies along another
    // dim) and are all admitted: one 16-byte (8-byte) access when the row start is aligned
    const bool same = !has_index || (index[0] == index[1 % VEC] && index[0] == index[2 % VEC] && index[0] == index[3 % VEC]);
    const bool all = !has_mask || ((mask[0] & mask[1 % VEC] & mask[2 % VEC] & mask[3 % VEC]) & 1u);
    const char *p = A.base + (e + (has_index ? (long long)(int)index[0] : 0ll)) * A.esize;
    if (same && all && ((uintptr_t)p % (4u * A.esize)) == 0) {
      if (A.esize == 4) {
        const uint4 v = *reinterpret_cast<const uint4 *>(p);
        out[0] = v.x; out[1 % VEC] = v.y; out[2 % VEC] = v.z; out[3 % VEC] = v.w;
      } else {
        const uint2 v = *reinterpret_cast<const uint2 *>(p);
        out[0] = v.x & 0xffffu; out[1 % VEC] = v.x >> 16; out[2 % VEC] = v.y & 0xffffu; out[3 % VEC] = v.y >> 16;
      }
      raw_to_reg<VEC>(A.dtype, out);
      return;
    }
  }
#pragma unroll
  for (int k = 0; k < VEC; ++k) {
    bool ok = outer && (i2 + k) < s.dim[2];
    if (has_mask) ok = ok && (mask[k] & 1u);
    long long ek = e + k * A.stride[2];
    if (A.n_wrap) ek += wrap_addend(A, s, i0, i1, i2 + k);
    if (has_index) ek += (long long)(int)index[k];
    out[k] = A.kind == 2 ? (ok ? 1u : 0u) : (A.kind == 3 ? (unsigned)ek : (ok ? ld_elem(A.base + ek * A.esize, A.dtype) : fill));
  }
}

template <int VEC>
__device__ __forceinline__ void store_vec_indirect(const DAcc &A, const ProgState &s, int i0, int i1, int i2,
                                                   bool has_index, bool has_mask, const unsigned (&index)[VEC],
                                                   const unsigned (&mask)[VEC], const unsigned (&in)[VEC]) {
  if (!(i0 < s.dim[0] && i1 < s.dim[1])) return;
  const long long e = s.off + i0 * A.stride[0] + i1 * A.stride[1] + i2 * A.stride[2];
  if (VEC == 4 && !A.n_wrap && A.stride[2] == 1 && A.esize >= 2 && A.esize <= 4 && i2 + VEC <= s.dim[2]) {
    // row scatter: see load_vec_indirect
    const bool same = !has_index || (index[0] == index[1 % VEC] && index[0] == index[2 % VEC] && index[0] == index[3 % VEC]);
    const bool all = !has_mask || ((mask[0] & mask[1 % VEC] & mask[2 % VEC] & mask[3 % VEC]) & 1u);
    char *p = A.base + (e + (has_index ? (long long)(int)index[0] : 0ll)) * A.esize;
    if (same && all && ((uintptr_t)p % (4u * A.esize)) == 0) {
      unsigned h[VEC];
#pragma unroll
      for (int k = 0; k < VEC; ++k) h[k] = in[k];
      reg_to_raw<VEC>(A.dtype, h);
      if (A.esize == 4) *reinterpret_cast<uint4 *>(p) = make_uint4(h[0], h[1 % VEC], h[2 % VEC], h[3 % VEC]);
      else *reinterpret_cast<uint2 *>(p) = make_uint2(h[0] | (h[1 % VEC] << 16), h[2 % VEC] | (h[3 % VEC] << 16));
      return;
    }
  }
#pragma unroll
  for (int k = 0; k < VEC; ++k) {
    bool ok = (i2 + k) < s.dim[2];
    if (has_mask) ok = ok && (mask[k] & 1u);
    if (!ok) continue;
    long long ek = e + k * A.stride[2];
    if (A.n_wrap) ek += wrap_addend(A, s, i0, i1, i2 + k);
    if (has_index) ek += (long long)(int)index[k];
    st_elem(A.base + ek * A.esize, A.dtype, in[k]);
  }
}

// ---- combiners of reductions and scans --------------------------------------------
__device__ __forceinline__ unsigned combine(int comb, int type, unsigned a, unsigned b) {
  if (comb >= TSB_OP_ADDF && comb < TSB_OP_EXP)
    return __float_as_uint(round_to(binf(comb, __uint_as_float(a), __uint_as_float(b)), type));
  return wrap_to(bini(comb, a, b), type);
}
// identity of the combiner (what the reference initialises the accumulator with,
// ConversionPatterns.hpp:1227-1278)
__device__ __forceinline__ unsigned combine_identity(int comb) {
  switch (comb) {
    case TSB_OP_ADDF: return 0u;
    case TSB_OP_MULF: return 0x3f800000u;
    case TSB_OP_MAXNUMF: case TSB_OP_MAXIMUMF: return 0xff800000u;
    case TSB_OP_MINNUMF: case TSB_OP_MINIMUMF: return 0x7f800000u;
    case TSB_OP_MULI: return 1u;
    case TSB_OP_ANDI: return 0xffffffffu;
    case TSB_OP_MAXSI: return 0x80000000u;
    case TSB_OP_MINSI: return 0x7fffffffu;
    case TSB_OP_MINUI: return 0xffffffffu;
  }
  return 0u;  // addi, ori, xori, maxui
}

// ---- lean accessors ------------------------------------------------------------
// The common case of an access (memory load or store, no wrap terms, contiguous innermost dim with
// aligned 4-lane vectors, in-block offsets that fit 32 bits) in 32 bytes, so that a kernel can keep
// it in shared memory and address a whole-vector sub-item with a handful of 32-bit instructions.
// A body whose accesses are all of this kind runs a kernel variant that holds only these paths.
struct LeanAcc {
  char *base;
  int s0, s1;      // element strides of dims 0 and 1 (dim 2 has stride 1)
  unsigned other;  // fill value in register representation (0 when the access has none)
  unsigned char esize, dtype, fast, pad_;
  unsigned pad2_[2];
};
static_assert(sizeof(LeanAcc) == 32, "LeanAcc is read as two 16-byte words");

__host__ __device__ inline bool lean_ok(const DAcc &A, const int size[3]) {
  const long long a0 = A.stride[0] < 0 ? -A.stride[0] : A.stride[0];
  const long long a1 = A.stride[1] < 0 ? -A.stride[1] : A.stride[1];
  const bool fits = a0 < (1ll << 31) && a1 < (1ll << 31) &&
                    (size[0] - 1) * a0 + (size[1] - 1) * a1 + size[2] < (1ll << 31);
  return A.kind < 2 && !A.n_wrap && A.vec_ok && A.esize <= 4 && fits;
}

__device__ __forceinline__ void make_lean(const DAcc &A, const int size[3], LeanAcc &L) {
  L.base = A.base;
  L.s0 = (int)A.stride[0];
  L.s1 = (int)A.stride[1];
  L.other = A.has_other ? A.other : 0u;
  L.esize = (unsigned char)A.esize;
  L.dtype = (unsigned char)A.dtype;
  L.fast = lean_ok(A, size) ? 1 : 0;
  L.pad_ = 0;
  L.pad2_[0] = L.pad2_[1] = 0u;
}

// All U sub-items of one load of a lean access (lean_ok).  Whole vectors inside the mask are one
// 16/8/4-byte access each; a ragged sub-item reads its admitted lanes one by one and the others
// take the fill value.
template <int U>
__device__ __forceinline__ void lean_load(const LeanAcc &L, const ProgState &S, const int (&c0)[U],
                                          const int (&c1)[U], const int (&c2)[U], unsigned (&out)[U][4]) {
  const int d0 = S.dim[0], d1 = S.dim[1], d2 = S.dim[2];
  const int es = L.esize;
  const char *p = L.base + S.off * es;
  bool ragged = false;
  // raw bits first: one word per lane for 4- and 1-byte elements, two packed words (out[u][0..1])
  // for 2-byte elements
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const bool outer = c0[u] < d0 && c1[u] < d1;
    const char *q = p + (long long)(c0[u] * L.s0 + c1[u] * L.s1 + c2[u]) * es;
    if (outer && c2[u] + 4 <= d2) {
      if (es == 4) {
        const uint4 v = *reinterpret_cast<const uint4 *>(q);
        out[u][0] = v.x; out[u][1] = v.y; out[u][2] = v.z; out[u][3] = v.w;
      } else if (es == 2) {
        const uint2 v = *reinterpret_cast<const uint2 *>(q);
        out[u][0] = v.x; out[u][1] = v.y;
      } else {
        const unsigned v = *reinterpret_cast<const unsigned *>(q);
#pragma unroll
        for (int k = 0; k < 4; ++k) out[u][k] = (v >> (8 * k)) & 0xffu;
      }
    } else {
      ragged = true;
      unsigned r[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) r[k] = (outer && c2[u] + k < d2) ? ld_raw(q + k * es, es) : 0u;
      if (es == 2) {
        out[u][0] = r[0] | (r[1] << 16); out[u][1] = r[2] | (r[3] << 16);
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) out[u][k] = r[k];
      }
    }
  }
  if (es == 2) {
    if (L.dtype == TSB_F16) {
#pragma unroll
      for (int u = 0; u < U; ++u) {  // two lanes per conversion
        const float2 f0 = __half22float2(*reinterpret_cast<const __half2 *>(&out[u][0]));
        const float2 f1 = __half22float2(*reinterpret_cast<const __half2 *>(&out[u][1]));
        out[u][0] = __float_as_uint(f0.x); out[u][1] = __float_as_uint(f0.y);
        out[u][2] = __float_as_uint(f1.x); out[u][3] = __float_as_uint(f1.y);
      }
    } else if (L.dtype == TSB_BF16) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const unsigned w0 = out[u][0], w1 = out[u][1];
        out[u][0] = w0 << 16; out[u][1] = w0 & 0xffff0000u; out[u][2] = w1 << 16; out[u][3] = w1 & 0xffff0000u;
      }
    } else {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const unsigned w0 = out[u][0], w1 = out[u][1];
        out[u][0] = w0 & 0xffffu; out[u][1] = w0 >> 16; out[u][2] = w1 & 0xffffu; out[u][3] = w1 >> 16;
        raw_to_reg<4>(L.dtype, out[u]);
      }
    }
  } else if (es == 1) {
#pragma unroll
    for (int u = 0; u < U; ++u) raw_to_reg<4>(L.dtype, out[u]);
  }
  if (ragged) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const bool outer = c0[u] < d0 && c1[u] < d1;
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (!(outer && c2[u] + k < d2)) out[u][k] = L.other;
    }
  }
}

template <int U>
__device__ __forceinline__ void lean_store(const LeanAcc &L, const ProgState &S, const int (&c0)[U],
                                           const int (&c1)[U], const int (&c2)[U], const unsigned (&in)[U][4]) {
  const int d0 = S.dim[0], d1 = S.dim[1], d2 = S.dim[2];
  const int es = L.esize;
  char *p = L.base + S.off * es;
  unsigned h[U][4];
#pragma unroll
  for (int u = 0; u < U; ++u)
#pragma unroll
    for (int k = 0; k < 4; ++k) h[u][k] = in[u][k];
  // 16-bit floats: two lanes per conversion, already packed (pk[u] holds the four lanes of sub-item u)
  uint2 pk[U];
  const bool packed16 = L.dtype == TSB_F16 || L.dtype == TSB_BF16;
  if (es != 4) {
    if (L.dtype == TSB_F16) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const __half2 lo = __floats2half2_rn(__uint_as_float(h[u][0]), __uint_as_float(h[u][1]));
        const __half2 hi = __floats2half2_rn(__uint_as_float(h[u][2]), __uint_as_float(h[u][3]));
        pk[u] = make_uint2(*reinterpret_cast<const unsigned *>(&lo), *reinterpret_cast<const unsigned *>(&hi));
      }
    } else if (L.dtype == TSB_BF16) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(__uint_as_float(h[u][0]), __uint_as_float(h[u][1]));
        const __nv_bfloat162 hi = __floats2bfloat162_rn(__uint_as_float(h[u][2]), __uint_as_float(h[u][3]));
        pk[u] = make_uint2(*reinterpret_cast<const unsigned *>(&lo), *reinterpret_cast<const unsigned *>(&hi));
      }
    } else {
#pragma unroll
      for (int u = 0; u < U; ++u) reg_to_raw<4>(L.dtype, h[u]);
    }
  }
#pragma unroll
  for (int u = 0; u < U; ++u) {
    if (!(c0[u] < d0 && c1[u] < d1)) continue;
    char *q = p + (long long)(c0[u] * L.s0 + c1[u] * L.s1 + c2[u]) * es;
    if (packed16 && c2[u] + 4 > d2) {  // ragged: back to one raw value per lane
      h[u][0] = pk[u].x & 0xffffu; h[u][1] = pk[u].x >> 16; h[u][2] = pk[u].y & 0xffffu; h[u][3] = pk[u].y >> 16;
    }
    if (c2[u] + 4 <= d2) {
      if (es == 4) *reinterpret_cast<uint4 *>(q) = make_uint4(h[u][0], h[u][1], h[u][2], h[u][3]);
      else if (packed16) *reinterpret_cast<uint2 *>(q) = pk[u];
      else if (es == 2) *reinterpret_cast<uint2 *>(q) = make_uint2(h[u][0] | (h[u][1] << 16), h[u][2] | (h[u][3] << 16));
      else *reinterpret_cast<unsigned *>(q) = h[u][0] | (h[u][1] << 8) | (h[u][2] << 16) | (h[u][3] << 24);
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (c2[u] + k < d2) st_raw(q + k * es, es, h[u][k]);
    }
  }
}

// One ALU op on one lane with the opcode known at compile time: the per-op switch is taken
// once per thread (see TSB_ALU_OPCODES), not once per lane.  ROUND = false leaves a float result
// unrounded (the caller rounds all lanes of the op at once when the op's type is 16-bit).
template <int OPC, bool ROUND = true>
__device__ __forceinline__ unsigned alu_op(const tsb_op &op, unsigned a, unsigned b, unsigned c) {
  if constexpr (OPC == TSB_OP_MOV || OPC == TSB_OP_BITCAST) return a;  // 32-bit <-> 32-bit bitcasts keep their bits
  else if constexpr (OPC >= TSB_OP_ADDF && OPC < TSB_OP_EXP) {
    const float r = binf(OPC, __uint_as_float(a), __uint_as_float(b));
    return __float_as_uint(ROUND ? round_to(r, op.type) : r);
  } else if constexpr (OPC >= TSB_OP_EXP && OPC < TSB_OP_ADDI) {
    const float r = unf(OPC, __uint_as_float(a));
    return __float_as_uint(ROUND ? round_to(r, op.type) : r);
  } else if constexpr (OPC == TSB_OP_ABSI) return wrap_to((unsigned)abs((int)a), op.type);
  else if constexpr (OPC >= TSB_OP_ADDI && OPC < TSB_OP_CMPF) return wrap_to(bini(OPC, a, b), op.type);
  else if constexpr (OPC == TSB_OP_CMPF) return cmpf_(op.imm, __uint_as_float(a), __uint_as_float(b));
  else if constexpr (OPC == TSB_OP_CMPI) return cmpi_(op.imm, a, b);
  else if constexpr (OPC == TSB_OP_SELECT) return (a & 1u) ? b : c;
  else if constexpr (OPC == TSB_OP_CAST) return cast_(a, (int)op.imm, op.type, op.imm2);
  else if constexpr (OPC == TSB_OP_FMA) {
    const float r = fmaf(__uint_as_float(a), __uint_as_float(b), __uint_as_float(c));
    return __float_as_uint(ROUND ? round_to(r, op.type) : r);
  } else return 0u;
}
// float-result ops whose result must be re-rounded when the op's type is f16 / bf16
template <int OPC>
__device__ __forceinline__ constexpr bool alu_rounds() {
  return (OPC >= TSB_OP_ADDF && OPC < TSB_OP_ADDI) || OPC == TSB_OP_FMA;
}

// Operands an ALU opcode reads (1, 2 or 3), known at compile time.
template <int OPC>
__device__ __forceinline__ constexpr int alu_arity() {
  if (OPC == TSB_OP_SELECT || OPC == TSB_OP_FMA) return 3;
  if ((OPC >= TSB_OP_EXP && OPC < TSB_OP_ADDI) || OPC == TSB_OP_ABSI || OPC == TSB_OP_CAST ||
      OPC == TSB_OP_BITCAST || OPC == TSB_OP_MOV)
    return 1;
  return 2;
}

// X(opcode) for every ALU opcode
#define TSB_ALU_OPCODES(X)                                                                          \
  X(TSB_OP_MOV) X(TSB_OP_BITCAST) X(TSB_OP_ADDF) X(TSB_OP_SUBF) X(TSB_OP_MULF) X(TSB_OP_DIVF)        \
  X(TSB_OP_MAXNUMF) X(TSB_OP_MINNUMF) X(TSB_OP_MAXIMUMF) X(TSB_OP_MINIMUMF) X(TSB_OP_REMF)          \
  X(TSB_OP_EXP) X(TSB_OP_EXP2) X(TSB_OP_LOG) X(TSB_OP_LOG2) X(TSB_OP_SQRT) X(TSB_OP_RSQRT)          \
  X(TSB_OP_SIN) X(TSB_OP_COS) X(TSB_OP_TANH) X(TSB_OP_ERF) X(TSB_OP_ABSF) X(TSB_OP_NEGF)            \
  X(TSB_OP_FLOOR) X(TSB_OP_CEIL) X(TSB_OP_ADDI) X(TSB_OP_SUBI) X(TSB_OP_MULI) X(TSB_OP_DIVSI)       \
  X(TSB_OP_REMSI) X(TSB_OP_DIVUI) X(TSB_OP_REMUI) X(TSB_OP_MINSI) X(TSB_OP_MAXSI) X(TSB_OP_MINUI)   \
  X(TSB_OP_MAXUI) X(TSB_OP_ANDI) X(TSB_OP_ORI) X(TSB_OP_XORI) X(TSB_OP_SHLI) X(TSB_OP_SHRSI)        \
  X(TSB_OP_SHRUI) X(TSB_OP_ABSI) X(TSB_OP_CMPF) X(TSB_OP_CMPI) X(TSB_OP_SELECT) X(TSB_OP_CAST)      \
  X(TSB_OP_FMA)

// Program id of the k-th program a kernel processes.  order[] lists the grid axes from fastest to
// slowest varying; {0,1,2} is the linearisation of the launch (x fastest).  Programs are
// independent, so when a launch covers the whole grid the kernels may walk them with the axis
// of smallest address step fastest, which keeps concurrently running CTAs on neighbouring memory.
__device__ __forceinline__ void split_pid(const int grid[3], const int order[3], long long k, long long &px,
                                          long long &py, long long &pz) {
  if (grid[1] == 1 && grid[2] == 1) {
    px = k; py = 0; pz = 0;
    return;
  }
  long long p[3];
  const unsigned long long g0 = (unsigned long long)grid[order[0]], g1 = (unsigned long long)grid[order[1]];
  const unsigned long long q = (unsigned long long)k / g0;
  p[order[0]] = (long long)((unsigned long long)k - q * g0);
  p[order[1]] = (long long)(q % g1);
  p[order[2]] = (long long)(q / g1);
  px = p[0]; py = p[1]; pz = p[2];
}


inline unsigned other_to_reg(uint64_t bits, int dt) {
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

inline int ilog2_exact(long long v) {
  int l = 0;
  while ((1ll << l) < v) ++l;
  return ((1ll << l) == v) ? l : -1;
}


// Order in which a kernel walks the programs of a launch: natural unless the launch covers the
// whole grid, in which case the axis along which the first store moves least goes fastest.
inline void choose_program_order(const DAcc *acc, int n_acc, const int grid[3], long long pid_lo,
                                 long long pid_hi, int order[3]) {
  order[0] = 0; order[1] = 1; order[2] = 2;
  const long long total = (long long)grid[0] * grid[1] * grid[2];
  if (pid_lo != 0 || pid_hi != total) return;
  const DAcc *st = nullptr;
  for (int a = 0; a < n_acc && !st; ++a)
    if (acc[a].kind == 1) st = &acc[a];
  if (!st) return;
  auto step = [&](int a) {
    long long v = st->off_pid[a] < 0 ? -st->off_pid[a] : st->off_pid[a];
    return grid[a] > 1 ? v : 0x7fffffffffffffffll;  // unit axes last
  };
  for (int i = 0; i < 3; ++i)
    for (int j = i + 1; j < 3; ++j)
      if (step(order[j]) < step(order[i])) { int t = order[i]; order[i] = order[j]; order[j] = t; }
}

// Device form of one access of a launch: validates `s` and pads it to the rank-3 iteration space
// `size` (leading unit dims). `vec` is the lane-vector width the kernel will use (4 or 1).
inline int convert_access(const tsb_access *acc, int a, int rank, const int size[3], const int32_t grid[3],
                          int vec, DAcc &d) {
  const tsb_access &s = acc[a];
  if (s.rank != rank) return fail(TSB_ERR_INVALID, "tsb_elementwise: access %d has rank %d, expected %d", a, s.rank, rank);
  const int es = dtype_size(s.dtype);
  if (es == 0 || s.dtype == TSB_F64)
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
  for (int l = 0; l < TSB_MAX_LOOPS; ++l) d.off_loop[l] = s.offset_loop[l];
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
      for (int l = 0; l < TSB_MAX_LOOPS; ++l) d.mstart_loop[o][l] = s.mask_start_loop[k][l];
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
  bool ok = vec == 4 && es <= 4 && d.stride[2] == 1 && ((uintptr_t)d.base % vb) == 0 && d.off0 % 4 == 0;
  for (int k = 0; k < 3; ++k) ok = ok && (grid[k] <= 1 || d.off_pid[k] % 4 == 0);
  for (int l = 0; l < TSB_MAX_LOOPS; ++l) ok = ok && d.off_loop[l] % 4 == 0;
  ok = ok && (size[1] <= 1 || d.stride[1] % 4 == 0) && (size[0] <= 1 || d.stride[0] % 4 == 0);
  ok = ok && !d.wrap_inner && !wrap_unaligned;
  d.vec_ok = ok ? 1 : 0;
  return TSB_OK;
}

}  // namespace tsb
