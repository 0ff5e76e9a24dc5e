// The register VM shared by the structured-access kernels: a pass over the op list for the
// lane-vectors of one thread, with the loads and stores supplied by the kernel.
#pragma once
#include "tsb_ew.cuh"

namespace tsb {

// ---- general body: a small register VM ----------------------------------------
// One pass over the op list for VEC lanes; `ld(access, regs)` and `st(access, regs)`
// are supplied by the kernel (blocked or flat addressing).
// The VM's registers live in shared memory: register r of thread t is the VEC consecutive
// words starting at (r*blockDim + t)*VEC, so one 16-byte access per register and thread (VEC = 4)
// and consecutive threads touch consecutive 16-byte slots (conflict-free).  A register file
// indexed by run-time register numbers cannot live in hardware registers; kept as a per-thread
// local array it overflowed L1.  The kernels are bound by instruction issue, so the opcode
// switch is taken once per op and thread, with operand count known inside each case.
// Each thread carries U independent lane-vectors ("sub-items") through the op list, so the cost
// of decoding an op is shared by U*VEC lanes and U loads per access are in flight per thread.
template <int VEC, int U>
struct VmRegs {
  unsigned *base;  // shared memory
  int nt, t;
  __device__ __forceinline__ unsigned *slot(int reg, int u) const {
    return base + ((reg * U + u) * nt + t) * VEC;  // at most 256 KB of shared memory: 32-bit arithmetic
  }
  __device__ __forceinline__ void get(int reg, int u, unsigned (&v)[VEC]) const {
    const unsigned *p = slot(reg, u);
    if (VEC == 4) {
      const uint4 q = *reinterpret_cast<const uint4 *>(p);
      v[0] = q.x; v[1 % VEC] = q.y; v[2 % VEC] = q.z; v[3 % VEC] = q.w;
    } else {
#pragma unroll
      for (int k = 0; k < VEC; ++k) v[k] = p[k];
    }
  }
  __device__ __forceinline__ void put(int reg, int u, const unsigned (&v)[VEC]) const {
    unsigned *p = slot(reg, u);
    if (VEC == 4) {
      *reinterpret_cast<uint4 *>(p) = make_uint4(v[0], v[1 % VEC], v[2 % VEC], v[3 % VEC]);
    } else {
#pragma unroll
      for (int k = 0; k < VEC; ++k) p[k] = v[k];
    }
  }
};

// All sub-items of one operand: a shared-memory register, the accumulator (the previous op's
// result, held in hardware registers), or an immediate.  The source is decoded once per op.
template <int VEC, int U>
__device__ __forceinline__ void vm_fetch(const tsb_op &op, int which, const VmRegs<VEC, U> &R,
                                         const unsigned (&acc)[U][VEC], unsigned (&v)[U][VEC]) {
  if (which == TSB_REG_ACC) {
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int k = 0; k < VEC; ++k) v[u][k] = acc[u][k];
  } else if (which == TSB_REG_IMM) {
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int k = 0; k < VEC; ++k) v[u][k] = op.imm2;
  } else {
#pragma unroll
    for (int u = 0; u < U; ++u) R.get(which, u, v[u]);
  }
}

// One ALU op on all sub-items.  The result always lands in `acc`.  Fetching every operand into
// a register array of its own costs a move per lane and operand wherever the three sources
// (register file, accumulator, immediate) merge; the cheap unary and binary opcodes are therefore
// compiled once per combination of sources and compute straight from them.
// The direct forms are compiled for the cheap opcodes only (FORMS, alu_light): an expensive op
// gains little from them and its code would be repeated per form.
template <int OPC>
__device__ __forceinline__ constexpr bool alu_light() {
  return OPC == TSB_OP_MOV || OPC == TSB_OP_BITCAST || OPC == TSB_OP_ADDF || OPC == TSB_OP_SUBF ||
         OPC == TSB_OP_MULF || (OPC >= TSB_OP_MAXNUMF && OPC <= TSB_OP_MINIMUMF) || OPC == TSB_OP_ABSF ||
         OPC == TSB_OP_NEGF || OPC == TSB_OP_FLOOR || OPC == TSB_OP_CEIL || OPC == TSB_OP_ADDI ||
         OPC == TSB_OP_SUBI || OPC == TSB_OP_MULI || (OPC >= TSB_OP_MINSI && OPC <= TSB_OP_ABSI) ||
         OPC == TSB_OP_CMPF || OPC == TSB_OP_CMPI;
}

// Result handling shared by all forms: 16-bit float ops round once per op, then the optional
// write to the register file.
template <int OPC, int VEC, int U>
__device__ __forceinline__ void vm_alu_finish(const tsb_op &op, const VmRegs<VEC, U> &R, unsigned (&acc)[U][VEC]) {
  if (alu_rounds<OPC>() && op.type != TSB_F32) {  // one decision per op, not per lane
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int v = 0; v < VEC; ++v) acc[u][v] = __float_as_uint(round_to(__uint_as_float(acc[u][v]), op.type));
  }
  if (op.dst >= 0) {
#pragma unroll
    for (int u = 0; u < U; ++u) R.put(op.dst, u, acc[u]);
  }
}

// A unary or binary op whose operand sources are known at compile time
// (0 accumulator, 1 immediate, 2 register file): straight from the sources into the accumulator.
template <int OPC, int SA, int SB, int VEC, int U>
__device__ __forceinline__ void vm_alu_direct(const tsb_op &op, const VmRegs<VEC, U> &R, unsigned (&acc)[U][VEC]) {
  const unsigned imm = op.imm2;
#pragma unroll
  for (int u = 0; u < U; ++u) {
    unsigned x[VEC], y[VEC];
    if (SA == 2) R.get(op.a, u, x);
    if (SB == 2) R.get(op.b, u, y);
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      const unsigned xa = SA == 0 ? acc[u][v] : (SA == 1 ? imm : x[v]);
      const unsigned yb = SB == 0 ? acc[u][v] : (SB == 1 ? imm : (SB == 2 ? y[v] : 0u));
      acc[u][v] = alu_op<OPC, false>(op, xa, yb, 0u);
    }
  }
  // The forms of one opcode differ only in where the operands come from; the optimiser would
  // merge them back into one computation behind per-lane operand selects, which is the cost the
  // forms exist to avoid.  An empty asm statement per lane is not merged.
#pragma unroll
  for (int u = 0; u < U; ++u)
#pragma unroll
    for (int v = 0; v < VEC; ++v) asm volatile("" : "+r"(acc[u][v]));
  vm_alu_finish<OPC, VEC, U>(op, R, acc);
}

template <int OPC, int VEC, int U, bool FORMS>
__device__ __forceinline__ void vm_alu(const tsb_op &op, const VmRegs<VEC, U> &R, unsigned (&acc)[U][VEC]) {
  constexpr int AR = alu_arity<OPC>();
  if constexpr (FORMS && alu_light<OPC>() && AR <= 2) {
    const int sa = op.a == TSB_REG_ACC ? 0 : (op.a == TSB_REG_IMM ? 1 : 2);
    if constexpr (AR == 1) {
      if (sa == 0) vm_alu_direct<OPC, 0, 3, VEC, U>(op, R, acc);
      else if (sa == 2) vm_alu_direct<OPC, 2, 3, VEC, U>(op, R, acc);
      else vm_alu_direct<OPC, 1, 3, VEC, U>(op, R, acc);
    } else {
      const int sb = op.b == TSB_REG_ACC ? 0 : (op.b == TSB_REG_IMM ? 1 : 2);
      switch (sa * 3 + sb) {
        case 0: vm_alu_direct<OPC, 0, 0, VEC, U>(op, R, acc); break;
        case 1: vm_alu_direct<OPC, 0, 1, VEC, U>(op, R, acc); break;
        case 2: vm_alu_direct<OPC, 0, 2, VEC, U>(op, R, acc); break;
        case 3: vm_alu_direct<OPC, 1, 0, VEC, U>(op, R, acc); break;
        case 5: vm_alu_direct<OPC, 1, 2, VEC, U>(op, R, acc); break;
        case 6: vm_alu_direct<OPC, 2, 0, VEC, U>(op, R, acc); break;
        case 7: vm_alu_direct<OPC, 2, 1, VEC, U>(op, R, acc); break;
        case 8: vm_alu_direct<OPC, 2, 2, VEC, U>(op, R, acc); break;
        default: vm_alu_direct<OPC, 1, 1, VEC, U>(op, R, acc); break;
      }
    }
  } else {
    unsigned a[U][VEC], b[U][VEC], c[U][VEC];
    vm_fetch<VEC, U>(op, op.a, R, acc, a);
    if (AR >= 2) vm_fetch<VEC, U>(op, op.b, R, acc, b);
    if (AR >= 3) vm_fetch<VEC, U>(op, op.c, R, acc, c);
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int v = 0; v < VEC; ++v)
        acc[u][v] = alu_op<OPC, false>(op, a[u][v], AR >= 2 ? b[u][v] : 0u, AR >= 3 ? c[u][v] : 0u);
    vm_alu_finish<OPC, VEC, U>(op, R, acc);
  }
}

// ld(access, regs[U][VEC]) / st(access, regs[U][VEC]) move all sub-items of one access; inactive
// sub-items load zeros and store nothing
// ldx / stx (access, u, flags, index, mask, regs): sub-item u with a per-lane element index added to the address and / or a per-lane
// mask bit (flags MEM_INDEX, MEM_MASK): the data-dependent accesses of gather / scatter kernels.
// INDIRECT = false compiles the flagged forms out (the flat kernel never has them).
// FORMS: see vm_alu.
// red(op, regs): TSB_OP_REDUCE, every lane of regs := the fold (combiner op.imm) of regs over all
// lanes of the program; kernels whose threads do not know their program pass vm_no_reduce.
struct vm_no_reduce {
  template <int U, int VEC>
  __device__ __forceinline__ void operator()(const tsb_op &, unsigned (&)[U][VEC]) const {}
};

template <int VEC, int U, bool INDIRECT, bool FORMS, typename LoadFn, typename StoreFn, typename LoadXFn,
          typename StoreXFn, typename ReduceFn = vm_no_reduce>
__device__ __forceinline__ void vm_exec(const tsb_op *ops, int n_ops, const VmRegs<VEC, U> R, LoadFn ld, StoreFn st,
                                        LoadXFn ldx, StoreXFn stx, ReduceFn red = ReduceFn()) {
  unsigned acc[U][VEC];
#pragma unroll
  for (int u = 0; u < U; ++u)
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[u][v] = 0u;
  for (int k = 0; k < n_ops; ++k) {
    const tsb_op &op = ops[k];
    switch (op.opcode) {
      case TSB_OP_LOAD:
        if (INDIRECT && (op.imm & (MEM_INDEX | MEM_MASK))) {
          unsigned ix[U][VEC], mk[U][VEC];
          if (op.imm & MEM_INDEX) vm_fetch<VEC, U>(op, op.b, R, acc, ix);
          if (op.imm & MEM_MASK) vm_fetch<VEC, U>(op, op.c, R, acc, mk);
#pragma unroll
          for (int u = 0; u < U; ++u) ldx(op.a, u, op.imm, ix[u], mk[u], acc[u]);
        } else {
          ld(op.a, acc);  // all sub-items' loads are issued before the first use
        }
        if (op.dst >= 0) {
#pragma unroll
          for (int u = 0; u < U; ++u) R.put(op.dst, u, acc[u]);
        }
        break;
      case TSB_OP_STORE:
#pragma unroll
        {
          unsigned t[U][VEC];
          vm_fetch<VEC, U>(op, op.b, R, acc, t);
          if (INDIRECT && (op.imm & (MEM_INDEX | MEM_MASK))) {
            unsigned ix[U][VEC], mk[U][VEC];
            if (op.imm & MEM_INDEX) vm_fetch<VEC, U>(op, op.c, R, acc, ix);
            if (op.imm & MEM_MASK) vm_fetch<VEC, U>(op, op.dst, R, acc, mk);
#pragma unroll
            for (int u = 0; u < U; ++u) stx(op.a, u, op.imm, ix[u], mk[u], t[u]);
          } else {
            st(op.a, t);
          }
        }
        break;
      case TSB_OP_REDUCE:
        if (op.a != TSB_REG_ACC) {
          unsigned t[U][VEC];
          vm_fetch<VEC, U>(op, op.a, R, acc, t);
#pragma unroll
          for (int u = 0; u < U; ++u)
#pragma unroll
            for (int v = 0; v < VEC; ++v) acc[u][v] = t[u][v];
        }
        red(op, acc);
        if (op.dst >= 0) {
#pragma unroll
          for (int u = 0; u < U; ++u) R.put(op.dst, u, acc[u]);
        }
        break;
      case TSB_OP_CONST:
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
          for (int v = 0; v < VEC; ++v) acc[u][v] = op.imm;
          if (op.dst >= 0) R.put(op.dst, u, acc[u]);
        }
        break;
#define TSB_VM_CASE(O) \
  case O: vm_alu<O, VEC, U, FORMS>(op, R, acc); break;
        TSB_ALU_OPCODES(TSB_VM_CASE)
#undef TSB_VM_CASE
      default: break;
    }
  }
}

}  // namespace tsb
