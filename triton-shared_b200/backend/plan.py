"""Launch plans: map an analysed kernel (structured accesses + block dataflow graph)
onto one of the pre-built CUDA kernel families of libtsb200.so and its parameters.

Families (tried in this order):
  gemm         scf.for {2 masked block loads, tt.dot} + truncf + masked store      -> tsb_gemm
  layernorm    the three-loop LayerNorm forward of python/examples/test_layernorm.py -> tsb_layernorm_fwd
  softmax      masked row load, max, exp, sum, div, masked row store              -> tsb_softmax_rows
  reduce_rows  loop of masked 2-D block loads + sum(axis) + add, masked 1-D store  -> tsb_reduce_rows
  reduce_all   loop of masked 1-D loads + add, full sum, scalar store              -> tsb_reduce_all
  elementwise  any loop-free body of loads, elementwise ops and stores             -> tsb_elementwise
A kernel that fits none raises UnsupportedTTIR at compile time; nothing falls
back to another executor.

A plan is JSON-serialisable (it is the "binary" of the Triton compile pipeline)
and is evaluated against concrete arguments at launch.
"""
from __future__ import annotations

import ctypes
import json
import struct
from typing import Dict, List, Optional, Tuple

import numpy as np

from . import runtime as rt
from .structured import (Access, Analyzer, Kernel, Loop, Node, Poly, TData, TMask, float_from_key)
from .ttir import UnsupportedTTIR

# --------------------------------------------------------------------------
# small pattern matcher over the hash-consed block graph

_COMMUTATIVE = {"addf", "mulf", "maxnumf", "minnumf", "maximumf", "minimumf", "addi", "muli", "andi", "ori", "xori"}


def _is_ext(n: Node):
    return n.op == "cast" and n.attr("kind") in ("extf", "fp_to_fp") and n.dtype == "f32"


def _is_trunc(n: Node):
    return n.op == "cast" and n.attr("kind") in ("truncf", "fp_to_fp")


def const_value(n: Node) -> Optional[float]:
    """Float value of a constant node, looking through splat/broadcast."""
    while n.op in ("splat", "broadcast", "expand_dims"):
        n = n.args[0]
    if n.op == "const":
        return float_from_key(n.attr("value"))
    return None


def match(n: Node, pat, b: Dict[str, Node]) -> bool:
    """pat: ("$", name) | ("op", name, *pats) | ("ext", pat) | ("trunc", pat) | ("splat", pat)
    | ("const", value) | ("reduce", comb, axis|None, pat) | ("attrs", pat, {k: v})"""
    kind = pat[0]
    if kind == "$":
        if pat[1] in b:
            return b[pat[1]] is n
        b[pat[1]] = n
        return True
    if kind == "ext":
        return match(n.args[0], pat[1], b) if _is_ext(n) else match(n, pat[1], b)
    if kind == "trunc":
        return match(n.args[0], pat[1], b) if _is_trunc(n) else match(n, pat[1], b)
    if kind == "splat":
        if n.op in ("splat", "broadcast"):
            return match(n.args[0], pat, b) or match(n.args[0], pat[1], b)
        return False
    if kind == "const":
        v = const_value(n)
        return v is not None and (v == pat[1] or (v != v and pat[1] != pat[1]))
    if kind == "reduce":
        if n.op != "reduce" or n.attr("comb") != pat[1]:
            return False
        if pat[2] is not None and n.attr("axis") != pat[2]:
            return False
        return match(n.args[0], pat[3], b)
    if kind == "attrs":
        return all(n.attr(k) == v for k, v in pat[2].items()) and match(n, pat[1], b)
    if kind == "op":
        name, subs = pat[1], pat[2:]
        if n.op != name or len(n.args) != len(subs):
            return False
        trial = dict(b)
        if all(match(a, p, trial) for a, p in zip(n.args, subs)):
            b.update(trial)
            return True
        if name in _COMMUTATIVE and len(subs) == 2:
            trial = dict(b)
            if match(n.args[0], subs[1], trial) and match(n.args[1], subs[0], trial):
                b.update(trial)
                return True
        return False
    raise AssertionError(pat)


# --------------------------------------------------------------------------
# JSON encoding of plan parameters

def enc(o):
    if isinstance(o, Poly):
        return {"$poly": o.to_json()}
    if isinstance(o, dict):
        return {k: enc(v) for k, v in o.items()}
    if isinstance(o, (list, tuple)):
        return [enc(v) for v in o]
    return o


def dec(o):
    if isinstance(o, dict):
        if "$poly" in o:
            return Poly.from_json(o["$poly"])
        return {k: dec(v) for k, v in o.items()}
    if isinstance(o, list):
        return [dec(v) for v in o]
    return o


# --------------------------------------------------------------------------
# launch-time helpers



class LaunchEnv:
    """Concrete values of the symbols a plan's polynomials mention."""

    def __init__(self, scalars: Dict[int, int], grid):
        self.base = {("arg", i): int(v) for i, v in scalars.items()}
        for a in range(3):
            self.base[("np", a)] = int(grid[a])
        self.grid = tuple(int(g) for g in grid)

    def at(self, pid=(0, 0, 0), **its):
        e = dict(self.base)
        for a in range(3):
            e[("pid", a)] = pid[a]
        for k, v in its.items():
            e[("it", int(k[2:]))] = v
        return e

    def affine_pid(self, p: Poly, its=None) -> Tuple[int, List[int]]:
        """(value at pid 0, per-axis increments). The caller has checked affinity symbolically."""
        its = its or {}
        v0 = int(p.evaluate(self.at((0, 0, 0), **its)))
        inc = []
        for a in range(3):
            if self.grid[a] <= 1:
                inc.append(0)
                continue
            pid = [0, 0, 0]
            pid[a] = 1
            inc.append(int(p.evaluate(self.at(tuple(pid), **its))) - v0)
        return v0, inc

    def all_pids(self):
        """Environment with numpy arrays for every program of the grid, linearised x fastest."""
        gx, gy, gz = self.grid
        lin = np.arange(gx * gy * gz, dtype=np.int64)
        e = dict(self.base)
        e[("pid", 0)] = lin % gx
        e[("pid", 1)] = (lin // gx) % gy
        e[("pid", 2)] = lin // (gx * gy)
        return e


def is_affine_in_pid(p: Poly) -> bool:
    for m in p.terms:
        deg = 0
        for a in m:
            if a[0] == "pid":
                deg += 1
            elif a[0] == "fn" and (a[2].depends_on(("pid",)) or a[3].depends_on(("pid",))):
                return False
        if deg > 1:
            return False
    return True


def _is_affine_in_its(p: Poly) -> bool:
    """Every loop counter appears at most linearly, never multiplied by another counter or inside a function."""
    for m in p.terms:
        deg = 0
        for a in m:
            if a[0] == "it":
                deg += 1
            elif a[0] == "fn" and (a[2].depends_on(("it",)) or a[3].depends_on(("it",))):
                return False
        if deg > 1:
            return False
    return True


def _float_bits(v: float, elem: str) -> int:
    if elem == "f32":
        return struct.unpack("<I", struct.pack("<f", v))[0]
    if elem == "f16":
        return int(np.asarray([v], dtype=np.float16).view(np.uint16)[0])
    if elem == "bf16":
        u = struct.unpack("<I", struct.pack("<f", v))[0]
        if (u & 0x7fffffff) > 0x7f800000:
            return (u >> 16) | 0x40
        return ((u + 0x7fff + ((u >> 16) & 1)) >> 16) & 0xffff
    raise UnsupportedTTIR(f"fill value of type {elem}")


def other_bits(node: Optional[Node], elem: str) -> Optional[int]:
    """Bit pattern of a load's `other` when it is a compile-time constant."""
    if node is None:
        return None
    n = node
    while n.op in ("splat", "broadcast", "expand_dims"):
        n = n.args[0]
    if n.op == "const":
        return _float_bits(float_from_key(n.attr("value")), elem)
    if n.op == "sint" and n.attr("poly").is_const:
        return n.attr("poly").as_const & ((1 << (8 * rt.DTYPE_SIZE[elem])) - 1)
    if n.op == "index" and n.attr("offset").is_const and all(s.is_zero for s in n.attr("strides")):
        return n.attr("offset").as_const & ((1 << (8 * rt.DTYPE_SIZE[elem])) - 1)
    if n.op == "cast":
        # e.g. other=-1 written as an int and converted to the element type
        inner = other_bits(n.args[0], n.args[0].dtype)
        if inner is not None and n.args[0].dtype.startswith("i") and elem.startswith("i"):
            return inner & ((1 << (8 * rt.DTYPE_SIZE[elem])) - 1)
        if inner is not None and n.args[0].dtype.startswith("i") and elem in ("f32", "f16", "bf16"):
            bits = 8 * rt.DTYPE_SIZE[n.args[0].dtype]
            sv = inner - (1 << bits) if inner >= (1 << (bits - 1)) else inner
            return _float_bits(float(sv), elem)
    raise UnsupportedTTIR("masked load whose `other` is not a compile-time constant")


class Plan:
    family = "?"

    def __init__(self, name: str, params: dict):
        self.name = name
        self.p = params
        self._memo = {}

    def memo(self, args, grid, compute):
        """Launch parameters depend only on the scalar arguments and the grid: evaluate once per value set."""
        key = (tuple(sorted(args.scalars.items())), tuple(sorted(args.floats.items())), tuple(grid))
        v = self._memo.get(key)
        if v is None:
            if len(self._memo) > 64:
                self._memo.clear()
            v = self._memo[key] = compute()
        return v

    def to_bytes(self) -> bytes:
        return json.dumps({"family": self.family, "name": self.name, "params": enc(self.p)}).encode()

    def launch_native(self, args, grid, pid_lo, pid_hi, stream) -> bool:
        """Launch through the library's own plan evaluator (tsb_plan_create / tsb_launch): the JSON
        text of this plan is handed over once and every call is one C call.  Returns False when the
        loaded library has no plan evaluator (the host stand-in of the tests), in which case the
        caller evaluates the plan here in Python (`launch`)."""
        L = rt.lib()
        fn = getattr(L, "tsb_launch", None)
        if fn is None:
            return False
        h = self.__dict__.get("_handle")
        if h is None:
            h = L.tsb_plan_create(self.to_bytes(), -1)
            if not h:
                raise rt.TsbError("tsb_plan_create failed: " + L.tsb_last_error().decode("utf-8", "replace"))
            self._handle = h
        n = args.n_args
        ptrs = (ctypes.c_void_p * max(n, 1))()
        scal = (rt.Scalar * max(n, 1))()
        for k in args.pointer_positions():
            ptrs[k] = args.pointer(k)
        for k, v in args.scalars.items():
            scal[k].kind, scal[k].i = 1, v
        for k, v in args.floats.items():
            scal[k].kind, scal[k].f = 2, v
        g = (ctypes.c_int32 * 3)(*grid)
        key = (tuple(sorted(args.scalars.items())), tuple(sorted(args.floats.items())), tuple(grid), pid_lo, pid_hi)
        need = self._memo.get(("scratch", key))
        if need is None:
            need = L.tsb_launch_scratch_bytes(h, g, pid_lo, pid_hi, scal, n)
            if need < 0:
                self._raise(int(need), "tsb_launch_scratch_bytes")
            if len(self._memo) > 64:
                self._memo.clear()
            self._memo[("scratch", key)] = need
        scratch = args.scratch(need, stream) if need > 0 else None
        status = args.status_word(stream) if self.family == "gemm" else None
        rc = fn(h, g, pid_lo, pid_hi, stream, ptrs, scal, n, scratch, need, status)
        if rc:
            self._raise(rc, "tsb_launch")
        return True

    def _raise(self, rc: int, what: str):
        msg = rt.lib().tsb_last_error().decode("utf-8", "replace")
        if rc == -2:  # well-formed but outside what the kernels implement: the same class as at compile time
            raise UnsupportedTTIR(msg)
        raise rt.TsbError(f"{what}[{self.name}] failed ({rc}): {msg}")

    def launch(self, args, grid, pid_lo, pid_hi, stream):
        raise NotImplementedError

    def describe(self) -> str:
        return f"{self.family}:{self.name}"


def plan_from_bytes(b: bytes) -> Plan:
    j = json.loads(b.decode())
    cls = _FAMILIES[j["family"]]
    return cls(j["name"], dec(j["params"]))


# --------------------------------------------------------------------------
# elementwise family

def _mask_json(mask: Optional[TMask], shape):
    if mask is None:
        return None
    return {"dims": [[[s, bnd] for (s, bnd) in d] for d in mask.dims], "conds": list(mask.scalar_conds)}


class _EwLowering:
    """Linearises the value graphs of all stores into VM ops over one iteration space."""
    FLAG_FIELD = "imm"  # where a load / store carries its MEM_INDEX / MEM_MASK flags

    def __init__(self, kernel: Kernel, an: Analyzer, space: Tuple[int, ...]):
        self.k, self.an, self.space = kernel, an, space
        self.accs: List[dict] = []
        self.ops: List[list] = []  # [opcode, dtype, dst, a, b, c, imm, imm2] with virtual registers
        self.memo: Dict[tuple, int] = {}
        self.nv = 0

    def new(self):
        self.nv += 1
        return self.nv - 1

    def acc_for(self, kind: str, elem: str, shape, dimmap, offset: Poly, strides, mask, other, arg=None,
                wrapped=()):
        """Access descriptor promoted to the iteration space; returns its index."""
        r = len(self.space)
        st = [Poly.const(0)] * r
        mdims = [[] for _ in range(r)]
        conds = list(mask["conds"]) if mask else []
        for d, it_d in enumerate(dimmap):
            if shape[d] > 1:
                st[it_d] = strides[d]
                if mask and mask["dims"][d]:
                    mdims[it_d] = mdims[it_d] + list(mask["dims"][d])
            elif mask and mask["dims"][d]:
                # a masked unit dim gates the whole block: lane 0 valid iff start < bound
                for s, bnd in mask["dims"][d]:
                    conds.append(Poly.fn("cmp_slt", s, bnd))
        wraps = []
        for w in wrapped:
            it_d = dimmap[w.dim]
            wraps.append({"dim": it_d, "offset": w.inner_offset, "stride": w.inner_stride,
                          "modulus": w.modulus, "scale": w.scale})
            for q in (w.inner_stride, w.modulus, w.scale):
                if q.depends_on(("pid", "carry")):
                    raise UnsupportedTTIR("wrap-around stride, modulus or scale depends on program_id")
        if len(wraps) > 2:
            raise UnsupportedTTIR("more than two wrap-around dims in one access")
        for p in [offset] + st + [x for dd in mdims for sb in dd for x in sb] + conds + [w["offset"] for w in wraps]:
            if p.depends_on(("carry",)):
                raise UnsupportedTTIR("elementwise body with an unresolved loop-carried access")
            if not is_affine_in_pid(p):
                raise UnsupportedTTIR("access offset is not affine in program_id")
        for p in st + [sb[1] for dd in mdims for sb in dd] + conds:
            if p.depends_on(("pid",)):
                raise UnsupportedTTIR("stride, mask bound or scalar mask condition depends on program_id")
        if any(len(dd) > 1 for dd in mdims):
            # several upper bounds on one dim: all must share the start; the bound is their minimum
            for i, dd in enumerate(mdims):
                if len(dd) > 1:
                    if any(s != dd[0][0] for s, _ in dd):
                        raise UnsupportedTTIR("conjunction of masks with different starts on one dim")
                    bnd = dd[0][1]
                    for _, b2 in dd[1:]:
                        bnd = Poly.fn("minsi", bnd, b2)
                    mdims[i] = [(dd[0][0], bnd)]
        desc = {"kind": kind, "elem": elem, "arg": arg, "offset": offset, "strides": st,
                "mask": [dd[0] if dd else None for dd in mdims], "conds": conds, "other": other,
                "wrap": wraps}
        self.accs.append(desc)
        return len(self.accs) - 1

    def emit(self, opcode, dtype, a=0, b=0, c=0, imm=0, imm2=0):
        dst = self.new()
        self.ops.append([opcode, dtype, dst, a, b, c, imm, imm2])
        return dst

    def weight(self, n) -> int:
        """Ops a value costs to compute (its distinct non-leaf nodes): the operand with the larger
        weight is evaluated first, so that the lighter one (often a leaf, which emits nothing) is
        what separates it from its consumer and the result stays in the accumulator."""
        memo = self.__dict__.setdefault("_weights", {})

        def nodes(m, seen):
            if not isinstance(m, Node) or m.id in seen or m.op in ("const", "sint", "farg", "load", "index", "maskval"):
                return
            seen.add(m.id)
            for a in m.args:
                nodes(a, seen)
        if n.id not in memo:
            seen = set()
            nodes(n, seen)
            memo[n.id] = len(seen)
        return memo[n.id]

    def values(self, nodes, dimmap):
        """Registers of several operands, evaluated heaviest first."""
        order = sorted(range(len(nodes)), key=lambda i: -self.weight(nodes[i]))
        out = [None] * len(nodes)
        for i in order:
            out[i] = self.value(nodes[i], dimmap)
        return out

    def value(self, n: Node, dimmap: Tuple[int, ...]) -> int:
        key = (n.id, dimmap)
        if key in self.memo:
            return self.memo[key]
        v = self._value(n, dimmap)
        self.memo[key] = v
        return v

    def _value(self, n: Node, dimmap):
        op = n.op
        if op == "load":
            acc: Access = self.an.access_of(n)
            ob = other_bits(acc.other, acc.elem)
            ai = self.acc_for("load", acc.elem, acc.shape, dimmap, acc.offset, acc.strides,
                              _mask_json(acc.mask, acc.shape), ob, acc.arg, acc.wrapped)
            idx, msk, flags = self.lane_operands(acc, dimmap)
            return self.emit("load", acc.elem, a=ai, b=idx, c=msk, **{self.FLAG_FIELD: flags})
        if op in ("splat",):
            return self.value(n.args[0], ())
        if op == "broadcast":
            return self.value(n.args[0], dimmap)
        if op == "expand_dims":
            ax = n.attr("axis")
            return self.value(n.args[0], dimmap[:ax] + dimmap[ax + 1:])
        if op == "const":
            v = float_from_key(n.attr("value"))
            bits = struct.unpack("<I", struct.pack("<f", v))[0]
            return self.emit("const", n.dtype, imm=bits)
        if op == "sint":
            p = n.attr("poly")
            if p.depends_on(("pid", "it", "carry")):
                ai = self.acc_for("index", n.dtype, (), (), p, (), None, None)
                return self.emit("load", n.dtype, a=ai)
            return self.emit("const", n.dtype, imm=("poly", p))
        if op == "farg":
            return self.emit("const", n.dtype, imm=("farg", n.attr("arg")))
        if op == "index":
            ai = self.acc_for("index", n.dtype, n.shape, dimmap, n.attr("offset"), n.attr("strides"), None, None)
            return self.emit("load", n.dtype, a=ai)
        if op == "maskval":
            m = {"dims": [[list(sb) for sb in d] for d in n.attr("dims")], "conds": list(n.attr("conds"))}
            ai = self.acc_for("maskprobe", "i1", n.shape, dimmap, Poly.const(0), [Poly.const(0)] * len(n.shape), m, None)
            return self.emit("load", "i1", a=ai)
        if op in ("addf", "subf", "mulf", "divf", "maxnumf", "minnumf", "maximumf", "minimumf", "remf",
                  "addi", "subi", "muli", "divsi", "remsi", "divui", "remui", "minsi", "maxsi", "minui",
                  "maxui", "andi", "ori", "xori", "shli", "shrsi", "shrui"):
            a, b = self.values(n.args, dimmap)
            return self.emit(op, n.dtype, a=a, b=b)
        if op in ("exp", "exp2", "log", "log2", "sqrt", "rsqrt", "sin", "cos", "tanh", "erf", "absf",
                  "negf", "floor", "ceil", "absi"):
            return self.emit(op, n.dtype, a=self.value(n.args[0], dimmap))
        if op == "fma":
            a, b, c = self.values(n.args, dimmap)
            return self.emit("fma", n.dtype, a=a, b=b, c=c)
        if op == "cmpf":
            a, b = self.values(n.args, dimmap)
            return self.emit("cmpf", n.args[0].dtype, a=a, b=b, imm=rt.CMPF[n.attr("pred")])
        if op == "cmpi":
            a, b = self.values(n.args, dimmap)
            return self.emit("cmpi", n.args[0].dtype, a=a, b=b, imm=rt.CMPI[n.attr("pred")])
        if op == "select":
            c, a, b = self.values(n.args, dimmap)
            return self.emit("select", n.dtype, a=c, b=a, c=b)
        if op == "cast":
            kind = n.attr("kind")
            src = n.args[0]
            a = self.value(src, dimmap)
            if kind == "bitcast":
                if rt.DTYPE_SIZE.get(src.dtype) != 4 or rt.DTYPE_SIZE.get(n.dtype) != 4:
                    raise UnsupportedTTIR("bitcast between types that are not 32 bits wide")
                return self.emit("bitcast", n.dtype, a=a)
            mode = 1 if kind in ("uitofp", "fptoui", "extui") else 0
            # registers hold f16 / bf16 values exactly widened to f32 and i8 / i16 sign-extended:
            # widening to f32 and signed widening to i32 change nothing
            if (kind in ("extf", "fp_to_fp") and n.dtype == "f32" and src.dtype in ("f16", "bf16")) or \
                    (kind == "extsi" and n.dtype == "i32" and src.dtype in ("i8", "i16")):
                return a
            return self.emit("cast", n.dtype, a=a, imm=rt.DTYPES[src.dtype], imm2=mode)
        if op == "reduce":
            # a full fold of a 1-D block whose lanes are the whole iteration space: every lane of the
            # result holds the total (the packed kernel folds across the threads of a program)
            src, comb = n.args[0], n.attr("comb")
            lanes = int(np.prod(self.space)) if self.space else 1
            if len(src.shape) != 1 or dimmap != () or src.shape[0] != lanes or self.space[-1] != lanes:
                raise UnsupportedTTIR("elementwise family: only full folds of the 1-D block the kernel stores")
            if lanes % 4 or not 16 <= lanes <= 4096:
                raise UnsupportedTTIR("elementwise family: a fold needs a block of 16 to 4096 lanes, a multiple of 4")
            if comb not in ("addf", "mulf", "maxnumf", "minnumf", "maximumf", "minimumf", "addi", "muli", "maxsi",
                            "minsi", "maxui", "minui", "andi", "ori", "xori"):
                raise UnsupportedTTIR(f"elementwise family: reduction with combiner {comb}")
            if type(self) is not _EwLowering:
                raise UnsupportedTTIR("not an elementwise lowering")
            a = self.value(src, (len(self.space) - 1,))
            return self.emit("reduce", n.dtype, a=a, imm=comb)
        raise UnsupportedTTIR(f"operation {op} has no elementwise lowering")

    def lane_operands(self, acc: Access, dimmap):
        """(index register, mask register, flags) of an access with data-dependent offsets / mask."""
        idx = msk = flags = 0
        if acc.indirect is not None:
            idx, flags = self.value(acc.indirect, dimmap), flags | rt.MEM_INDEX
        if acc.mask_data is not None:
            msk, flags = self.value(acc.mask_data, dimmap), flags | rt.MEM_MASK
        return idx, msk, flags

    def lower(self, stores: List[Access]):
        for acc in stores:
            shape = acc.shape
            dimmap = tuple(range(len(self.space) - len(shape), len(self.space)))
            v = self.value(acc.value, dimmap)
            ai = self.acc_for("store", acc.elem, shape, dimmap, acc.offset, acc.strides,
                              _mask_json(acc.mask, shape), None, acc.arg, acc.wrapped)
            idx, msk, flags = self.lane_operands(acc, dimmap)
            self.ops.append(["store", acc.elem, msk if flags & rt.MEM_MASK else -1, ai, v, idx, flags, 0])
        return self.allocate()

    def allocate(self):
        """Hoist loads; turn constants into immediate operands; keep a value that only the next op
        reads in the accumulator; map what remains onto TSB_NUM_REGS shared-memory registers."""
        return self._allocate(True)

    def _allocate(self, hoist_loads: bool):
        ACC, IMM = rt.REG_ACC, rt.REG_IMM
        # plain loads go first (all of them in flight before the first use); a load that takes an index
        # or mask operand stays where its operands are computed
        plain = lambda o: o[0] == "load" and o[6] == 0
        loads = [o for o in self.ops if plain(o)]
        rest = [o for o in self.ops if not plain(o)]
        ops = [list(o) for o in (loads + rest if hoist_loads else self.ops)]
        slots = {"select": (3, 4, 5), "fma": (3, 4, 5)}

        def read_slots(o):
            if o[0] == "const":
                return ()
            if o[0] == "load":   # [load, type, dst, access, index, mask, flags, -]
                return ((4,) if o[6] & rt.MEM_INDEX else ()) + ((5,) if o[6] & rt.MEM_MASK else ())
            if o[0] == "store":  # [store, type, mask, access, value, index, flags, -]
                return (4,) + ((5,) if o[6] & rt.MEM_INDEX else ()) + ((2,) if o[6] & rt.MEM_MASK else ())
            if o[0] in slots:
                return slots[o[0]]
            return (3,) if len(_reads(o)) == 1 else (3, 4)

        # 1. constants become immediates (one per op; casts use imm2 themselves; stores need a value)
        consts = {o[2]: o for o in ops if o[0] == "const"}
        marks: Dict[tuple, int] = {}  # (op index, slot) -> ACC / IMM
        for i, o in enumerate(ops):
            if o[0] in ("store", "cast", "load", "const", "reduce"):
                continue
            for sl in read_slots(o):
                if o[sl] in consts and not any(marks.get((i, s2)) == IMM for s2 in read_slots(o)):
                    marks[(i, sl)] = IMM
                    o[7] = consts[o[sl]][6]
        still_used = {o[sl] for i, o in enumerate(ops) for sl in read_slots(o) if (i, sl) not in marks}
        keep = [i for i, o in enumerate(ops) if not (o[0] == "const" and o[2] not in still_used)]
        remap_idx = {old: new for new, old in enumerate(keep)}
        marks = {(remap_idx[i], sl): m for (i, sl), m in marks.items() if i in remap_idx}
        ops = [ops[i] for i in keep]
        # 2. the previous op's result is read from the accumulator
        prev = None
        for i, o in enumerate(ops):
            for sl in read_slots(o):
                if (i, sl) not in marks and prev is not None and o[sl] == prev:
                    marks[(i, sl)] = ACC
            prev = o[2] if o[0] != "store" else None
        # 3. registers for every value that is read in some other way
        last_use: Dict[int, int] = {}
        for i, o in enumerate(ops):
            for sl in read_slots(o):
                if (i, sl) not in marks:
                    last_use[o[sl]] = i
        free = list(range(rt.TSB_NUM_REGS - 1, -1, -1))
        phys: Dict[int, int] = {}
        out = []
        for i, o in enumerate(ops):
            reads = [(sl, o[sl]) for sl in read_slots(o) if (i, sl) not in marks]
            mapped = {v: phys[v] for _, v in reads}
            for v in {v for _, v in reads}:
                if last_use[v] == i:
                    free.append(phys.pop(v))
            if o[0] != "store":
                if o[2] in last_use:
                    if not free:
                        raise UnsupportedTTIR(f"elementwise body needs more than {rt.TSB_NUM_REGS} live block values")
                    phys[o[2]] = free.pop()
                    o[2] = phys[o[2]]
                else:
                    o[2] = ACC  # only the next op (or nothing) reads it
            for sl in read_slots(o):
                m = marks.get((i, sl))
                o[sl] = m if m is not None else mapped[o[sl]]
            out.append(o)
        if len(out) > rt.TSB_MAX_OPS:
            raise UnsupportedTTIR(f"elementwise body of {len(out)} ops exceeds {rt.TSB_MAX_OPS}")
        if len(self.accs) > rt.TSB_MAX_ACCESSES:
            raise UnsupportedTTIR(f"{len(self.accs)} block accesses exceed {rt.TSB_MAX_ACCESSES}")
        return out


def _reads(o):
    opc = o[0]
    if opc == "load":   # block programs: flags in imm2, index in b, mask in c
        f = o[7] if isinstance(o[7], int) else 0
        return ([o[4]] if f & rt.MEM_INDEX else []) + ([o[5]] if f & rt.MEM_MASK else [])
    if opc in ("const", "iota", "loop_begin", "loop_end"):
        return []
    if opc == "store":  # value in b; block programs: index in c, mask in dst
        f = o[7] if isinstance(o[7], int) else 0
        return [o[4]] + ([o[5]] if f & rt.MEM_INDEX else []) + ([o[2]] if f & rt.MEM_MASK else [])
    if opc in ("select", "fma"):
        return [o[3], o[4], o[5]]
    if opc in ("exp", "exp2", "log", "log2", "sqrt", "rsqrt", "sin", "cos", "tanh", "erf", "absf", "negf",
               "floor", "ceil", "absi", "cast", "bitcast", "mov", "reduce", "scan"):
        return [o[3]]
    return [o[3], o[4]]


def _remap(o, mapped):
    opc = o[0]
    if opc in ("store", "load"):
        f = o[7] if isinstance(o[7], int) else 0
        if opc == "store":
            o[4] = mapped[o[4]]
            if f & rt.MEM_INDEX:
                o[5] = mapped[o[5]]
            if f & rt.MEM_MASK:
                o[2] = mapped[o[2]]
        else:
            if f & rt.MEM_INDEX:
                o[4] = mapped[o[4]]
            if f & rt.MEM_MASK:
                o[5] = mapped[o[5]]
        return
    rs = _reads(o)
    if len(rs) >= 1:
        o[3] = mapped[o[3]]
    if len(rs) >= 2:
        o[4] = mapped[o[4]]
    if len(rs) >= 3:
        o[5] = mapped[o[5]]


class ElementwisePlan(Plan):
    """Loop-free bodies, and bodies whose scf.for loops carry no data (only pointers/integers):
    every run of consecutive stores is one VM program ("segment"); loops are walked on the host,
    one launch per iteration and segment, with the iteration counter folded into the offsets.
    Launches are stream-ordered, so the sequential meaning of the loops is preserved."""
    family = "elementwise"

    @staticmethod
    def build(kernel: Kernel, an: Analyzer) -> "ElementwisePlan":
        segments: List[dict] = []
        stored_args = set()

        def lower_segment(stores: List[Access]):
            shapes = {s.shape for s in stores}
            full = max(shapes, key=lambda sh: (len(sh), int(np.prod(sh)) if sh else 1))
            rank = max(len(full), 1)
            space = tuple([1] * (rank - len(full)) + list(full))
            for sh in shapes:
                pad = tuple([1] * (rank - len(sh)) + list(sh))
                if any(x != y and x != 1 for x, y in zip(pad, space)):
                    raise UnsupportedTTIR("stores of different block shapes in one kernel")
            if rank > rt.TSB_MAX_RANK:
                raise UnsupportedTTIR(f"blocks of rank {rank} (max {rt.TSB_MAX_RANK})")
            low = _EwLowering(kernel, an, space)
            ops = low.lower(stores)
            if any(o[0] == "reduce" for o in ops) and any(tuple(s.shape) != tuple(full) for s in stores):
                # a scalar result stored beside the block (mean / rstd of a one-block LayerNorm) would be
                # written by every lane: leave such bodies to the block-program engine
                raise UnsupportedTTIR("elementwise family: a fold whose result is also stored as a scalar")
            segments.append({"space": list(space), "accs": low.accs, "ops": ops})
            stored_args.update(s.arg for s in stores)
            return len(segments) - 1

        def lower_run(stores: List[Access]):
            """A run of consecutive stores as one segment, or as several (launched in order) when
            together they exceed the engine's limits on accesses, ops or live values."""
            try:
                return [lower_segment(stores)]
            except UnsupportedTTIR:
                if len(stores) == 1:
                    raise
                half = len(stores) // 2
                return lower_run(stores[:half]) + lower_run(stores[half:])

        def walk(effects):
            tree, run = [], []
            for kind, e in effects:
                if kind == "store":
                    run.append(e)
                    continue
                if run:
                    tree.extend(["seg", i] for i in lower_run(run))
                    run = []
                loop: Loop = e
                for init in loop.inits:
                    if isinstance(init, TData):
                        raise UnsupportedTTIR("elementwise family: a loop carries block data (an accumulator)")
                for q in (loop.lb, loop.ub, loop.step):
                    if q.depends_on(("pid", "carry")):
                        raise UnsupportedTTIR("elementwise family: loop bounds depend on program_id")
                tree.append(["loop", loop.id, loop.lb, loop.ub, loop.step, walk(loop.effects)])
            if run:
                tree.extend(["seg", i] for i in lower_run(run))
            return tree

        tree = walk(kernel.effects)
        if not segments:
            raise UnsupportedTTIR("kernel stores nothing")
        if len(segments) > 1:
            # values are recomputed (reloaded) per segment: a pointer that is both read and written
            # could then observe a different order than the kernel text
            loaded = {d["arg"] for sg in segments for d in sg["accs"] if d["kind"] == "load"}
            if loaded & stored_args:
                raise UnsupportedTTIR("elementwise family: a buffer is both loaded and stored across loop segments")
        return ElementwisePlan(kernel.name, {"segments": segments, "tree": tree})

    def launch(self, args, grid, pid_lo, pid_hi, stream):
        plan = self.memo(args, grid, lambda: self._schedule(args, grid))
        g = (ctypes.c_int32 * 3)(*grid)
        fn = rt.lib().tsb_elementwise
        for accs, ops, arg_of in plan:
            for a, i in zip(accs, arg_of):
                if i is not None:
                    a.base = args.pointer(i)
            rc = fn(accs, len(accs), ops, len(ops), g, pid_lo, pid_hi, stream)
            if rc:
                rt.check(rc, f"tsb_elementwise[{self.name}]")

    def _perfect_nest(self):
        """(segment index, [(loop id, lb, ub, step)] outermost first) when the kernel is one segment
        inside a perfect loop nest whose iterations only shift offsets and mask starts; else None.
        Such a nest runs on the device, inside one launch (TSB_OP_LOOP_BEGIN / END around the body)."""
        node, loops = self.p["tree"], []
        while len(node) == 1 and node[0][0] == "loop":
            _, lid, lb, ub, step, children = node[0]
            loops.append((lid, lb, ub, step))
            node = children
        if not loops or len(loops) > rt.TSB_MAX_LOOPS or len(node) != 1 or node[0][0] != "seg":
            return None
        for _, lb, ub, step in loops:
            if any(q.depends_on(("it",)) for q in (lb, ub, step)):
                return None
        seg = self.p["segments"][node[0][1]]
        for d in seg["accs"]:
            fixed = d["strides"] + [m[1] for m in d["mask"] if m] + d["conds"] + \
                [x for w in d["wrap"] for x in w.values() if isinstance(x, Poly)]
            if any(q.depends_on(("it",)) for q in fixed):
                return None
            if not all(_is_affine_in_its(q) for q in [d["offset"]] + [m[0] for m in d["mask"] if m]):
                return None
        for o in seg["ops"]:
            for imm in (o[6], o[7]):
                if isinstance(imm, (list, tuple)) and imm[0] == "poly" and imm[1].depends_on(("it",)):
                    return None
        return node[0][1], loops

    def _schedule(self, args, grid):
        """The ordered list of launches for these scalar arguments: one launch with device-side loops
        for a perfect nest, else the loop tree flattened on the host (one launch per iteration)."""
        out = []
        env = LaunchEnv(args.scalars, grid)
        nest = self._perfect_nest()
        if nest is not None:
            si, loops = nest
            seg = dict(self.p["segments"][si])
            seg["loop_depth"] = {str(lid): depth for depth, (lid, _, _, _) in enumerate(loops)}
            head = [["loop_begin", "i32", -1, depth, 0, 0, ("trip", lid), 0] for depth, (lid, _, _, _) in enumerate(loops)]
            tail = [["loop_end", "i32", -1, depth, 0, 0, 0, 0] for depth in reversed(range(len(loops)))]
            seg["ops"] = head + list(seg["ops"]) + tail
            trips = {str(lid): Poly.fn("ceildivsi", ub - lb, step) for lid, lb, ub, step in loops}
            e = env.at()
            if any(int(step.evaluate(e)) <= 0 for _, _, _, step in loops):
                raise UnsupportedTTIR("loop with a non-positive step")
            for lid, _, _, _ in loops:
                env.base[("it", lid)] = 0
            return [self._evaluate(seg, args, env, trips)]

        def run(tree):
            for node in tree:
                if node[0] == "seg":
                    out.append(self._evaluate(self.p["segments"][node[1]], args, env))
                    continue
                _, lid, lb, ub, step, children = node
                e = env.at()
                lo, hi, st = int(lb.evaluate(e)), int(ub.evaluate(e)), int(step.evaluate(e))
                if st <= 0:
                    raise UnsupportedTTIR("loop with a non-positive step")
                trips = max(0, -(-(hi - lo) // st))
                if len(out) + trips > 4096:
                    raise UnsupportedTTIR("elementwise family: more than 4096 launches for one kernel call")
                for it in range(trips):
                    env.base[("it", lid)] = it
                    run(children)
                env.base.pop(("it", lid), None)
        run(self.p["tree"])
        return out

    def _evaluate(self, seg, args, env, trips=None):
        space = seg["space"]
        rank = len(space)
        n = len(seg["accs"])
        accs = (rt.Access * n)()
        arg_of = []
        e0 = env.at()
        for ai, d in enumerate(seg["accs"]):
            a = accs[ai]
            kind = d["kind"]
            a.dtype = rt.DTYPES[d["elem"]]
            a.rank = rank
            a.is_store = {"load": 0, "store": 1, "maskprobe": 2, "index": 3}[kind]
            off0, inc = env.affine_pid(d["offset"])
            a.offset0 = off0
            for k in range(3):
                a.offset_pid[k] = inc[k]
            gate = all(int(c.evaluate(e0)) != 0 for c in d["conds"])
            for k in range(rank):
                a.sizes[k] = space[k]
                a.strides[k] = int(d["strides"][k].evaluate(e0))
                m = d["mask"][k]
                if m is not None:
                    a.masked[k] = 1
                    s0, sinc = env.affine_pid(m[0])
                    a.mask_start0[k] = s0
                    for j in range(3):
                        a.mask_start_pid[k][j] = sinc[j]
                    a.mask_bound[k] = int(m[1].evaluate(e0))
            if not gate:
                # a false scalar conjunct empties the block (MaskAnalysis.cpp:224-267)
                a.masked[0] = 1
                a.mask_bound[0] = -(1 << 62)
            if d["other"] is not None:
                a.has_other = 1
                a.other_bits = d["other"]
            wraps = d.get("wrap") or []
            a.n_wrap = len(wraps)
            for wi, w in enumerate(wraps):
                ww = a.wrap[wi]
                ww.dim = w["dim"]
                o0, oinc = env.affine_pid(w["offset"])
                ww.offset0 = o0
                for j in range(3):
                    ww.offset_pid[j] = oinc[j]
                ww.stride = int(w["stride"].evaluate(e0))
                ww.modulus = int(w["modulus"].evaluate(e0))
                ww.scale = int(w["scale"].evaluate(e0))
                if ww.modulus <= 0:
                    raise UnsupportedTTIR("wrap-around access with a non-positive modulus")
            # block programs: advance per iteration of each enclosing loop (slot = nesting depth)
            for lid, depth in (seg.get("loop_depth") or {}).items():
                lid = int(lid)
                if not (d["offset"].depends_on(("it",)) or any(m and m[0].depends_on(("it",)) for m in d["mask"])):
                    continue
                env.base[("it", lid)] = 1
                a.offset_loop[depth] += int(d["offset"].evaluate(env.at())) - off0
                for k in range(rank):
                    m = d["mask"][k]
                    if m is not None:
                        a.mask_start_loop[k][depth] += int(m[0].evaluate(env.at())) - a.mask_start0[k]
                env.base[("it", lid)] = 0
            arg_of.append(d.get("arg"))
        ops = (rt.Op * len(seg["ops"]))()
        for k, o in enumerate(seg["ops"]):
            opc, dt, dst, ra, rb, rc, imm, imm2 = o
            x = ops[k]
            x.opcode = rt.OPCODES[opc]
            x.type = rt.DTYPES[dt]
            # a store names no result; in tsb_elementwise bodies its dst field carries the mask operand
            flags = imm2 if "loops" in seg else imm  # block programs keep the memory flags in imm2
            store_mask = opc == "store" and isinstance(flags, int) and flags & rt.MEM_MASK
            x.dst, x.a, x.b, x.c = (dst if (opc != "store" or store_mask) else 0), ra, rb, rc
            if isinstance(imm, (list, tuple)) and imm[0] == "trip":
                q = trips[str(imm[1])]
                x.imm = max(0, int(q.evaluate(e0)))
            elif isinstance(imm, str):
                x.imm = rt.OPCODES[imm]  # combiner of a reduction
            elif isinstance(imm, (list, tuple)):
                if imm[0] == "poly":
                    x.imm = int(imm[1].evaluate(e0)) & 0xffffffff
                else:  # farg
                    x.imm = struct.unpack("<I", struct.pack("<f", float(args.floats[imm[1]])))[0]
            else:
                x.imm = imm
            if isinstance(imm2, (list, tuple)):  # an immediate operand that is a launch-time scalar
                if imm2[0] == "poly":
                    x.imm2 = int(imm2[1].evaluate(e0)) & 0xffffffff
                else:
                    x.imm2 = struct.unpack("<I", struct.pack("<f", float(args.floats[imm2[1]])))[0]
            else:
                x.imm2 = imm2
        return accs, ops, arg_of


# --------------------------------------------------------------------------
# block programs: loop-free bodies with reductions along block axes

class _DimUnion:
    """Union-find over symbolic block dims, used to discover the iteration space of a body with reductions."""

    def __init__(self):
        self.parent, self.size = {}, {}

    def fresh(self, size: int):
        d = len(self.parent)
        self.parent[d], self.size[d] = d, size
        return d

    def find(self, d):
        while self.parent[d] != d:
            self.parent[d] = self.parent[self.parent[d]]
            d = self.parent[d]
        return d

    def union(self, a, b):
        ra, rb = self.find(a), self.find(b)
        if ra == rb:
            return
        if self.size[ra] != self.size[rb]:
            raise UnsupportedTTIR("block program: dims of different sizes would have to coincide")
        self.parent[max(ra, rb)] = min(ra, rb)


def _discover_space(stores: List[Access], loops: Dict[int, Loop] = None):
    """Symbolic dims of every node reachable from the stores.  A reduction introduces a dim its result
    does not have; a node reached along two paths has one set of dims (they are unified); a
    loop-carried value, its initial value, its yielded value and the loop's result share their dims.
    Returns (space sizes, {node id: tuple of space positions}, {reduce node id: reduced space position})."""
    uf = _DimUnion()
    loops = loops or {}
    node_dims: Dict[int, tuple] = {}
    order: List[tuple] = []  # (a, b): dim a precedes dim b in some node
    red_dim: Dict[int, int] = {}
    carried: Dict[tuple, tuple] = {}

    def visit(n: Node, dims: tuple):
        if n.id in node_dims:
            for a, b in zip(node_dims[n.id], dims):
                uf.union(a, b)
            return
        node_dims[n.id] = dims
        order.extend(zip(dims, dims[1:]))
        if n.op in ("splat",):
            visit(n.args[0], ())
        elif n.op == "broadcast":
            visit(n.args[0], dims)
        elif n.op == "expand_dims":
            ax = n.attr("axis")
            visit(n.args[0], dims[:ax] + dims[ax + 1:])
        elif n.op == "reduce":
            ax = n.attr("axis")
            src = n.args[0]
            d = red_dim.setdefault(n.id, uf.fresh(src.shape[ax]))
            visit(src, dims[:ax] + (d,) + dims[ax:])
        elif n.op == "argreduce":
            ax = n.attr("axis")
            # both results of one tt.reduce share the reduced dim
            key = ("arg", n.args[0].id, n.args[1].id, ax)
            d = red_dim.setdefault(key, uf.fresh(n.args[0].shape[ax]))
            red_dim[n.id] = d
            for a in n.args:
                visit(a, dims[:ax] + (d,) + dims[ax:])
        elif n.op in ("iter_arg", "loop_result"):
            key = (n.attr("loop"), n.attr("k"))
            if key in carried:
                for a, b in zip(carried[key], dims):
                    uf.union(a, b)
                return
            carried[key] = dims
            loop = loops.get(key[0])
            if loop is None:
                raise UnsupportedTTIR("block program: loop-carried value of an unknown loop")
            init, yld = loop.inits[key[1]], loop.yields[key[1]]
            if not isinstance(init, TData) or not isinstance(yld, TData):
                raise UnsupportedTTIR("block program: loop-carried value is not block data")
            visit(init.node, dims)
            visit(yld.node, dims)
        elif n.op == "dot":
            raise UnsupportedTTIR("block program: operation dot")
        else:
            for a in n.args:
                if isinstance(a, Node):
                    visit(a, dims if a.shape == n.shape or len(a.shape) == len(dims) else ())

    for st in stores:
        visit(st.value, tuple(uf.fresh(sz) for sz in st.shape))
        node_dims[("store", id(st))] = node_dims[st.value.id]
    reps = []
    for dims in node_dims.values():
        r = [uf.find(d) for d in dims]
        if len(set(r)) != len(r):
            raise UnsupportedTTIR("block program: one value is indexed twice by the same dim")
        for d in r:
            if d not in reps:
                reps.append(d)
    # order the space so that every node's dims appear in increasing position
    edges = {(uf.find(a), uf.find(b)) for a, b in order if uf.find(a) != uf.find(b)}
    space: List[int] = []
    remaining = list(reps)
    while remaining:
        free = [d for d in remaining if not any(b == d and a in remaining for a, b in edges)]
        if not free:
            raise UnsupportedTTIR("block program: the values' dims cannot be ordered consistently (transposed use)")
        space.append(free[0])
        remaining.remove(free[0])
    pos = {d: i for i, d in enumerate(space)}
    maps = {k: tuple(pos[uf.find(d)] for d in dims) for k, dims in node_dims.items()}
    sizes = [uf.size[d] for d in space]
    red_pos = {nid: pos[uf.find(d)] for nid, d in red_dim.items() if isinstance(nid, int)}
    return sizes, maps, red_pos


class _BpLowering(_EwLowering):
    """Lowering for tsb_block_program: registers carry a mask of the space dims they extend along."""

    def __init__(self, kernel, an, space, red_pos):
        super().__init__(kernel, an, tuple(space))
        self.vmask: Dict[int, int] = {}
        self.acc_mask: Dict[int, int] = {}
        self.red_pos = red_pos
        self.arg_pairs: Dict[tuple, tuple] = {}

    FLAG_FIELD = "imm2"  # a block-program store's imm names the dims it walks

    def acc_for(self, kind, elem, shape, dimmap, offset, strides, mask, other, arg=None, wrapped=()):
        # a mask bound that moves with a loop counter (`k < K - it*BLOCK`) is the same mask with the
        # counter moved into the start (`it*BLOCK + k < K`): dims = max(min(s+size,b),s)-s is shift-invariant
        if mask:
            dims = []
            for dd in mask["dims"]:
                nd = []
                for st, bnd in dd:
                    var = Poly({m: c for m, c in bnd.terms.items() if any(a[0] == "it" for a in m)})
                    nd.append([st - var, bnd - var])
                dims.append(nd)
            mask = {"dims": dims, "conds": mask["conds"]}
        ai = super().acc_for(kind, elem, shape, dimmap, offset, strides, mask, other, arg, wrapped)
        d = self.accs[ai]
        for q in d["strides"] + [sb[1] for sb in d["mask"] if sb] + d["conds"] + \
                [x for w in d["wrap"] for x in w.values() if isinstance(x, Poly)]:
            if q.depends_on(("it",)):
                raise UnsupportedTTIR("block program: stride, mask bound or wrap-around term depends on a loop counter")
        for q in [d["offset"]] + [sb[0] for sb in d["mask"] if sb]:
            if not _is_affine_in_its(q):
                raise UnsupportedTTIR("block program: access offset is not affine in the loop counters")
        m = 0
        for d, it_d in enumerate(dimmap):
            if shape[d] > 1:
                m |= 1 << it_d
        self.acc_mask[ai] = m
        return ai

    def emit(self, opcode, dtype, a=0, b=0, c=0, imm=0, imm2=0, mask=None):
        dst = self.new()
        op = [opcode, dtype, dst, a, b, c, imm, imm2]
        if mask is None:
            if opcode == "load":
                mask = self.acc_mask[a]
            else:
                mask = 0
                for r in _reads(op):
                    mask |= self.vmask[r]
        self.vmask[dst] = mask
        self.ops.append(op)
        return dst

    def _value(self, n: Node, dimmap):
        if n.op in ("iter_arg", "loop_result"):
            key = (n.attr("loop"), n.attr("k"))
            if key not in self.carried_reg:
                raise UnsupportedTTIR("block program: loop-carried value used outside its loop's scope")
            return self.carried_reg[key]
        if n.op == "argreduce":
            ax, d = n.attr("axis"), self.red_pos[n.id]
            sub = dimmap[:ax] + (d,) + dimmap[ax:]
            key = ("arg", n.args[0].id, n.args[1].id, dimmap)
            pair = self.arg_pairs.get(key)
            if pair is None:
                val = self.value(n.args[0], sub)
                idx = self.value(n.args[1], sub)
                m = (self.vmask[val] | self.vmask[idx]) & ~(1 << d)
                rv = self.emit("argreduce", n.args[0].dtype, a=val, b=idx, imm=1 if n.attr("comb") == "argmax" else 0,
                               imm2=d, mask=m)
                ri = self.new()  # the op writes a second register: the winning index
                self.vmask[ri] = m
                self.ops[-1][5] = ri
                pair = self.arg_pairs[key] = (rv, ri)
            return pair[n.attr("out")]
        if n.op == "scan":
            src = self.value(n.args[0], dimmap)
            return self.emit("scan", n.dtype, a=src, imm=n.attr("comb"), imm2=dimmap[n.attr("axis")], mask=self.vmask[src])
        if n.op == "reduce":
            ax, comb = n.attr("axis"), n.attr("comb")
            if comb not in ("addf", "mulf", "maxnumf", "minnumf", "maximumf", "minimumf", "addi", "muli", "maxsi",
                            "minsi", "maxui", "minui", "andi", "ori", "xori"):
                raise UnsupportedTTIR(f"block program: reduction with combiner {comb}")
            d = self.red_pos[n.id]
            src = self.value(n.args[0], dimmap[:ax] + (d,) + dimmap[ax:])
            return self.emit("reduce", n.dtype, a=src, imm=comb, imm2=d, mask=self.vmask[src] & ~(1 << d))
        return super()._value(n, dimmap)

    def lower(self, effects, maps, loops):
        self.carried_reg: Dict[tuple, int] = {}
        self.loop_spans: List[tuple] = []   # (first op index, last op index) of every loop
        self.loop_trips: Dict[int, Poly] = {}
        self.loop_depth: Dict[int, int] = {}
        self._walk(effects, maps, loops, 0)
        return self.allocate_masked()

    def _walk(self, effects, maps, loops, depth):
        for kind, e in effects:
            if kind == "store":
                dimmap = maps[("store", id(e))]
                v = self.value(e.value, dimmap)
                ai = self.acc_for("store", e.elem, e.shape, dimmap, e.offset, e.strides,
                                  _mask_json(e.mask, e.shape), None, e.arg, e.wrapped)
                idx, msk, flags = self.lane_operands(e, dimmap)
                self.ops.append(["store", e.elem, msk if flags & rt.MEM_MASK else -1, ai, v, idx, self.acc_mask[ai], flags])
                continue
            loop: Loop = e
            if depth >= 4:
                raise UnsupportedTTIR("block program: loops nested more than four deep")
            if loop.trip.depends_on(("pid", "it", "carry")):
                raise UnsupportedTTIR("block program: loop trip count depends on program_id or on an outer loop")
            # carried block values that something reads (dead ones have no dims and need no register)
            data_k = [k for k, init in enumerate(loop.inits) if isinstance(init, TData) and init.node.id in maps
                      and isinstance(loop.yields[k], TData) and loop.yields[k].node.id in maps]
            # carried registers: written before the loop (initial value) and at the end of every iteration
            for k in data_k:
                init = loop.inits[k].node
                dimmap = maps[init.id]
                src = self.value(init, dimmap)
                r = self.emit("mov", init.dtype, a=src, mask=self._mask_of(init, dimmap))
                self.carried_reg[(loop.id, k)] = r
            begin = len(self.ops)
            self.ops.append(["loop_begin", "i32", -1, depth, 0, 0, ("trip", loop.id), 0])
            self.loop_trips[loop.id] = loop.trip
            self.loop_depth[loop.id] = depth
            self._walk(loop.effects, maps, loops, depth + 1)
            new_vals = []
            for k in data_k:
                y = loop.yields[k].node
                v = self.value(y, maps[y.id])
                # through a temporary, so that carried values that exchange places are not clobbered
                new_vals.append(self.emit("mov", y.dtype, a=v, mask=self.vmask[self.carried_reg[(loop.id, k)]])
                                if len(data_k) > 1 else v)
            for k, v in zip(data_k, new_vals):
                r = self.carried_reg[(loop.id, k)]
                self.ops.append(["mov", loop.yields[k].node.dtype, r, v, 0, 0, 0, 0])
            self.ops.append(["loop_end", "i32", -1, depth, 0, 0, 0, 0])
            self.ops[begin][4] = len(self.ops)  # index of the op after the loop end
            self.loop_spans.append((begin, len(self.ops) - 1))

    def _mask_of(self, n: Node, dimmap):
        m = 0
        for d, it_d in enumerate(dimmap):
            if n.shape[d] > 1:
                m |= 1 << it_d
        return m

    def allocate_masked(self):
        """Physical registers are shared-memory regions; a region is reused only by values of the same mask."""
        ops = self.ops
        last_use: Dict[int, int] = {}
        first_def: Dict[int, int] = {}
        for i, o in enumerate(ops):
            for r in _reads(o):
                last_use[r] = i
            if o[0] not in ("store", "loop_begin", "loop_end"):
                first_def.setdefault(o[2], i)
        # a value defined before a loop and read inside it is read again in every iteration
        for b, e in getattr(self, "loop_spans", []):
            for r, d in first_def.items():
                if d < b and b <= last_use.get(r, -1) <= e:
                    last_use[r] = e
        free: Dict[int, List[int]] = {}
        masks: List[int] = []
        phys: Dict[int, int] = {}
        out = []
        for i, o in enumerate(ops):
            o = list(o)
            if o[0] in ("loop_begin", "loop_end"):
                out.append(o)
                continue
            reads = _reads(o)
            mapped = {r: phys[r] for r in reads}
            if o[0] != "store" and o[2] in phys:
                # second definition of a loop-carried register: same region
                o[2] = phys[o[2]]
                _remap(o, mapped)
                for r in set(reads):
                    if last_use[r] == i and r in phys:
                        free.setdefault(self.vmask[r], []).append(phys.pop(r))
                out.append(o)
                continue
            if o[0] != "store":
                m = self.vmask[o[2]]
                # an elementwise result may overwrite an operand of the same mask that dies here; a
                # reduction never writes into its own source
                if o[0] not in ("reduce", "argreduce", "scan"):
                    for r in set(reads):
                        if last_use[r] == i and r in phys:
                            free.setdefault(self.vmask[r], []).append(phys.pop(r))
                if free.get(m):
                    dst = free[m].pop()
                else:
                    dst = len(masks)
                    masks.append(m)
                second = None
                if o[0] == "argreduce":  # writes two registers: the winning value and its index
                    if free.get(m):
                        second = free[m].pop()
                    else:
                        second = len(masks)
                        masks.append(m)
                if o[2] in last_use:
                    phys[o[2]] = dst
                else:
                    free.setdefault(m, []).append(dst)
                o[2] = dst
                if second is not None:
                    v2 = o[5]
                    if v2 in last_use:
                        phys[v2] = second
                    else:
                        free.setdefault(m, []).append(second)
            _remap(o, mapped)
            if o[0] == "argreduce":
                o[5] = second
            for r in set(reads):
                if last_use[r] == i and r in phys:
                    free.setdefault(self.vmask[r], []).append(phys.pop(r))
            out.append(o)
        if len(masks) > 24:
            raise UnsupportedTTIR("block program: more than 24 block values alive")
        if len(out) > rt.TSB_MAX_OPS or len(self.accs) > rt.TSB_MAX_ACCESSES:
            raise UnsupportedTTIR(f"block program: {len(out)} ops or {len(self.accs)} accesses exceed {rt.TSB_MAX_OPS} / {rt.TSB_MAX_ACCESSES}")
        words = sum(int(np.prod([self.space[d] for d in range(len(self.space)) if m & (1 << d)])) for m in masks)
        if words * 4 > 200 * 1024:
            raise UnsupportedTTIR(f"block program: {words * 4} bytes of block values exceed the 200 KB on-chip budget")
        return out, masks


class BlockProgramPlan(Plan):
    """Loop-free bodies with tt.reduce along block axes: one CTA per program, values in shared memory."""
    family = "block_program"

    @staticmethod
    def build(kernel: Kernel, an: Analyzer) -> "BlockProgramPlan":
        stores: List[Access] = []

        def collect(effects):
            for kind, e in effects:
                if kind == "store":
                    stores.append(e)
                else:
                    collect(e.effects)
        collect(kernel.effects)
        if not stores:
            raise UnsupportedTTIR("kernel stores nothing")
        sizes, maps, red_pos = _discover_space(stores, kernel.loops)
        if not sizes:
            sizes = [1]
        if len(sizes) > rt.TSB_MAX_RANK:
            raise UnsupportedTTIR(f"block program: iteration space of rank {len(sizes)}")
        low = _BpLowering(kernel, an, sizes, red_pos)
        ops, masks = low.lower(kernel.effects, maps, kernel.loops)
        return BlockProgramPlan(kernel.name, {"seg": {"space": list(sizes), "accs": low.accs, "ops": ops,
                                                      "loops": sorted(low.loop_trips),
                                                      "loop_depth": {str(k): v for k, v in low.loop_depth.items()}},
                                              "reg_masks": masks, "trips": {str(k): v for k, v in low.loop_trips.items()}})

    def launch(self, args, grid, pid_lo, pid_hi, stream):
        def compute():
            env = LaunchEnv(args.scalars, grid)
            for lid in self.p["seg"].get("loops", []):
                env.base[("it", lid)] = 0
            accs, ops, arg_of = ElementwisePlan._evaluate(self, self.p["seg"], args, env, self.p.get("trips"))
            masks = (ctypes.c_int32 * len(self.p["reg_masks"]))(*self.p["reg_masks"])
            return accs, ops, arg_of, masks
        accs, ops, arg_of, masks = self.memo(args, grid, compute)
        for a, i in zip(accs, arg_of):
            if i is not None:
                a.base = args.pointer(i)
        g = (ctypes.c_int32 * 3)(*grid)
        rc = rt.lib().tsb_block_program(accs, len(accs), ops, len(ops), masks, len(masks), g, pid_lo, pid_hi, stream)
        if rc:
            rt.check(rc, f"tsb_block_program[{self.name}]")


# --------------------------------------------------------------------------
# row softmax

def _row_access(acc: Access, what: str):
    """Checks a 1-D unit-stride row access whose offset is row*stride + const; returns (stride Poly per pid0, mask)."""
    if len(acc.shape) != 1 or acc.wrapped:
        raise UnsupportedTTIR(f"{what}: not a 1-D block")
    if acc.strides[0] != Poly.const(1):
        raise UnsupportedTTIR(f"{what}: row is not unit-stride")
    if not is_affine_in_pid(acc.offset):
        raise UnsupportedTTIR(f"{what}: offset not affine in program_id")


def _single_bound(mask: Optional[TMask], d: int):
    if mask is None or not mask.dims[d]:
        return None
    if len(mask.dims[d]) != 1 or mask.scalar_conds:
        raise UnsupportedTTIR("compound mask on a row access")
    return mask.dims[d][0]


class SoftmaxPlan(Plan):
    family = "softmax"

    @staticmethod
    def build(kernel: Kernel, an: Analyzer) -> "SoftmaxPlan":
        if len(kernel.effects) != 1 or kernel.effects[0][0] != "store":
            raise UnsupportedTTIR("softmax family: expects exactly one store")
        st: Access = kernel.effects[0][1]
        b: Dict[str, Node] = {}
        num = ("op", "exp", ("op", "subf", ("$", "x"), ("splat", ("reduce", "maxnumf", 0, ("$", "x")))))
        num_alt = ("op", "exp", ("op", "subf", ("$", "x"), ("splat", ("reduce", "maximumf", 0, ("$", "x")))))
        ok = False
        for nm in (num, num_alt):
            b = {}
            if match(st.value, ("op", "divf", nm, ("splat", ("reduce", "addf", 0, nm))), b):
                ok = True
                break
        if not ok or b["x"].op != "load":
            raise UnsupportedTTIR("softmax family: body is not exp(x-max(x))/sum(exp(x-max(x)))")
        ld = an.access_of(b["x"])
        _row_access(ld, "softmax load")
        _row_access(st, "softmax store")
        if ld.elem != "f32" or st.elem != "f32":
            raise UnsupportedTTIR("softmax family: only fp32 rows")
        lb, sb = _single_bound(ld.mask, 0), _single_bound(st.mask, 0)
        block = ld.shape[0]
        if lb is not None:
            if not lb[0].is_zero:
                raise UnsupportedTTIR("softmax family: column mask does not start at 0")
            ob = other_bits(ld.other, "f32") if ld.other is not None else None
            if ob != 0xff800000:
                raise UnsupportedTTIR("softmax family: masked row load needs other=-inf")
        if (lb is None) != (sb is None) or (lb is not None and (lb[1] != sb[1] or not sb[0].is_zero)):
            raise UnsupportedTTIR("softmax family: load and store masks differ")
        n_cols = lb[1] if lb is not None else Poly.const(block)
        if n_cols.depends_on(("pid",)):
            raise UnsupportedTTIR("softmax family: n_cols depends on program_id")
        return SoftmaxPlan(kernel.name, {"in_arg": ld.arg, "out_arg": st.arg, "in_off": ld.offset,
                                         "out_off": st.offset, "n_cols": n_cols, "block": block})

    def _resolve(self, args, grid):
        p = self.p
        env = LaunchEnv(args.scalars, grid)
        i0, iinc = env.affine_pid(p["in_off"])
        o0, oinc = env.affine_pid(p["out_off"])
        if any(iinc[1:]) or any(oinc[1:]) or grid[1] * grid[2] != 1:
            raise UnsupportedTTIR("softmax family: rows must be indexed by program_id(0) only")
        return i0, iinc[0], o0, oinc[0], int(p["n_cols"].evaluate(env.at()))

    def launch(self, args, grid, pid_lo, pid_hi, stream):
        p = self.p
        i0, istride, o0, ostride, n_cols = self.memo(args, grid, lambda: self._resolve(args, grid))
        rc = rt.lib().tsb_softmax_rows(args.pointer(p["in_arg"]) + 4 * i0, args.pointer(p["out_arg"]) + 4 * o0,
                                       rt.DTYPES["f32"], istride, ostride, n_cols, p["block"], pid_lo, pid_hi, stream)
        if rc:
            rt.check(rc, f"tsb_softmax_rows[{self.name}]")


# --------------------------------------------------------------------------
# LayerNorm forward

class LayerNormPlan(Plan):
    family = "layernorm"

    @staticmethod
    def build(kernel: Kernel, an: Analyzer) -> "LayerNormPlan":
        eff = kernel.effects
        loops = [e for k, e in eff if k == "loop"]
        stores = [e for k, e in eff if k == "store"]
        if len(loops) != 3 or len(stores) > 2:
            raise UnsupportedTTIR("layernorm family: expects three loops and at most two scalar stores")
        l1, l2, l3 = loops
        if l1.effects or l2.effects or len(l3.effects) != 1 or l3.effects[0][0] != "store":
            raise UnsupportedTTIR("layernorm family: loop structure differs")
        for l in loops:
            if not l.lb.is_zero or l.ub != l1.ub or l.step != l1.step or not l.step.is_const:
                raise UnsupportedTTIR("layernorm family: loops must all run 0..N step BLOCK")
        if len(l1.yields) != 1 or len(l2.yields) != 1 or l3.yields:
            raise UnsupportedTTIR("layernorm family: unexpected loop-carried values")
        ysto: Access = l3.effects[0][1]
        b: Dict[str, Node] = {}
        it1 = ("attrs", ("$", "acc1"), {"loop": l1.id, "k": 0})
        if not match(l1.yields[0].node, ("op", "addf", it1, ("ext", ("$", "x1"))), b) or b["acc1"].op != "iter_arg":
            raise UnsupportedTTIR("layernorm family: first loop is not a lane-accumulated sum of x")
        sum1 = ("reduce", "addf", 0, ("attrs", ("$", "r1"), {"loop": l1.id, "k": 0}))
        mean = ("op", "divf", sum1, ("$", "nf"))
        d = ("op", "select", ("$", "mask2"), ("op", "subf", ("ext", ("$", "x2")), ("splat", mean)), ("const", 0.0))
        it2 = ("attrs", ("$", "acc2"), {"loop": l2.id, "k": 0})
        if not match(l2.yields[0].node, ("op", "addf", it2, ("op", "mulf", d, d)), b):
            raise UnsupportedTTIR("layernorm family: second loop is not a lane-accumulated sum of (x-mean)^2")
        var = ("op", "divf", ("reduce", "addf", 0, ("attrs", ("$", "r2"), {"loop": l2.id, "k": 0})), ("$", "nf"))
        rstd = ("op", "divf", ("const", 1.0), ("op", "sqrt", ("op", "addf", var, ("$", "eps"))))
        yv = ("trunc", ("op", "addf", ("op", "mulf", ("op", "mulf", ("op", "subf", ("ext", ("$", "x3")), ("splat", mean)),
                                                      ("splat", rstd)), ("ext", ("$", "w"))), ("ext", ("$", "bias"))))
        if not match(ysto.value, yv, b):
            raise UnsupportedTTIR("layernorm family: third loop is not ((x-mean)*rstd)*w+b")
        for k in ("r1", "r2"):
            if b[k].op != "loop_result":
                raise UnsupportedTTIR("layernorm family: reductions do not consume the loop results")
        if b["mask2"].op != "maskval" or b["eps"].op != "farg":
            raise UnsupportedTTIR("layernorm family: unexpected select mask or eps")
        nf = b["nf"]
        if not (nf.op == "cast" and nf.args[0].op == "sint"):
            raise UnsupportedTTIR("layernorm family: divisor is not float(N)")
        n_poly = nf.args[0].attr("poly")
        if n_poly != l1.ub:
            raise UnsupportedTTIR("layernorm family: divisor differs from the loop bound")
        for k in ("x1", "x2", "x3", "w", "bias"):
            if b[k].op != "load":
                raise UnsupportedTTIR("layernorm family: operand is not a block load")
        x1, x2, x3, w, bias = (an.access_of(b[k]) for k in ("x1", "x2", "x3", "w", "bias"))
        block = l1.step.as_const
        it_atoms = {l.id: Poly.atom(("it", l.id)) for l in loops}
        # every x load reads row*stride + iv + lane with mask iv + lane < N and other = 0
        base_off = None
        for acc, l in ((x1, l1), (x2, l2), (x3, l3)):
            _row_access(acc, "layernorm x")
            off = acc.offset - l.step * it_atoms[l.id]
            if off.depends_on(("it", "carry")) or acc.shape != (block,):
                raise UnsupportedTTIR("layernorm family: x offset is not row base + loop offset")
            if base_off is None:
                base_off = off
            if off != base_off or acc.arg != x1.arg or acc.elem != x1.elem:
                raise UnsupportedTTIR("layernorm family: the three x loads differ")
            mb = _single_bound(acc.mask, 0)
            if mb is None or mb[0] != l.step * it_atoms[l.id] or mb[1] != n_poly:
                raise UnsupportedTTIR("layernorm family: x mask is not offs < N")
            if other_bits(acc.other, acc.elem) != 0:
                raise UnsupportedTTIR("layernorm family: x loads need other=0")
        for acc in (w, bias):
            _row_access(acc, "layernorm weight/bias")
            if acc.offset != l3.step * it_atoms[l3.id] or acc.elem != x1.elem:
                raise UnsupportedTTIR("layernorm family: weight/bias are not indexed by column only")
        _row_access(ysto, "layernorm y")
        yoff = ysto.offset - l3.step * it_atoms[l3.id]
        if yoff.depends_on(("it", "carry")) or ysto.elem != x1.elem:
            raise UnsupportedTTIR("layernorm family: y offset is not row base + loop offset")
        mean_arg = rstd_arg = None
        mean_off = rstd_off = None
        for s in stores:
            bb = dict(b)
            if s.shape != () or s.elem != "f32":
                raise UnsupportedTTIR("layernorm family: unexpected extra store")
            if match(s.value, mean, bb):
                mean_arg, mean_off = s.arg, s.offset
            elif match(s.value, rstd, bb):
                rstd_arg, rstd_off = s.arg, s.offset
            else:
                raise UnsupportedTTIR("layernorm family: extra store is neither mean nor rstd")
        return LayerNormPlan(kernel.name, {
            "x": x1.arg, "y": ysto.arg, "w": w.arg, "b": bias.arg, "mean": mean_arg, "rstd": rstd_arg,
            "x_off": base_off, "y_off": yoff, "mean_off": mean_off, "rstd_off": rstd_off, "n": n_poly,
            "eps_arg": b["eps"].attr("arg"), "elem": x1.elem})

    def _resolve(self, args, grid):
        p = self.p
        env = LaunchEnv(args.scalars, grid)
        x0, xinc = env.affine_pid(p["x_off"])
        y0, yinc = env.affine_pid(p["y_off"])
        if any(xinc[1:]) or any(yinc[1:]) or grid[1] * grid[2] != 1:
            raise UnsupportedTTIR("layernorm family: rows must be indexed by program_id(0) only")
        offs = {}
        for key in ("mean", "rstd"):
            if p[key] is not None:
                o0, oinc = env.affine_pid(p[key + "_off"])
                if grid[0] > 1 and oinc[0] != 1:
                    raise UnsupportedTTIR("layernorm family: mean/rstd must be stored at index row")
                offs[key] = o0
        return x0, xinc[0], y0, yinc[0], offs, int(p["n"].evaluate(env.at()))

    def launch(self, args, grid, pid_lo, pid_hi, stream):
        p = self.p
        x0, xs, y0, ys, offs, n = self.memo(args, grid, lambda: self._resolve(args, grid))
        es = rt.DTYPE_SIZE[p["elem"]]
        mean_p = args.pointer(p["mean"]) + 4 * offs["mean"] if "mean" in offs else None
        rstd_p = args.pointer(p["rstd"]) + 4 * offs["rstd"] if "rstd" in offs else None
        rc = rt.lib().tsb_layernorm_fwd(args.pointer(p["x"]) + es * x0, args.pointer(p["y"]) + es * y0,
                                        args.pointer(p["w"]), args.pointer(p["b"]), mean_p, rstd_p,
                                        rt.DTYPES[p["elem"]], xs, ys, n,
                                        float(args.floats[p["eps_arg"]]), pid_lo, pid_hi, stream)
        if rc:
            rt.check(rc, f"tsb_layernorm_fwd[{self.name}]")


# --------------------------------------------------------------------------
# strided 2-D reduction along one axis, and the full sum

class ReduceRowsPlan(Plan):
    family = "reduce_rows"

    @staticmethod
    def build(kernel: Kernel, an: Analyzer) -> "ReduceRowsPlan":
        eff = kernel.effects
        if len(eff) != 2 or eff[0][0] != "loop" or eff[1][0] != "store":
            raise UnsupportedTTIR("reduce_rows family: expects one loop followed by one store")
        loop: Loop = eff[0][1]
        st: Access = eff[1][1]
        if loop.effects or len(loop.yields) != 1 or not loop.lb.is_zero or not loop.step.is_const:
            raise UnsupportedTTIR("reduce_rows family: loop shape differs")
        b: Dict[str, Node] = {}
        it = ("attrs", ("$", "acc"), {"loop": loop.id, "k": 0})
        if not match(loop.yields[0].node, ("op", "addf", it, ("reduce", "addf", None, ("$", "x"))), b):
            raise UnsupportedTTIR("reduce_rows family: loop body is not acc += sum(block, axis)")
        if b["acc"].op != "iter_arg" or b["x"].op != "load" or const_value(loop.inits[0].node) != 0.0:
            raise UnsupportedTTIR("reduce_rows family: accumulator is not a zero-initialised loop-carried block")
        rb: Dict[str, Node] = {}
        if not match(st.value, ("attrs", ("$", "r"), {"loop": loop.id, "k": 0}), rb) or rb["r"].op != "loop_result":
            raise UnsupportedTTIR("reduce_rows family: store does not write the accumulated sums")
        red = loop.yields[0].node.args[1] if loop.yields[0].node.args[1].op == "reduce" else loop.yields[0].node.args[0]
        axis = red.attr("axis")
        ld = an.access_of(b["x"])
        if len(ld.shape) != 2 or ld.wrapped or ld.elem != "f32" or st.elem != "f32":
            raise UnsupportedTTIR("reduce_rows family: expects a 2-D fp32 block load")
        keep = 1 - axis
        itp = Poly.atom(("it", loop.id))
        # offset = rows0(pid)*stride_keep + (step*it)*stride_red
        off = ld.offset - loop.step * itp * ld.strides[axis]
        if off.depends_on(("it", "carry")) or not is_affine_in_pid(off):
            raise UnsupportedTTIR("reduce_rows family: block offset is not row block + loop offset")
        mk, mr = _single_bound(ld.mask, keep), _single_bound(ld.mask, axis)
        if mr is None or mr[0] != loop.step * itp:
            raise UnsupportedTTIR("reduce_rows family: the reduced dim needs a mask col < N starting at the loop offset")
        if other_bits(ld.other, "f32") != 0:
            raise UnsupportedTTIR("reduce_rows family: masked load needs other=0")
        if len(st.shape) != 1 or st.strides[0] != Poly.const(1) or st.shape[0] != ld.shape[keep]:
            raise UnsupportedTTIR("reduce_rows family: store is not a unit-stride 1-D block of row sums")
        sm = _single_bound(st.mask, 0)
        if (mk is None) != (sm is None) or (mk is not None and (mk[0] != sm[0] or mk[1] != sm[1])):
            raise UnsupportedTTIR("reduce_rows family: row masks of load and store differ")
        if mk is not None and st.offset - mk[0] != Poly.const(0) and (st.offset - mk[0]).depends_on(("pid",)):
            raise UnsupportedTTIR("reduce_rows family: store offset does not follow the row index")
        return ReduceRowsPlan(kernel.name, {
            "x": ld.arg, "out": st.arg, "block_rows": ld.shape[keep], "stride_keep": ld.strides[keep],
            "stride_red": ld.strides[axis], "x_off": off, "out_off": st.offset,
            # columns the loop reaches: whole blocks, so a bound beyond `ub` still admits the last partial block
            "n_valid": Poly.fn("minsi", mr[1], loop.trip * loop.step), "row_start": mk[0] if mk is not None else None,
            "row_bound": mk[1] if mk is not None else None})

    def __init__(self, name, params):
        super().__init__(name, params)
        self._scratch = None

    def launch(self, args, grid, pid_lo, pid_hi, stream):
        p = self.p
        env = LaunchEnv(args.scalars, grid)
        if grid[1] * grid[2] != 1:
            raise UnsupportedTTIR("reduce_rows family: expects a 1-D grid")
        bm = p["block_rows"]
        sk = int(p["stride_keep"].evaluate(env.at()))
        sr = int(p["stride_red"].evaluate(env.at()))
        x0, xinc = env.affine_pid(p["x_off"])
        o0, oinc = env.affine_pid(p["out_off"])
        if xinc[0] != bm * sk or oinc[0] != bm:
            raise UnsupportedTTIR("reduce_rows family: programs do not tile the rows contiguously")
        n_valid = max(int(p["n_valid"].evaluate(env.at())), 0)
        total_rows = grid[0] * bm
        if p["row_bound"] is not None:
            s0, sinc = env.affine_pid(p["row_start"])
            if s0 != 0 or sinc[0] != bm:
                raise UnsupportedTTIR("reduce_rows family: row mask does not start at pid*BLOCK")
            total_rows = min(total_rows, int(p["row_bound"].evaluate(env.at())))
        row_lo, row_hi = min(pid_lo * bm, total_rows), min(pid_hi * bm, total_rows)
        if row_hi <= row_lo:
            return
        need = rt.lib().tsb_reduce_rows_scratch_bytes(row_hi - row_lo, n_valid, sk, sr)
        scratch = args.scratch(need, stream) if need > 0 else None
        rc = rt.lib().tsb_reduce_rows(args.pointer(p["x"]) + 4 * x0, args.pointer(p["out"]) + 4 * o0, sk, sr, 1,
                                      n_valid, row_lo, row_hi, scratch, stream)
        rt.check(rc, f"tsb_reduce_rows[{self.name}]")


class ReduceAllPlan(Plan):
    family = "reduce_all"

    @staticmethod
    def build(kernel: Kernel, an: Analyzer) -> "ReduceAllPlan":
        eff = kernel.effects
        if len(eff) != 2 or eff[0][0] != "loop" or eff[1][0] != "store":
            raise UnsupportedTTIR("reduce_all family: expects one loop followed by one store")
        loop: Loop = eff[0][1]
        st: Access = eff[1][1]
        if st.shape != () or st.elem != "f32" or loop.effects or len(loop.yields) != 1 or not loop.lb.is_zero:
            raise UnsupportedTTIR("reduce_all family: shape differs")
        b: Dict[str, Node] = {}
        it = ("attrs", ("$", "acc"), {"loop": loop.id, "k": 0})
        if not match(loop.yields[0].node, ("op", "addf", it, ("$", "x")), b) or b["x"].op != "load" \
                or b["acc"].op != "iter_arg" or const_value(loop.inits[0].node) != 0.0:
            raise UnsupportedTTIR("reduce_all family: loop body is not acc += block")
        rb: Dict[str, Node] = {}
        if not match(st.value, ("reduce", "addf", 0, ("attrs", ("$", "r"), {"loop": loop.id, "k": 0})), rb):
            raise UnsupportedTTIR("reduce_all family: store is not sum(acc)")
        ld = an.access_of(b["x"])
        itp = Poly.atom(("it", loop.id))
        if len(ld.shape) != 1 or ld.elem != "f32" or ld.wrapped:
            raise UnsupportedTTIR("reduce_all family: expects a 1-D fp32 block load")
        off = ld.offset - loop.step * itp * ld.strides[0]
        m = _single_bound(ld.mask, 0)
        if off.depends_on(("it", "carry", "pid")) or st.offset.depends_on(("pid",)):
            raise UnsupportedTTIR("reduce_all family: offsets depend on the loop or the program")
        if m is None or m[0] != loop.step * itp or other_bits(ld.other, "f32") != 0:
            raise UnsupportedTTIR("reduce_all family: load needs mask offs < n and other=0")
        return ReduceAllPlan(kernel.name, {"x": ld.arg, "out": st.arg, "x_off": off, "out_off": st.offset,
                                           "stride": ld.strides[0], "n": Poly.fn("minsi", m[1], loop.trip * loop.step)})

    def launch(self, args, grid, pid_lo, pid_hi, stream):
        p = self.p
        if pid_hi <= pid_lo:
            return
        env = LaunchEnv(args.scalars, grid).at()
        n = max(int(p["n"].evaluate(env)), 0)
        rc = rt.lib().tsb_reduce_all(args.pointer(p["x"]) + 4 * int(p["x_off"].evaluate(env)),
                                     args.pointer(p["out"]) + 4 * int(p["out_off"].evaluate(env)), n,
                                     int(p["stride"].evaluate(env)), stream)
        rt.check(rc, f"tsb_reduce_all[{self.name}]")


# --------------------------------------------------------------------------
# tt.dot

class GemmPlan(Plan):
    family = "gemm"

    @staticmethod
    def build(kernel: Kernel, an: Analyzer) -> "GemmPlan":
        eff = kernel.effects
        if len(eff) != 2 or eff[0][0] != "loop" or eff[1][0] != "store":
            raise UnsupportedTTIR("gemm family: expects one K loop followed by one store")
        loop: Loop = eff[0][1]
        st: Access = eff[1][1]
        if loop.effects:
            raise UnsupportedTTIR("gemm family: stores inside the K loop")
        acc_k = None
        b: Dict[str, Node] = {}
        for k, y in enumerate(loop.yields):
            if isinstance(y, TData) and y.node.op == "dot":
                bb: Dict[str, Node] = {}
                if match(y.node, ("op", "dot", ("$", "a"), ("$", "b"), ("attrs", ("$", "acc"), {"loop": loop.id, "k": k})), bb) \
                        and bb["acc"].op == "iter_arg":
                    acc_k, b = k, bb
        if acc_k is None or b["a"].op != "load" or b["b"].op != "load":
            raise UnsupportedTTIR("gemm family: loop body is not acc = dot(load, load, acc)")
        if const_value(loop.inits[acc_k].node) != 0.0:
            raise UnsupportedTTIR("gemm family: accumulator does not start at zero")
        rb: Dict[str, Node] = {}
        res = ("attrs", ("$", "r"), {"loop": loop.id, "k": acc_k})
        tail = None
        if not match(st.value, ("trunc", res), rb) or rb["r"].op != "loop_result":
            # a peeled last K step after the loop: acc = dot(load, load, loop result), masked along K
            rb = {}
            if not match(st.value, ("trunc", ("op", "dot", ("$", "a2"), ("$", "b2"), res)), rb) or rb["r"].op != "loop_result" \
                    or rb["a2"].op != "load" or rb["b2"].op != "load":
                raise UnsupportedTTIR("gemm family: store does not write the (truncated) accumulator")
            tail = (an.access_of(rb["a2"]), an.access_of(rb["b2"]))
        A, B = an.access_of(b["a"]), an.access_of(b["b"])
        if A.elem not in ("f16", "bf16", "f32") or B.elem != A.elem or st.elem != A.elem:
            raise UnsupportedTTIR("gemm family: operands and result must all be f16, all bf16 or all f32")
        if len(A.shape) != 2 or len(B.shape) != 2 or len(st.shape) != 2 or A.shape[1] != B.shape[0] \
                or st.shape != (A.shape[0], B.shape[1]):
            raise UnsupportedTTIR("gemm family: block shapes do not form a matmul")
        BM, BK = A.shape
        BN = B.shape[1]
        itp = Poly.atom(("it", loop.id))

        def split(acc: Access, kdim: int, what: str):
            """-> (tile offset Poly (it = 0), k advance per iteration Poly, wrapped on the non-K dim or None)"""
            if len(acc.wrapped) > 1 or (acc.wrapped and acc.wrapped[0].dim == kdim):
                raise UnsupportedTTIR(f"gemm family: {what} wraps along K or along both dims")
            # offset is linear in `it`: offset = base + it * adv
            terms_it = {m: c for m, c in acc.offset.terms.items() if ("it", loop.id) in m}
            adv = Poly({tuple(a for a in m if a != ("it", loop.id)): c for m, c in terms_it.items()
                        if m.count(("it", loop.id)) == 1})
            base = acc.offset - adv * itp
            if base.depends_on(("it", "carry")) or adv.depends_on(("it", "carry", "pid")):
                raise UnsupportedTTIR(f"gemm family: {what} offset is not tile base + it * step")
            return base, adv, (acc.wrapped[0] if acc.wrapped else None)

        a_base, a_adv, a_wrap = split(A, 1, "A")
        b_base, b_adv, b_wrap = split(B, 0, "B")
        mka = _single_bound(A.mask, 1)
        mkb = _single_bound(B.mask, 0)
        for m, what in ((mka, "A"), (mkb, "B")):
            if m is not None and other_bits((A if what == "A" else B).other, A.elem) != 0:
                raise UnsupportedTTIR(f"gemm family: masked {what} load needs other=0")
        params = {
            "a": A.arg, "b": B.arg, "c": st.arg, "elem": A.elem, "BM": BM, "BN": BN, "BK": BK,
            "a_base": a_base, "a_adv": a_adv, "b_base": b_base, "b_adv": b_adv,
            "sam": a_wrap.scale * a_wrap.inner_stride if a_wrap else A.strides[0], "sak": A.strides[1],
            "sbk": B.strides[0], "sbn": b_wrap.scale * b_wrap.inner_stride if b_wrap else B.strides[1],
            "scm": st.strides[0], "scn": st.strides[1], "c_off": st.offset,
            "trip": loop.trip, "loop": loop.id,
            # K mask: lanes k with start + k < bound (evaluated at it = 0 gives K itself)
            "ka": list(mka) if mka else None, "kb": list(mkb) if mkb else None,
            "am": list(_single_bound(A.mask, 0)) if _single_bound(A.mask, 0) else None,
            "bn": list(_single_bound(B.mask, 1)) if _single_bound(B.mask, 1) else None,
            "cm": list(_single_bound(st.mask, 0)) if _single_bound(st.mask, 0) else None,
            "cn": list(_single_bound(st.mask, 1)) if _single_bound(st.mask, 1) else None,
            "a_wrap": [a_wrap.inner_offset, a_wrap.inner_stride, a_wrap.modulus, a_wrap.scale] if a_wrap else None,
            "b_wrap": [b_wrap.inner_offset, b_wrap.inner_stride, b_wrap.modulus, b_wrap.scale] if b_wrap else None,
        }
        if st.wrapped:
            raise UnsupportedTTIR("gemm family: wrap-around store")
        if tail is not None:
            A2, B2 = tail
            if A2.arg != A.arg or B2.arg != B.arg or A2.shape != A.shape or B2.shape != B.shape or \
                    A2.strides != A.strides or B2.strides != B.strides or A2.wrapped != A.wrapped or B2.wrapped != B.wrapped:
                raise UnsupportedTTIR("gemm family: the peeled K step addresses other blocks than the loop")
            ka2, kb2 = _single_bound(A2.mask, 1), _single_bound(B2.mask, 0)
            if ka2 is None or kb2 is None or other_bits(A2.other, A.elem) != 0 or other_bits(B2.other, A.elem) != 0:
                raise UnsupportedTTIR("gemm family: the peeled K step needs K masks with other=0")
            if mka is not None or mkb is not None:
                raise UnsupportedTTIR("gemm family: K masks both in the loop and in a peeled step")
            params["tail"] = {"a_off": A2.offset, "b_off": B2.offset, "ka": list(ka2), "kb": list(kb2)}
        return GemmPlan(kernel.name, params)

    def __init__(self, name, params):
        super().__init__(name, params)
        self._cache = {}

    def resolve(self, args, grid):
        """Evaluate the plan for concrete scalars: problem sizes, strides and the pid -> tile table."""
        p = self.p
        env = LaunchEnv(args.scalars, grid)
        env.base[("it", p["loop"])] = 0  # masks and offsets are read at the first K step
        e0 = env.at()
        ev = lambda q: int(q.evaluate(e0))
        BM, BN, BK = p["BM"], p["BN"], p["BK"]
        sam, sak, sbk, sbn, scm, scn = (ev(p[k]) for k in ("sam", "sak", "sbk", "sbn", "scm", "scn"))
        trip = ev(p["trip"])
        # K
        K = None
        for key in ("ka", "kb"):
            if p[key] is not None:
                k_here = ev(p[key][1]) - ev(p[key][0])
                if K is not None and K != k_here:
                    raise UnsupportedTTIR("gemm family: A and B K-masks disagree")
                K = k_here
        tail = p.get("tail")
        if tail is not None:
            # loop of `trip` full steps plus one masked step: the same product with K taken from the tail mask
            ks = ev(tail["ka"][0])
            if ks != trip * BK or ev(tail["kb"][0]) != ks or ev(tail["kb"][1]) != ev(tail["ka"][1]):
                raise UnsupportedTTIR("gemm family: the peeled K step does not continue where the loop ends")
            K = ev(tail["ka"][1])
            if not (ks < K <= ks + BK):
                raise UnsupportedTTIR(f"gemm family: peeled K step covers [{ks}, {K}) which is not one block")
            trip += 1
        if K is None:
            K = trip * BK
        if trip != -(-K // BK) and not (K <= 0 and trip == 0):
            raise UnsupportedTTIR(f"gemm family: loop runs {trip} steps but K={K}, BLOCK_K={BK}")
        if ev(p["a_adv"]) != BK * sak or ev(p["b_adv"]) != BK * sbk:
            raise UnsupportedTTIR("gemm family: pointers do not advance by BLOCK_K per iteration")
        # tiles per program, from every program's offsets
        ea = env.all_pids()
        n_prog = grid[0] * grid[1] * grid[2]
        full = lambda q: np.broadcast_to(np.asarray(q.evaluate(ea), dtype=np.int64), (n_prog,))
        c_off = full(p["c_off"])
        if p["cm"] is not None:
            row0 = full(p["cm"][0])
            M = ev(p["cm"][1])
        elif p["a_wrap"] is not None:
            row0 = full(p["a_wrap"][0])
            M = None
        else:
            if sam == 0:
                raise UnsupportedTTIR("gemm family: cannot derive tile rows (stride_am == 0)")
            row0 = full(p["a_base"]) // sam
            M = None
        if p["cn"] is not None:
            col0 = full(p["cn"][0])
            N = ev(p["cn"][1])
        elif p["b_wrap"] is not None:
            col0 = full(p["b_wrap"][0])
            N = None
        else:
            if sbn == 0:
                raise UnsupportedTTIR("gemm family: cannot derive tile columns (stride_bn == 0)")
            col0 = full(p["b_base"]) // sbn
            N = None
        if np.any(row0 % BM) or np.any(col0 % BN) or np.any(row0 < 0) or np.any(col0 < 0):
            raise UnsupportedTTIR("gemm family: tiles are not aligned to the block shape")
        if M is None:
            M = int(row0.max()) + BM if n_prog else 0
        if N is None:
            N = int(col0.max()) + BN if n_prog else 0
        if np.any(c_off != row0 * scm + col0 * scn):
            raise UnsupportedTTIR("gemm family: store offsets do not match the tile indices")
        # operand offsets must address the same tiles (a wrap modulo M/N only changes rows the
        # store mask discards, which requires the modulus to equal the store bound)
        if p["a_wrap"] is not None:
            w = p["a_wrap"]
            if ev(w[2]) != M or ev(w[1]) != 1 or ev(w[3]) != sam or np.any(full(w[0]) != row0) or np.any(full(p["a_base"]) != 0):
                raise UnsupportedTTIR("gemm family: A row wrap-around is not `% M` of the tile rows")
        elif np.any(full(p["a_base"]) != row0 * sam):
            raise UnsupportedTTIR("gemm family: A offsets do not match the tile rows")
        if p["b_wrap"] is not None:
            w = p["b_wrap"]
            if ev(w[2]) != N or ev(w[1]) != 1 or ev(w[3]) != sbn or np.any(full(w[0]) != col0) or np.any(full(p["b_base"]) != 0):
                raise UnsupportedTTIR("gemm family: B column wrap-around is not `% N` of the tile columns")
        elif np.any(full(p["b_base"]) != col0 * sbn):
            raise UnsupportedTTIR("gemm family: B offsets do not match the tile columns")
        for key, lim, what in (("am", M, "A rows"), ("bn", N, "B columns")):
            if p[key] is not None and ev(p[key][1]) != lim:
                raise UnsupportedTTIR(f"gemm family: mask bound of {what} differs from the store bound")
        if tail is not None:
            steps = ev(p["trip"])
            if np.any(full(tail["a_off"]) != full(p["a_base"]) + steps * ev(p["a_adv"])) or \
                    np.any(full(tail["b_off"]) != full(p["b_base"]) + steps * ev(p["b_adv"])):
                raise UnsupportedTTIR("gemm family: the peeled K step does not address the next K block")
        unmasked_rows = p["am"] is None and p["a_wrap"] is None and p["cm"] is None
        tiles = np.stack([row0 // BM, col0 // BN], axis=1).astype(np.int32)
        return dict(M=M, N=N, K=K, sam=sam, sak=sak, sbk=sbk, sbn=sbn, scm=scm, scn=scn, tiles=tiles,
                    n_prog=n_prog, unmasked_rows=unmasked_rows)

    @staticmethod
    def pair_tiles(tiles: np.ndarray):
        """Split a list of (tile_m, tile_n) into vertically adjacent pairs (even tile_m first) and the rest."""
        index = {(int(tm), int(tn)): i for i, (tm, tn) in enumerate(tiles)}
        used = np.zeros(len(tiles), dtype=bool)
        pairs = []
        for i, (tm, tn) in enumerate(tiles):
            j = index.get((int(tm) + 1, int(tn)))
            if tm % 2 == 0 and j is not None:
                pairs.append((int(tm), int(tn)))
                used[i] = used[j] = True
        singles = tiles[~used]
        return np.asarray(pairs, dtype=np.int32).reshape(-1, 2), np.ascontiguousarray(singles, dtype=np.int32)

    def launch(self, args, grid, pid_lo, pid_hi, stream):
        p = self.p
        key = tuple(sorted(args.scalars.items())) + tuple(grid)
        r = self._cache.get(key)
        if r is None:
            r = self.resolve(args, grid)
            if len(self._cache) > 16:
                self._cache.clear()
            self._cache[key] = r
        status = args.status_word(stream)
        common = (args.pointer(p["a"]), args.pointer(p["b"]), args.pointer(p["c"]), rt.DTYPES[p["elem"]],
                  r["M"], r["N"], r["K"], r["sam"], r["sak"], r["sbk"], r["sbn"], r["scm"], r["scn"],
                  p["BM"], p["BN"], p["BK"])
        L = rt.lib()
        if p["BM"] == 128 and r["K"] > 0 and not r.get("no_pairs"):
            # two-CTA form for every pair of vertically adjacent tiles in the range, one-CTA form for the rest
            pk = ("split", pid_lo, pid_hi)
            sp = r.get(pk)
            if sp is None:
                pr, sg = self.pair_tiles(r["tiles"][pid_lo:pid_hi])
                sp = r[pk] = (pr, sg, _digest(pr), _digest(sg))
            pairs, singles, key_pairs, key_singles = sp
            if len(pairs):
                dev = args.device_table(("gemm_pairs", key_pairs), pairs, stream)
                rc = L.tsb_gemm_paired(*common, dev, len(pairs), status, stream)
                if rc == -2:
                    r["no_pairs"] = True  # operands not eligible: the one-CTA entry decides (tensor or SIMT)
                else:
                    if rc:
                        rt.check(rc, f"tsb_gemm_paired[{self.name}]")
                    if len(singles):
                        dev1 = args.device_table(("gemm_singles", key_singles), singles, stream)
                        rc = L.tsb_gemm(*common, dev1, len(singles), 0, len(singles), status, stream)
                        if rc:
                            rt.check(rc, f"tsb_gemm[{self.name}]")
                    return
        if "tiles_key" not in r:
            r["tiles_key"] = _digest(r["tiles"])
        tiles_dev = args.device_table(("gemm_tiles", r["tiles_key"]), r["tiles"], stream)
        rc = L.tsb_gemm(*common, tiles_dev, r["n_prog"], pid_lo, pid_hi, status, stream)
        if rc:
            rt.check(rc, f"tsb_gemm[{self.name}]")


def _digest(table: np.ndarray):
    """Key of a device-resident table: its shape and content (two plans, or two specialisations of
    one kernel, share a table only when they would upload the same bytes)."""
    import hashlib
    a = np.ascontiguousarray(table)
    return (a.shape, hashlib.sha1(a.tobytes()).digest())


_FAMILIES = {c.family: c for c in (GemmPlan, LayerNormPlan, SoftmaxPlan, ReduceRowsPlan, ReduceAllPlan,
                                   ElementwisePlan, BlockProgramPlan)}
_ORDER = [GemmPlan, LayerNormPlan, SoftmaxPlan, ReduceRowsPlan, ReduceAllPlan, ElementwisePlan, BlockProgramPlan]


def make_plan(kernel: Kernel, an: Analyzer) -> Plan:
    """Pick the kernel family for an analysed kernel or raise UnsupportedTTIR with every reason."""
    reasons = []
    for cls in _ORDER:
        try:
            return cls.build(kernel, an)
        except UnsupportedTTIR as e:
            reasons.append(f"{cls.family}: {e}")
    raise UnsupportedTTIR(f"kernel {kernel.name} fits no pre-built kernel family:\n  " + "\n  ".join(reasons))
