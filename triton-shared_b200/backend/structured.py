"""Structured-access analysis of TTIR: the subset of triton-shared's PtrAnalysis and
MaskAnalysis that the executed kernels need, restated over parsed TTIR text.

What the reference does in MLIR C++ and this module re-derives (paths inside
microsoft/triton-shared):

* pointer arithmetic -> {source, offsets, sizes, strides, modulo} per block
  pointer (``PtrState``, lib/AnalysisStructured/PtrAnalysis.cpp:276-503 add,
  539-625 mul, 901-1100 make_range/splat/expand_dims/broadcast/addptr,
  1536-1602 loop-carried pointers);
* mask arithmetic -> per-dim access sizes ``max(min(end, bound), start) - start``
  (``MaskState``, lib/Analysis/MaskAnalysis.cpp:461-603 cmp, 355-453 and,
  224-286 scalar conjuncts);
* everything else becomes a small dataflow graph of block values whose ops keep
  the arith/math semantics of TritonArithToLinalg (one op per node).

Scalar integers are kept symbolic (``Poly``: polynomials over kernel arguments,
program ids, grid sizes and loop iteration counters) and evaluated at launch.
Anything outside the subset raises ``UnsupportedTTIR``; there is no fallback.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import numpy as np

from .ttir import Block, Function, Op, Type, UnsupportedTTIR

# --------------------------------------------------------------------------
# symbolic integers


def _atom_key(a):
    return repr(a)


class Poly:
    """Immutable polynomial with integer coefficients over atoms.

    Atoms: ("arg", i) | ("pid", axis) | ("np", axis) | ("it", loop_id) |
           ("carry", loop_id, k) | ("fn", name, Poly, Poly)
    """
    __slots__ = ("terms", "_hash")

    def __init__(self, terms: Dict[tuple, int]):
        self.terms = {m: c for m, c in terms.items() if c != 0}
        self._hash = None

    # constructors
    @staticmethod
    def const(c: int) -> "Poly":
        return Poly({(): int(c)})

    @staticmethod
    def atom(a) -> "Poly":
        return Poly({(a,): 1})

    @staticmethod
    def fn(name: str, a: "Poly", b: "Poly") -> "Poly":
        if a.is_const and b.is_const:
            return Poly.const(_fn_eval(name, a.as_const, b.as_const))
        return Poly.atom(("fn", name, a, b))

    def __hash__(self):
        if self._hash is None:
            self._hash = hash(tuple(sorted((tuple(_atom_key(a) for a in m), c) for m, c in self.terms.items())))
        return self._hash

    def __eq__(self, other):
        return isinstance(other, Poly) and self.terms == other.terms

    def __repr__(self):
        if not self.terms:
            return "0"
        parts = []
        for m, c in sorted(self.terms.items(), key=lambda kv: [_atom_key(a) for a in kv[0]]):
            names = "*".join(_atom_str(a) for a in m)
            parts.append(f"{c}" if not m else (names if c == 1 else f"{c}*{names}"))
        return " + ".join(parts)

    @property
    def is_const(self):
        return all(m == () for m in self.terms)

    @property
    def as_const(self):
        assert self.is_const
        return self.terms.get((), 0)

    @property
    def is_zero(self):
        return not self.terms

    def __add__(self, o):
        o = _poly(o)
        t = dict(self.terms)
        for m, c in o.terms.items():
            t[m] = t.get(m, 0) + c
        return Poly(t)

    __radd__ = __add__

    def __neg__(self):
        return Poly({m: -c for m, c in self.terms.items()})

    def __sub__(self, o):
        return self + (-_poly(o))

    def __mul__(self, o):
        o = _poly(o)
        t: Dict[tuple, int] = {}
        for m1, c1 in self.terms.items():
            for m2, c2 in o.terms.items():
                m = tuple(sorted(m1 + m2, key=_atom_key))
                t[m] = t.get(m, 0) + c1 * c2
        return Poly(t)

    __rmul__ = __mul__

    def atoms(self):
        """All atoms, including those nested inside fn atoms."""
        out = set()
        for m in self.terms:
            for a in m:
                out.add(a)
                if a[0] == "fn":
                    out |= a[2].atoms() | a[3].atoms()
        return out

    def depends_on(self, kinds) -> bool:
        return any(a[0] in kinds for a in self.atoms())

    def evaluate(self, env):
        """env maps atoms to ints or numpy int64 arrays."""
        total = 0
        for m, c in self.terms.items():
            v = c
            for a in m:
                v = v * _atom_eval(a, env)
            total = total + v
        return total

    def to_json(self):
        return [[[_atom_json(a) for a in m], c] for m, c in sorted(
            self.terms.items(), key=lambda kv: [_atom_key(a) for a in kv[0]])]

    @staticmethod
    def from_json(j) -> "Poly":
        return Poly({tuple(_atom_unjson(a) for a in m): c for m, c in j})


def _poly(x) -> Poly:
    return x if isinstance(x, Poly) else Poly.const(x)


def _atom_str(a):
    if a[0] == "fn":
        return f"{a[1]}({a[2]!r}, {a[3]!r})"
    return a[0] + "".join(str(x) for x in a[1:])


def _atom_json(a):
    if a[0] == "fn":
        return ["fn", a[1], a[2].to_json(), a[3].to_json()]
    return list(a)


def _atom_unjson(j):
    if j[0] == "fn":
        return ("fn", j[1], Poly.from_json(j[2]), Poly.from_json(j[3]))
    return tuple(j)


def _fn_eval(name, a, b):
    """Integer functions with the semantics of arith.* (division truncates toward zero)."""
    if name in ("divsi", "remsi", "ceildivsi"):
        bz = (b == 0)
        bb = np.where(bz, 1, b) if isinstance(bz, np.ndarray) else (1 if bz else b)
        if name == "ceildivsi":
            # trip count of scf.for: ceil(a / b) for positive b, 0 when a <= 0
            q = -((-a) // bb)
            return np.maximum(q, 0) if isinstance(q, np.ndarray) else max(q, 0)
        q = np.abs(a) // np.abs(bb) * np.sign(a) * np.sign(bb) if isinstance(a, np.ndarray) or isinstance(bb, np.ndarray) \
            else (abs(a) // abs(bb)) * (1 if (a >= 0) == (bb > 0) else -1)
        return q if name == "divsi" else a - q * bb
    if name == "minsi":
        return np.minimum(a, b) if isinstance(a, np.ndarray) or isinstance(b, np.ndarray) else min(a, b)
    if name == "maxsi":
        return np.maximum(a, b) if isinstance(a, np.ndarray) or isinstance(b, np.ndarray) else max(a, b)
    if name.startswith("cmp_"):
        r = {"slt": a < b, "sle": a <= b, "sgt": a > b, "sge": a >= b, "eq": a == b, "ne": a != b,
             "ult": a < b, "ule": a <= b, "ugt": a > b, "uge": a >= b}[name[4:]]
        return r.astype(np.int64) if isinstance(r, np.ndarray) else int(r)
    if name == "andi":
        return a & b
    if name == "ori":
        return a | b
    if name == "xori":
        return a ^ b
    if name == "shli":
        return a << b
    if name == "shrsi":
        return a >> b
    raise UnsupportedTTIR(f"integer function {name}")


def _atom_eval(a, env):
    if a[0] == "fn":
        return _fn_eval(a[1], a[2].evaluate(env), a[3].evaluate(env))
    try:
        return env[a]
    except KeyError:
        raise UnsupportedTTIR(f"no value for symbol {a} at launch") from None


# --------------------------------------------------------------------------
# abstract values

_INT_BITS = {"i1": 1, "i8": 8, "i16": 16, "i32": 32, "i64": 64}
_FLOATS = {"f16", "bf16", "f32", "f64"}


@dataclass(frozen=True)
class Wrapped:
    """Addend scale * ((inner_offset + inner_stride * i_dim) % modulus) of an index tensor."""
    dim: int
    inner_offset: Poly
    inner_stride: Poly
    modulus: Poly
    scale: Poly


@dataclass(frozen=True)
class SInt:
    poly: Poly
    elem: str = "i32"


@dataclass(frozen=True)
class TIdx:
    """Integer tensor affine in the lane coordinates: offset + sum_d strides[d] * i_d (+ wrapped addends)."""
    shape: Tuple[int, ...]
    offset: Poly
    strides: Tuple[Poly, ...]
    elem: str = "i32"
    wrapped: Tuple[Wrapped, ...] = ()

    @property
    def uniform(self):
        return all(s.is_zero for s in self.strides) and not self.wrapped

    def varying_dims(self):
        return [d for d, s in enumerate(self.strides) if not s.is_zero and self.shape[d] > 1]


@dataclass(frozen=True)
class SPtr:
    arg: int
    elem: str
    offset: Poly


@dataclass(frozen=True)
class TPtr:
    arg: int
    elem: str
    shape: Tuple[int, ...]
    offset: Poly
    strides: Tuple[Poly, ...]
    wrapped: Tuple[Wrapped, ...] = ()


@dataclass(frozen=True)
class TMask:
    """Per dim a tuple of (start, bound) upper-bound constraints (lanes i with start + i < bound),
    plus scalar conditions that gate the whole block."""
    shape: Tuple[int, ...]
    dims: Tuple[Tuple[Tuple[Poly, Poly], ...], ...]
    scalar_conds: Tuple[Poly, ...] = ()


class Node:
    """One value of the block dataflow graph (hash-consed)."""
    __slots__ = ("op", "args", "attrs", "shape", "dtype", "id")

    def __init__(self, op, args, attrs, shape, dtype, nid):
        self.op, self.args, self.attrs, self.shape, self.dtype, self.id = op, args, attrs, shape, dtype, nid

    def attr(self, k, default=None):
        return dict(self.attrs).get(k, default)

    def __repr__(self):
        a = ",".join(f"n{x.id}" if isinstance(x, Node) else repr(x) for x in self.args)
        return f"n{self.id}={self.op}({a}){dict(self.attrs) if self.attrs else ''}:{self.shape}x{self.dtype}"


@dataclass(frozen=True)
class TData:
    node: Node


@dataclass
class Access:
    """One tt.load / tt.store: the tts.make_tptr + tts.load/store descriptor."""
    kind: str  # "load" | "store"
    arg: int
    elem: str
    shape: Tuple[int, ...]
    offset: Poly
    strides: Tuple[Poly, ...]
    mask: Optional[TMask]
    other: Optional[Node]  # fill value (a const/splat node) for masked loads
    wrapped: Tuple[Wrapped, ...] = ()
    value: Optional[Node] = None  # stored value
    loops: Tuple[int, ...] = ()
    index: int = -1


@dataclass
class Loop:
    id: int
    lb: Poly
    ub: Poly
    step: Poly
    inits: List[object] = field(default_factory=list)
    yields: List[object] = field(default_factory=list)
    effects: List[object] = field(default_factory=list)  # ("store", Access) | ("loop", Loop)
    parent: Optional[int] = None

    @property
    def trip(self) -> Poly:
        return Poly.fn("ceildivsi", self.ub - self.lb, self.step)


@dataclass
class Kernel:
    name: str
    args: List[Tuple[str, Type]]
    accesses: List[Access]
    effects: List[object]
    loops: Dict[int, Loop]


# --------------------------------------------------------------------------

_BIN_INT = {"arith.addi", "arith.subi", "arith.muli", "arith.divsi", "arith.remsi", "arith.minsi",
            "arith.maxsi", "arith.andi", "arith.ori", "arith.xori", "arith.shli", "arith.shrsi",
            "arith.divui", "arith.remui", "arith.minui", "arith.maxui", "arith.shrui"}
_BIN_FLOAT = {"arith.addf", "arith.subf", "arith.mulf", "arith.divf", "arith.maxnumf", "arith.minnumf",
              "arith.maximumf", "arith.minimumf", "arith.remf"}
_UN_FLOAT = {"math.exp", "math.exp2", "math.log", "math.log2", "math.sqrt", "math.rsqrt", "math.sin",
             "math.cos", "math.tanh", "math.erf", "math.absf", "arith.negf", "math.floor", "math.ceil"}
_CASTS = {"arith.extf", "arith.truncf", "arith.sitofp", "arith.uitofp", "arith.fptosi", "arith.fptoui",
          "arith.extsi", "arith.extui", "arith.trunci", "arith.index_cast", "arith.bitcast", "tt.fp_to_fp",
          "tt.bitcast", "tt.int_to_ptr", "tt.ptr_to_int"}


def parse_float_literal(text: str, elem: str) -> float:
    text = text.strip()
    if text.startswith("0x") or text.startswith("-0x"):
        bits = int(text, 16)
        if elem == "f32":
            return struct.unpack("<f", struct.pack("<I", bits & 0xffffffff))[0]
        if elem == "f64":
            return struct.unpack("<d", struct.pack("<Q", bits))[0]
        if elem == "f16":
            return float(np.frombuffer(struct.pack("<H", bits & 0xffff), dtype=np.float16)[0])
        if elem == "bf16":
            return struct.unpack("<f", struct.pack("<I", (bits & 0xffff) << 16))[0]
    return float(text)


class Analyzer:
    """Walks a parsed tt.func once and produces a ``Kernel``."""

    def __init__(self, fn: Function):
        self.fn = fn
        self.nodes: Dict[tuple, Node] = {}
        self.accesses: List[Access] = []
        self.loops: Dict[int, Loop] = {}
        self._next_loop = 0

    # ---- graph construction
    def node(self, op, args=(), attrs=(), shape=(), dtype="f32") -> Node:
        attrs = tuple(sorted(attrs.items())) if isinstance(attrs, dict) else tuple(attrs)
        key = (op, tuple(a.id if isinstance(a, Node) else a for a in args), attrs, tuple(shape), dtype)
        n = self.nodes.get(key)
        if n is None:
            n = Node(op, tuple(args), attrs, tuple(shape), dtype, len(self.nodes))
            self.nodes[key] = n
        return n

    def run(self) -> Kernel:
        env: Dict[str, object] = {}
        for i, (name, ty) in enumerate(self.fn.args):
            if ty.is_tensor:
                raise UnsupportedTTIR("tensor-typed kernel argument")
            if ty.is_ptr:
                env[name] = SPtr(i, ty.pointee, Poly.const(0))
            elif ty.elem in _INT_BITS:
                env[name] = SInt(Poly.atom(("arg", i)), ty.elem)
            elif ty.elem in _FLOATS:
                env[name] = TData(self.node("farg", (), {"arg": i}, (), ty.elem))
            else:
                raise UnsupportedTTIR(f"kernel argument of type {ty.elem}")
        effects: List[object] = []
        self.walk(self.fn.body, env, effects, (), True)
        return Kernel(self.fn.name, self.fn.args, self.accesses, effects, self.loops)

    # ---- helpers
    def as_data(self, v, ty_shape=None) -> Node:
        """Materialise any abstract value as a graph node."""
        if isinstance(v, TData):
            return v.node
        if isinstance(v, SInt):
            return self.node("sint", (), {"poly": v.poly}, (), v.elem)
        if isinstance(v, TIdx):
            if v.wrapped:
                raise UnsupportedTTIR("wrapped (modulo) index tensor used as data")
            return self.node("index", (), {"offset": v.offset, "strides": v.strides}, v.shape, v.elem)
        if isinstance(v, TMask):
            return self.node("maskval", (), {"dims": v.dims, "conds": v.scalar_conds}, v.shape, "i1")
        raise UnsupportedTTIR(f"value of kind {type(v).__name__} used as data")

    @staticmethod
    def _shape_of(v):
        if isinstance(v, (TIdx, TPtr, TMask)):
            return v.shape
        if isinstance(v, TData):
            return v.node.shape
        return ()

    # ---- the walk
    def walk(self, block: Block, env, effects, loop_stack, record: bool):
        for op in block.ops:
            self.visit(op, env, effects, loop_stack, record)

    def visit(self, op: Op, env, effects, loop_stack, record):
        n = op.name
        get = lambda k: env[op.operands[k]]
        res = op.results[0][0] if op.results else None
        rty = op.results[0][1] if op.results else None

        if n == "arith.constant":
            env[res] = self._constant(op, rty)
        elif n == "tt.get_program_id":
            env[res] = SInt(Poly.atom(("pid", op.attrs["axis"])))
        elif n == "tt.get_num_programs":
            env[res] = SInt(Poly.atom(("np", op.attrs["axis"])))
        elif n == "tt.make_range":
            s, e = op.attrs["start"], op.attrs["end"]
            env[res] = TIdx((e - s,), Poly.const(s), (Poly.const(1),), rty.elem)
        elif n == "tt.splat":
            env[res] = self._splat(get(0), rty)
        elif n == "tt.expand_dims":
            env[res] = self._expand_dims(get(0), op.attrs["axis"], rty)
        elif n == "tt.broadcast":
            env[res] = self._broadcast(get(0), rty)
        elif n == "tt.addptr":
            env[res] = self._addptr(get(0), get(1))
        elif n in _BIN_INT:
            env[res] = self._bin_int(n.split(".")[1], get(0), get(1), rty)
        elif n in _BIN_FLOAT:
            a, b = self.as_data(get(0)), self.as_data(get(1))
            env[res] = TData(self.node(n.split(".")[1], (a, b), (), rty.shape, rty.elem))
        elif n in _UN_FLOAT:
            a = self.as_data(get(0))
            env[res] = TData(self.node(n.split(".")[1], (a,), (), rty.shape, rty.elem))
        elif n == "math.fma":
            a, b, c = (self.as_data(get(k)) for k in range(3))
            env[res] = TData(self.node("fma", (a, b, c), (), rty.shape, rty.elem))
        elif n == "math.absi":
            env[res] = TData(self.node("absi", (self.as_data(get(0)),), (), rty.shape, rty.elem))
        elif n in _CASTS:
            env[res] = self._cast(n, get(0), op, rty)
        elif n == "arith.cmpi":
            env[res] = self._cmpi(op.attrs["predicate"], get(0), get(1), rty)
        elif n == "arith.cmpf":
            a, b = self.as_data(get(0)), self.as_data(get(1))
            env[res] = TData(self.node("cmpf", (a, b), {"pred": op.attrs["predicate"]}, rty.shape, "i1"))
        elif n == "arith.select":
            c, a, b = self.as_data(get(0)), self.as_data(get(1)), self.as_data(get(2))
            env[res] = TData(self.node("select", (c, a, b), (), rty.shape, rty.elem))
        elif n == "tt.load":
            env[res] = self._load(op, env, loop_stack, record, rty)
        elif n == "tt.store":
            self._store(op, env, effects, loop_stack, record)
        elif n == "tt.reduce":
            self._reduce(op, env)
        elif n == "tt.dot":
            a, b, c = (self.as_data(get(k)) for k in range(3))
            env[res] = TData(self.node("dot", (a, b, c), (), rty.shape, rty.elem))
        elif n == "scf.for":
            self._for(op, env, effects, loop_stack, record)
        elif n in ("tt.return",):
            pass
        elif n == "tt.assert" or n == "tt.print":
            pass  # debugging aids have no effect on results
        else:
            raise UnsupportedTTIR(f"operation {n} is outside the structured subset: {op.text}")

    # ---- individual ops
    def _constant(self, op: Op, ty: Type):
        text = op.attrs["value"]
        dense = text.startswith("dense<")
        lit = text[6:-1] if dense else text
        if "[" in lit:
            raise UnsupportedTTIR("non-splat dense constant")
        if ty.elem in _INT_BITS:
            v = {"true": 1, "false": 0}.get(lit)
            if v is None:
                v = int(lit, 0)
            if ty.is_tensor:
                return TIdx(ty.shape, Poly.const(v), tuple(Poly.const(0) for _ in ty.shape), ty.elem)
            return SInt(Poly.const(v), ty.elem)
        if ty.elem in _FLOATS:
            v = parse_float_literal(lit, ty.elem)
            return TData(self.node("const", (), {"value": _float_key(v)}, ty.shape, ty.elem))
        raise UnsupportedTTIR(f"constant of type {ty.elem}")

    def _splat(self, v, ty: Type):
        zeros = tuple(Poly.const(0) for _ in ty.shape)
        if isinstance(v, SInt):
            return TIdx(ty.shape, v.poly, zeros, v.elem)
        if isinstance(v, SPtr):
            return TPtr(v.arg, v.elem, ty.shape, v.offset, zeros)
        if isinstance(v, TData):
            return TData(self.node("splat", (v.node,), (), ty.shape, v.node.dtype))
        raise UnsupportedTTIR("tt.splat of an unsupported value")

    def _expand_dims(self, v, axis: int, ty: Type):
        def ins(t, x):
            t = list(t)
            t.insert(axis, x)
            return tuple(t)

        def shift(ws):
            return tuple(Wrapped(w.dim + (1 if w.dim >= axis else 0), w.inner_offset, w.inner_stride,
                                 w.modulus, w.scale) for w in ws)
        if isinstance(v, TIdx):
            return TIdx(ins(v.shape, 1), v.offset, ins(v.strides, Poly.const(0)), v.elem, shift(v.wrapped))
        if isinstance(v, TPtr):
            return TPtr(v.arg, v.elem, ins(v.shape, 1), v.offset, ins(v.strides, Poly.const(0)), shift(v.wrapped))
        if isinstance(v, TMask):
            return TMask(ins(v.shape, 1), ins(v.dims, ()), v.scalar_conds)
        if isinstance(v, TData):
            return TData(self.node("expand_dims", (v.node,), {"axis": axis}, ty.shape, v.node.dtype))
        raise UnsupportedTTIR("tt.expand_dims of an unsupported value")

    def _broadcast(self, v, ty: Type):
        if isinstance(v, (TIdx, TPtr)):
            strides = tuple(Poly.const(0) if (a == 1 and b != 1) else s
                            for s, a, b in zip(v.strides, v.shape, ty.shape))
            for w in v.wrapped:
                if v.shape[w.dim] == 1 and ty.shape[w.dim] != 1:
                    raise UnsupportedTTIR("broadcast along a wrapped dimension")
            if isinstance(v, TIdx):
                return TIdx(ty.shape, v.offset, strides, v.elem, v.wrapped)
            return TPtr(v.arg, v.elem, ty.shape, v.offset, strides, v.wrapped)
        if isinstance(v, TMask):
            return TMask(ty.shape, v.dims, v.scalar_conds)
        if isinstance(v, TData):
            return TData(self.node("broadcast", (v.node,), (), ty.shape, v.node.dtype))
        raise UnsupportedTTIR("tt.broadcast of an unsupported value")

    def _addptr(self, p, o):
        if isinstance(p, SPtr) and isinstance(o, SInt):
            return SPtr(p.arg, p.elem, p.offset + o.poly)
        if isinstance(p, TPtr) and isinstance(o, TIdx):
            if p.shape != o.shape:
                raise UnsupportedTTIR("tt.addptr shape mismatch")
            return TPtr(p.arg, p.elem, p.shape, p.offset + o.offset,
                        tuple(a + b for a, b in zip(p.strides, o.strides)), p.wrapped + o.wrapped)
        raise UnsupportedTTIR("tt.addptr with a data-dependent offset (gather/scatter) is outside the structured subset")

    def _bin_int(self, name, a, b, ty: Type):
        if isinstance(a, SInt) and isinstance(b, SInt):
            pa, pb = a.poly, b.poly
            if name == "addi":
                return SInt(pa + pb, ty.elem)
            if name == "subi":
                return SInt(pa - pb, ty.elem)
            if name == "muli":
                return SInt(pa * pb, ty.elem)
            if name in ("divsi", "remsi", "minsi", "maxsi", "andi", "ori", "xori", "shli", "shrsi"):
                return SInt(Poly.fn(name, pa, pb), ty.elem)
            raise UnsupportedTTIR(f"scalar arith.{name}")
        if isinstance(a, TMask) and isinstance(b, TMask) and name == "andi":
            return TMask(a.shape, tuple(x + y for x, y in zip(a.dims, b.dims)), a.scalar_conds + b.scalar_conds)
        if isinstance(a, (TMask, SInt)) and isinstance(b, (TMask, SInt)) and name == "andi" and ty.elem == "i1":
            m, s = (a, b) if isinstance(a, TMask) else (b, a)
            return TMask(m.shape, m.dims, m.scalar_conds + (s.poly,))
        if name == "andi" and ty.elem == "i1":
            # a scalar condition splat over the block gates the whole mask (MaskAnalysis.cpp:224-267)
            m, s = (a, b) if isinstance(a, TMask) else (b, a)
            if isinstance(m, TMask) and isinstance(s, TIdx) and s.uniform:
                return TMask(m.shape, m.dims, m.scalar_conds + (s.offset,))
        if isinstance(a, TIdx) and isinstance(b, TIdx):
            if name in ("addi", "subi"):
                if name == "subi" and b.wrapped:
                    raise UnsupportedTTIR("subtraction of a wrapped index tensor")
                sgn = 1 if name == "addi" else -1
                return TIdx(a.shape, a.offset + sgn * b.offset,
                            tuple(x + sgn * y for x, y in zip(a.strides, b.strides)), ty.elem,
                            a.wrapped + b.wrapped)
            if name == "muli" and (a.uniform or b.uniform):
                t, u = (a, b) if b.uniform else (b, a)
                c = u.offset
                return TIdx(t.shape, t.offset * c, tuple(s * c for s in t.strides), ty.elem,
                            tuple(Wrapped(w.dim, w.inner_offset, w.inner_stride, w.modulus, w.scale * c)
                                  for w in t.wrapped))
            if name == "remsi" and b.uniform and not a.wrapped:
                vd = a.varying_dims()
                if len(vd) == 1:
                    d = vd[0]
                    zeros = tuple(Poly.const(0) for _ in a.shape)
                    return TIdx(a.shape, Poly.const(0), zeros, ty.elem,
                                (Wrapped(d, a.offset, a.strides[d], b.offset, Poly.const(1)),))
                if not vd:
                    return TIdx(a.shape, Poly.fn("remsi", a.offset, b.offset),
                                tuple(Poly.const(0) for _ in a.shape), ty.elem)
            if a.uniform and b.uniform and name in ("divsi", "remsi", "minsi", "maxsi"):
                return TIdx(a.shape, Poly.fn(name, a.offset, b.offset), a.strides, ty.elem)
        # integer data arithmetic
        na, nb = self.as_data(a), self.as_data(b)
        return TData(self.node(name, (na, nb), (), ty.shape, ty.elem))

    def _cast(self, name, v, op: Op, ty: Type):
        short = name.split(".")[1]
        if short in ("extsi", "extui", "trunci", "index_cast") and isinstance(v, SInt):
            return SInt(v.poly, ty.elem)
        if short in ("extsi", "extui", "trunci", "index_cast") and isinstance(v, TIdx):
            return TIdx(v.shape, v.offset, v.strides, ty.elem, v.wrapped)
        if short in ("int_to_ptr", "ptr_to_int"):
            raise UnsupportedTTIR(f"{name} is outside the structured subset")
        src = self.as_data(v)
        return TData(self.node("cast", (src,), {"kind": short, "from": src.dtype}, ty.shape, ty.elem))

    def _cmpi(self, pred, a, b, ty: Type):
        if isinstance(a, SInt) and isinstance(b, SInt):
            return SInt(Poly.fn("cmp_" + pred, a.poly, b.poly), "i1")
        if isinstance(a, TIdx) and isinstance(b, TIdx) and not a.wrapped and not b.wrapped:
            if pred in ("slt", "ult") and b.uniform:
                vd = a.varying_dims()
                if len(vd) == 1 and a.strides[vd[0]] == Poly.const(1):
                    dims = tuple(((a.offset, b.offset),) if d == vd[0] else () for d in range(len(a.shape)))
                    return TMask(a.shape, dims)
                if not vd:
                    return TMask(a.shape, tuple(() for _ in a.shape), (Poly.fn("cmp_" + pred, a.offset, b.offset),))
            if pred == "sgt" and a.uniform:  # bound > idx  ==  idx < bound
                return self._cmpi("slt", b, a, ty)
            if pred == "sge" and b.uniform and b.offset.is_zero:
                # idx >= 0: the reference assumes this comparison is true: dims already carry an implicit
                # lower bound of zero (lib/Analysis/MaskAnalysis.cpp:522-532)
                return TMask(a.shape, tuple(() for _ in a.shape))
        na, nb = self.as_data(a), self.as_data(b)
        return TData(self.node("cmpi", (na, nb), {"pred": pred}, ty.shape, "i1"))

    def _load(self, op: Op, env, loop_stack, record, ty: Type):
        p = env[op.operands[0]]
        mask = env[op.operands[1]] if len(op.operands) > 1 else None
        other = env[op.operands[2]] if len(op.operands) > 2 else None
        if mask is not None and not isinstance(mask, TMask):
            if isinstance(mask, SInt) and isinstance(p, SPtr):
                mask = TMask((), (), (mask.poly,))
            else:
                raise UnsupportedTTIR("load mask is not a structured range comparison")
        other_node = None
        if other is not None:
            other_node = self.as_data(other)
        if isinstance(p, SPtr):
            acc = Access("load", p.arg, p.elem, (), p.offset, (), mask, other_node, (), None, loop_stack)
        elif isinstance(p, TPtr):
            acc = Access("load", p.arg, p.elem, p.shape, p.offset, p.strides, mask, other_node, p.wrapped,
                         None, loop_stack)
        else:
            raise UnsupportedTTIR("load from a non-structured pointer")
        if record:
            acc.index = len(self.accesses)
            self.accesses.append(acc)
        key = len(self.accesses) if not record else acc.index
        node = self.node("load", (), {"access": key, "rec": record}, ty.shape, ty.elem)
        if record:
            self._load_nodes = getattr(self, "_load_nodes", {})
            self._load_nodes[node.id] = acc
        return TData(node)

    def access_of(self, node: Node) -> Access:
        return self._load_nodes[node.id]

    def _store(self, op: Op, env, effects, loop_stack, record):
        p = env[op.operands[0]]
        val = self.as_data(env[op.operands[1]])
        mask = env[op.operands[2]] if len(op.operands) > 2 else None
        if mask is not None and not isinstance(mask, TMask):
            if isinstance(mask, SInt) and isinstance(p, SPtr):
                mask = TMask((), (), (mask.poly,))
            else:
                raise UnsupportedTTIR("store mask is not a structured range comparison")
        if isinstance(p, SPtr):
            acc = Access("store", p.arg, p.elem, (), p.offset, (), mask, None, (), val, loop_stack)
        elif isinstance(p, TPtr):
            acc = Access("store", p.arg, p.elem, p.shape, p.offset, p.strides, mask, None, p.wrapped, val,
                         loop_stack)
        else:
            raise UnsupportedTTIR("store to a non-structured pointer")
        if record:
            acc.index = len(self.accesses)
            self.accesses.append(acc)
            effects.append(("store", acc))

    def _reduce(self, op: Op, env):
        blk = op.regions[0]
        body = [o for o in blk.ops if o.name != "tt.reduce.return"]
        if len(op.operands) == 2 and len(op.results) == 2:
            return self._arg_reduce(op, env, blk, body)
        if len(op.operands) != 1 or len(body) != 1 or len(body[0].operands) != 2:
            raise UnsupportedTTIR("tt.reduce with more than one input or a multi-op body")
        comb = body[0].name.split(".")[1]
        names = {a for a, _ in blk.args}
        if set(body[0].operands) != names:
            raise UnsupportedTTIR("tt.reduce body does not combine its two block arguments")
        src = self.as_data(env[op.operands[0]])
        rty = op.results[0][1]
        env[op.results[0][0]] = TData(self.node("reduce", (src,), {"axis": op.attrs["axis"], "comb": comb},
                                                rty.shape, rty.elem))

    def _arg_reduce(self, op: Op, env, blk: Block, body):
        """tl.argmax / tl.argmin: a reduction over (value, index) pairs that keeps the larger
        (smaller) value and, among equal values, the smaller index (the reference lowers the same
        region, ConversionPatterns.hpp:1442-1769)."""
        names = [o.name for o in body]
        preds = [o.attrs.get("predicate") for o in body if o.name == "arith.cmpf"]
        shape_ok = sorted(names) == sorted(["arith.cmpf", "arith.cmpi", "arith.andi", "arith.cmpf", "arith.ori",
                                            "arith.select", "arith.select"])
        if not shape_ok or "oeq" not in preds or not ({"ogt", "olt"} & set(preds)):
            raise UnsupportedTTIR("two-input tt.reduce that is not the argmax / argmin pattern")
        cmpi = [o for o in body if o.name == "arith.cmpi"][0]
        if cmpi.attrs.get("predicate") != "slt":
            raise UnsupportedTTIR("argmax / argmin with an unexpected tie-break")
        kind = "argmax" if "ogt" in preds else "argmin"
        val = self.as_data(env[op.operands[0]])
        idx = self.as_data(env[op.operands[1]])
        for k in range(2):
            rty = op.results[k][1]
            env[op.results[k][0]] = TData(self.node("argreduce", (val, idx),
                                                    {"axis": op.attrs["axis"], "comb": kind, "out": k},
                                                    rty.shape, rty.elem))

    def _for(self, op: Op, env, effects, loop_stack, record):
        lb, ub, step = (env[o] for o in op.operands[:3])
        if not all(isinstance(x, SInt) for x in (lb, ub, step)):
            raise UnsupportedTTIR("scf.for bounds are not scalar integers")
        lid = self._next_loop
        self._next_loop += 1
        blk = op.regions[0]
        iv_name = blk.args[0][0]
        iter_args = blk.args[1:]
        inits = [env[o] for o in op.operands[3:]]
        it = Poly.atom(("it", lid))
        iv = SInt(lb.poly + step.poly * it, blk.args[0][1].elem)
        if blk.ops and blk.ops[-1].name == "scf.yield":
            yield_op, body_ops = blk.ops[-1], blk.ops[:-1]
        else:  # a loop without carried values prints no terminator
            yield_op, body_ops = None, blk.ops
        if (yield_op is None) != (not iter_args):
            raise UnsupportedTTIR("scf.for terminator does not match its iter_args")

        def seed(deltas):
            e = dict(env)
            e[iv_name] = iv
            for k, ((name, ty), init) in enumerate(zip(iter_args, inits)):
                if isinstance(init, (TPtr, SPtr, SInt, TIdx)):
                    adv = Poly.atom(("carry", lid, k)) if deltas is None else it * deltas[k]
                    if isinstance(init, TPtr):
                        e[name] = TPtr(init.arg, init.elem, init.shape, init.offset + adv, init.strides, init.wrapped)
                    elif isinstance(init, SPtr):
                        e[name] = SPtr(init.arg, init.elem, init.offset + adv)
                    elif isinstance(init, SInt):
                        e[name] = SInt(init.poly + adv, init.elem)
                    else:
                        e[name] = TIdx(init.shape, init.offset + adv, init.strides, init.elem, init.wrapped)
                elif isinstance(init, TData):
                    e[name] = TData(self.node("iter_arg", (), {"loop": lid, "k": k}, ty.shape, ty.elem))
                else:
                    raise UnsupportedTTIR("unsupported loop-carried value")
            return e

        # pass 1 (not recorded): how far does each carried pointer/integer advance per iteration?
        saved_next = self._next_loop
        e1 = seed(None)
        self.walk(Block(blk.args, body_ops), e1, [], loop_stack + (lid,), False)
        deltas: List[Optional[Poly]] = []
        for k, ((name, ty), init) in enumerate(zip(iter_args, inits)):
            if isinstance(init, TData):
                deltas.append(None)
                continue
            y = e1[yield_op.operands[k]]
            cur = e1[name]
            off = (lambda v: v.poly if isinstance(v, SInt) else v.offset)
            if type(y) is not type(cur):
                raise UnsupportedTTIR("loop-carried value changes kind")
            if isinstance(y, (TPtr, TIdx)) and (y.strides != cur.strides or y.wrapped != cur.wrapped):
                raise UnsupportedTTIR("loop-carried pointer changes strides")
            if isinstance(y, (TPtr, SPtr)) and y.arg != cur.arg:
                raise UnsupportedTTIR("loop-carried pointer changes base")
            d = off(y) - off(cur)
            if any(a[0] == "carry" and a[1] == lid for a in d.atoms()) or any(a == ("it", lid) for a in d.atoms()):
                raise UnsupportedTTIR("loop-carried pointer advance is not loop-invariant")
            deltas.append(d)
        self._next_loop = saved_next
        # pass 2 (recorded when the enclosing walk is)
        loop = Loop(lid, lb.poly, ub.poly, step.poly, inits, [], [], loop_stack[-1] if loop_stack else None)
        self.loops[lid] = loop
        e2 = seed(deltas)
        self.walk(Block(blk.args, body_ops), e2, loop.effects, loop_stack + (lid,), record)
        for k, ((name, ty), init) in enumerate(zip(iter_args, inits)):
            y = e2[yield_op.operands[k]]
            loop.yields.append(y)
            rname = op.results[k][0]
            if isinstance(init, TData):
                env[rname] = TData(self.node("loop_result", (), {"loop": lid, "k": k}, ty.shape, ty.elem))
            else:
                total = loop.trip * deltas[k]
                if isinstance(init, TPtr):
                    env[rname] = TPtr(init.arg, init.elem, init.shape, init.offset + total, init.strides, init.wrapped)
                elif isinstance(init, SPtr):
                    env[rname] = SPtr(init.arg, init.elem, init.offset + total)
                elif isinstance(init, SInt):
                    env[rname] = SInt(init.poly + total, init.elem)
                else:
                    env[rname] = TIdx(init.shape, init.offset + total, init.strides, init.elem, init.wrapped)
        if record:
            effects.append(("loop", loop))


def _float_key(v: float):
    """Hashable, NaN-safe representation of a float constant (its fp64 bit pattern)."""
    return struct.unpack("<q", struct.pack("<d", v))[0]


def float_from_key(k: int) -> float:
    return struct.unpack("<d", struct.pack("<q", k))[0]


def analyze(fn: Function) -> Tuple[Kernel, Analyzer]:
    a = Analyzer(fn)
    return a.run(), a
