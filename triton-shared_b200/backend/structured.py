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
    indirect: Optional["Node"] = None  # data-dependent element offset (a scalar integer value)


@dataclass(frozen=True)
class TPtr:
    arg: int
    elem: str
    shape: Tuple[int, ...]
    offset: Poly
    strides: Tuple[Poly, ...]
    wrapped: Tuple[Wrapped, ...] = ()
    # data-dependent element offsets (an integer block value of this shape) added to the structured
    # address: what the reference turns into tts.make_gather_scatter_tptr / unstructured accesses
    indirect: Optional["Node"] = None


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
    indirect: Optional[Node] = None   # per-lane element offsets computed as data (gather / scatter)
    mask_data: Optional[Node] = None  # per-lane i1 mask computed as data (conjoined with `mask`)


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
        self.guards: List[object] = []  # conditions under which the rest of the kernel runs (early returns)
        self._walk_cfg(self.fn.body, env, effects, 0)
        return Kernel(self.fn.name, self.fn.args, self.accesses, effects, self.loops)

    def _walk_cfg(self, block: Block, env, effects, depth: int):
        """Walk a function body whose only control flow between blocks is the early return
        (`if cond: return`): a conditional branch one of whose targets returns at once.  The
        condition becomes a guard and-ed into the mask of every later access."""
        if depth > 16:
            raise UnsupportedTTIR("control flow between blocks nests too deeply")
        for op in block.ops:
            if op.name == "cf.br":
                return self._walk_cfg(self._target(op.attrs["dests"][0]), env, effects, depth + 1)
            if op.name == "cf.cond_br":
                cond = env[op.operands[0]]
                yes, no = (self._target(d) for d in op.attrs["dests"])
                returns = lambda b: len(b.ops) == 1 and b.ops[0].name == "tt.return"
                if returns(yes):
                    self.guards.append((cond, False))
                    return self._walk_cfg(no, env, effects, depth + 1)
                if returns(no):
                    self.guards.append((cond, True))
                    return self._walk_cfg(yes, env, effects, depth + 1)
                raise UnsupportedTTIR("conditional branch other than an early return")
            self.visit(op, env, effects, (), True)

    def _target(self, label: str) -> Block:
        b = self.fn.blocks.get(label)
        if b is None or b.args:
            raise UnsupportedTTIR(f"branch to {label}: unknown block or block with arguments")
        return b

    def _guarded(self, shape, mask, mask_data):
        """(mask, mask_data) with the early-return guards added."""
        for cond, want in self.guards:
            if isinstance(cond, SInt):
                p = cond.poly if want else Poly.fn("cmp_eq", cond.poly, Poly.const(0))
                base = mask if mask is not None else TMask(tuple(shape), tuple(() for _ in shape))
                mask = TMask(base.shape, base.dims, base.scalar_conds + (p,))
            else:
                n = self.as_data(cond)
                if n.shape != ():
                    raise UnsupportedTTIR("branch on a block value")
                if not want:
                    one = self.node("sint", (), {"poly": Poly.const(1)}, (), "i1")
                    n = self.node("xori", (n, one), (), (), "i1")
                if shape:
                    n = self.node("splat", (n,), (), tuple(shape), "i1")
                mask_data = n if mask_data is None else self.node("andi", (mask_data, n), (), tuple(shape), "i1")
        return mask, mask_data

    # ---- helpers
    def as_data(self, v, ty_shape=None) -> Node:
        """Materialise any abstract value as a graph node."""
        if isinstance(v, TData):
            return v.node
        if isinstance(v, SInt):
            return self.node("sint", (), {"poly": v.poly}, (), v.elem)
        if isinstance(v, TIdx):
            n = self.node("index", (), {"offset": v.offset, "strides": v.strides}, v.shape, v.elem)
            zero = Poly.const(0)
            for w in v.wrapped:
                # scale * ((inner_offset + inner_stride * i_dim) mod modulus) as lane arithmetic
                st = tuple(w.inner_stride if d == w.dim else zero for d in range(len(v.shape)))
                inner = self.node("index", (), {"offset": w.inner_offset, "strides": st}, v.shape, v.elem)
                r = self.node("remsi", (inner, self._splat_int(w.modulus, v.shape, v.elem)), (), v.shape, v.elem)
                if w.scale != Poly.const(1):
                    r = self.node("muli", (r, self._splat_int(w.scale, v.shape, v.elem)), (), v.shape, v.elem)
                n = self.node("addi", (n, r), (), v.shape, v.elem)
            return n
        if isinstance(v, TMask):
            return self.node("maskval", (), {"dims": v.dims, "conds": v.scalar_conds}, v.shape, "i1")
        raise UnsupportedTTIR(f"value of kind {type(v).__name__} used as data")

    def _splat_int(self, p: Poly, shape, elem) -> Node:
        n = self.node("sint", (), {"poly": p}, (), elem)
        return self.node("splat", (n,), (), tuple(shape), elem) if shape else n

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
        elif n == "tt.reshape":
            env[res] = self._reshape(get(0), rty.shape)
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
        elif n == "tt.scan":
            self._scan(op, env)
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
            ind = None if v.indirect is None else self.node("splat", (v.indirect,), (), ty.shape, v.indirect.dtype)
            return TPtr(v.arg, v.elem, ty.shape, v.offset, zeros, (), ind)
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
            ind = None if v.indirect is None else self.node("expand_dims", (v.indirect,), {"axis": axis}, ins(v.shape, 1),
                                                            v.indirect.dtype)
            return TPtr(v.arg, v.elem, ins(v.shape, 1), v.offset, ins(v.strides, Poly.const(0)), shift(v.wrapped), ind)
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
            ind = None if v.indirect is None else self.node("broadcast", (v.indirect,), (), ty.shape, v.indirect.dtype)
            return TPtr(v.arg, v.elem, ty.shape, v.offset, strides, v.wrapped, ind)
        if isinstance(v, TMask):
            return TMask(ty.shape, v.dims, v.scalar_conds)
        if isinstance(v, TData):
            return TData(self.node("broadcast", (v.node,), (), ty.shape, v.node.dtype))
        raise UnsupportedTTIR("tt.broadcast of an unsupported value")

    def _add_indirect(self, ind: Optional[Node], n: Node, shape) -> Node:
        return n if ind is None else self.node("addi", (ind, n), (), tuple(shape), n.dtype)

    def _addptr(self, p, o):
        if isinstance(p, SPtr) and isinstance(o, SInt):
            return SPtr(p.arg, p.elem, p.offset + o.poly, p.indirect)
        if isinstance(p, SPtr) and isinstance(o, TData) and o.node.shape == ():
            # a scalar offset that was loaded from memory: a data-dependent base
            return SPtr(p.arg, p.elem, p.offset, self._add_indirect(p.indirect, o.node, ()))
        if isinstance(p, TPtr) and isinstance(o, TIdx):
            if p.shape != o.shape:
                raise UnsupportedTTIR("tt.addptr shape mismatch")
            return TPtr(p.arg, p.elem, p.shape, p.offset + o.offset,
                        tuple(a + b for a, b in zip(p.strides, o.strides)), p.wrapped + o.wrapped, p.indirect)
        if isinstance(p, TPtr) and isinstance(o, TData):
            # offsets that are block data (loaded indices, divisions of lane numbers, ...): kept as a
            # per-lane index added to the structured part of the address (gather / scatter)
            if o.node.shape != p.shape:
                raise UnsupportedTTIR("tt.addptr shape mismatch")
            return TPtr(p.arg, p.elem, p.shape, p.offset, p.strides, p.wrapped,
                        self._add_indirect(p.indirect, o.node, p.shape))
        raise UnsupportedTTIR("tt.addptr of these operand kinds is outside the supported subset")

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

    def _split_mask(self, mask, p):
        """A tt.load / tt.store mask operand as (structured TMask or None, data mask node or None)."""
        if mask is None or isinstance(mask, TMask):
            return mask, None
        if isinstance(mask, SInt) and isinstance(p, SPtr):
            return TMask((), (), (mask.poly,)), None
        if isinstance(mask, TData) and mask.node.dtype == "i1":
            return None, mask.node
        if isinstance(mask, TIdx) and mask.elem == "i1" and mask.uniform:
            return TMask(mask.shape, tuple(() for _ in mask.shape), (mask.offset,)), None
        raise UnsupportedTTIR("mask operand of an unsupported kind")

    def _load(self, op: Op, env, loop_stack, record, ty: Type):
        p = env[op.operands[0]]
        mask = env[op.operands[1]] if len(op.operands) > 1 else None
        other = env[op.operands[2]] if len(op.operands) > 2 else None
        if not isinstance(p, (SPtr, TPtr)):
            raise UnsupportedTTIR("load from a non-structured pointer")
        mask, mask_data = self._split_mask(mask, p)
        other_node = None
        if other is not None:
            other_node = self.as_data(other)
        shape = p.shape if isinstance(p, TPtr) else ()
        mask, mask_data = self._guarded(shape, mask, mask_data)
        if isinstance(p, SPtr):
            acc = Access("load", p.arg, p.elem, (), p.offset, (), mask, other_node, (), None, loop_stack)
        else:
            acc = Access("load", p.arg, p.elem, p.shape, p.offset, p.strides, mask, other_node, p.wrapped,
                         None, loop_stack)
        acc.indirect, acc.mask_data = p.indirect, mask_data
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
        if not isinstance(p, (SPtr, TPtr)):
            raise UnsupportedTTIR("store to a non-structured pointer")
        if val.op == "reshape" and isinstance(p, TPtr):
            # store(ptr, reshape(v)) == store(reshape(ptr), v): the reshape moves to the address side
            src = val.args[0]
            p = self._reshape(p, src.shape)
            if mask is not None:
                mask = self._reshape(mask, src.shape)
            val = src
        mask, mask_data = self._split_mask(mask, p)
        shape = p.shape if isinstance(p, TPtr) else ()
        mask, mask_data = self._guarded(shape, mask, mask_data)
        if isinstance(p, SPtr):
            acc = Access("store", p.arg, p.elem, (), p.offset, (), mask, None, (), val, loop_stack)
        else:
            acc = Access("store", p.arg, p.elem, p.shape, p.offset, p.strides, mask, None, p.wrapped, val,
                         loop_stack)
        acc.indirect, acc.mask_data = p.indirect, mask_data
        if record:
            acc.index = len(self.accesses)
            self.accesses.append(acc)
            effects.append(("store", acc))

    # ---- tt.reshape: row-major re-indexing of the same elements
    @staticmethod
    def _row_major_strides(shape, unit: Poly):
        st, acc = [], unit
        for n in reversed(shape):
            st.append(acc)
            acc = acc * n
        return tuple(reversed(st))

    def _reshape(self, v, shape):
        shape = tuple(shape)
        if isinstance(v, (TIdx, TPtr)):
            if v.wrapped or (isinstance(v, TPtr) and v.indirect is not None):
                raise UnsupportedTTIR("tt.reshape of a wrapped or data-dependent pointer")
            # the source must enumerate its elements as base + unit * (row-major lane number)
            live = [d for d in range(len(v.shape)) if v.shape[d] > 1]
            unit = v.strides[live[-1]] if live else Poly.const(0)
            if tuple(v.strides[d] for d in live) != tuple(self._row_major_strides([v.shape[d] for d in live], unit)):
                raise UnsupportedTTIR("tt.reshape of a block whose lanes are not evenly spaced in row-major order")
            st = tuple(s if n > 1 else Poly.const(0) for s, n in zip(self._row_major_strides(shape, unit), shape))
            if isinstance(v, TIdx):
                return TIdx(shape, v.offset, st, v.elem)
            return TPtr(v.arg, v.elem, shape, v.offset, st)
        if isinstance(v, TMask):
            dims = []
            for d, cons in enumerate(v.dims):
                for start, bound in cons:
                    # only a constraint that is known to admit the whole dim can be dropped
                    if not (start.is_const and bound.is_const and start.as_const + v.shape[d] <= bound.as_const):
                        raise UnsupportedTTIR("tt.reshape of a mask that may cut the block")
            return TMask(shape, tuple(() for _ in shape), v.scalar_conds)
        if isinstance(v, TData):
            n = v.node
            if n.op == "load" and n.id in getattr(self, "_load_nodes", {}):
                # reshape(load(ptr)) == load(reshape(ptr)): re-issue the load with the reshaped address
                acc = self._load_nodes[n.id]
                if acc.indirect is None and acc.mask_data is None and not acc.wrapped:
                    src = TPtr(acc.arg, acc.elem, acc.shape, acc.offset, acc.strides)
                    q = self._reshape(src, shape)
                    mask = self._reshape(acc.mask, shape) if acc.mask is not None else None
                    other = acc.other
                    if other is not None and other.shape not in ((), shape):
                        base = other
                        while base.op in ("splat", "broadcast", "expand_dims"):
                            base = base.args[0]
                        if base.op == "const":
                            other = self.node("const", (), dict(base.attrs), shape, base.dtype)
                        elif base.op == "index" and all(st.is_zero for st in base.attr("strides")):
                            other = self.node("index", (), {"offset": base.attr("offset"),
                                                            "strides": tuple(Poly.const(0) for _ in shape)}, shape, base.dtype)
                        else:
                            other = self.node("splat", (base,), (), shape, base.dtype) if base.shape == () else None
                        if other is None:
                            raise UnsupportedTTIR("tt.reshape of a load whose `other` is not a splat")
                    new = Access("load", q.arg, q.elem, shape, q.offset, q.strides, mask, other, (), None, acc.loops)
                    new.index = len(self.accesses)
                    self.accesses.append(new)
                    node = self.node("load", (), {"access": new.index, "rec": True}, shape, n.dtype)
                    self._load_nodes[node.id] = new
                    return TData(node)
            return TData(self.node("reshape", (n,), (), shape, n.dtype))
        raise UnsupportedTTIR("tt.reshape of an unsupported value")

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

    def _scan(self, op: Op, env):
        """tl.cumsum: the one scan the reference lowers (a single add combining the two block
        arguments, CumSumConverter, ConversionPatterns.hpp:1941-2007)."""
        blk = op.regions[0]
        body = [o for o in blk.ops if o.name != "tt.scan.return"]
        if len(op.operands) != 1 or len(body) != 1 or body[0].name not in ("arith.addf", "arith.addi") or \
                set(body[0].operands) != {a for a, _ in blk.args}:
            raise UnsupportedTTIR("tt.scan other than a cumulative sum")
        if op.attrs.get("reverse"):
            raise UnsupportedTTIR("reverse tt.scan")
        src = self.as_data(env[op.operands[0]])
        rty = op.results[0][1]
        env[op.results[0][0]] = TData(self.node("scan", (src,), {"axis": op.attrs["axis"], "comb": body[0].name.split(".")[1]},
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

    MAX_UNROLL = 64

    def _for(self, op: Op, env, effects, loop_stack, record):
        """A loop is first analysed symbolically (carried pointers and integers advance by a
        loop-invariant amount, carried block data become iter_arg nodes).  Where that fails (a
        carried index tensor that is recomputed non-linearly, a carried value that changes kind, ...)
        and the trip count is a small constant, the loop is unrolled instead: its body is walked
        once per iteration with the induction variable a constant."""
        snap = (len(self.accesses), len(effects), set(self.loops), self._next_loop, dict(getattr(self, "_load_nodes", {})),
                dict(env))
        lb, ub, step = (env.get(o) for o in op.operands[:3])
        const = all(isinstance(x, SInt) and x.poly.is_const for x in (lb, ub, step))
        trip = -(-(ub.poly.as_const - lb.poly.as_const) // step.poly.as_const) if const and step.poly.as_const > 0 else None
        can_unroll = trip is not None and trip <= self.MAX_UNROLL
        # a carried integer block value is an index tensor that the body recomputes: as a loop-carried
        # datum it could only run as a block program, which has no data-dependent addressing
        carried_index = any(isinstance(env.get(o), TData) and env[o].node.dtype.startswith("i") and env[o].node.shape
                            for o in op.operands[3:])
        try:
            if can_unroll and carried_index:
                raise UnsupportedTTIR("loop carries an index tensor as data")
            return self._for_structured(op, env, effects, loop_stack, record)
        except UnsupportedTTIR:
            if not can_unroll:
                raise
            del self.accesses[snap[0]:]
            del effects[snap[1]:]
            for k in set(self.loops) - snap[2]:
                del self.loops[k]
            self._next_loop = snap[3]
            self._load_nodes = snap[4]
            env.clear()
            env.update(snap[5])
            self._for_unrolled(op, env, effects, loop_stack, record, lb.poly.as_const, step.poly.as_const, max(trip, 0))

    def _for_unrolled(self, op: Op, env, effects, loop_stack, record, lb: int, step: int, trip: int):
        blk = op.regions[0]
        iv_name, iv_ty = blk.args[0]
        iter_args = blk.args[1:]
        if blk.ops and blk.ops[-1].name == "scf.yield":
            yield_op, body_ops = blk.ops[-1], blk.ops[:-1]
        else:
            yield_op, body_ops = None, blk.ops
        cur = [env[o] for o in op.operands[3:]]
        for t in range(trip):
            e = dict(env)
            e[iv_name] = SInt(Poly.const(lb + t * step), iv_ty.elem)
            for (name, _), v in zip(iter_args, cur):
                e[name] = v
            self.walk(Block(blk.args, body_ops), e, effects, loop_stack, record)
            if yield_op is not None:
                cur = [e[y] for y in yield_op.operands]
        for (rname, _), v in zip(op.results, cur):
            env[rname] = v

    def _for_structured(self, op: Op, env, effects, loop_stack, record):
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
                if isinstance(init, (TPtr, SPtr)) and init.indirect is not None:
                    raise UnsupportedTTIR("loop-carried pointer with data-dependent offsets")
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
            if isinstance(y, (TPtr, SPtr)) and (y.arg != cur.arg or y.indirect is not None):
                raise UnsupportedTTIR("loop-carried pointer changes base or gains data-dependent offsets")
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
