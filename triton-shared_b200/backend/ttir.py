"""Parser for the textual Triton IR (TTIR) that the backend's ``ttir`` stage produces.

The installed Triton exposes no generic attribute getters on ``ir.operation``, so
the plan compiler reads ``module.str_nodebug()``.  Only the op set that the
reference's middle layer accepts on its structured path is parsed
(``tt``, ``arith``, ``math``, ``scf.for/if/yield``); anything else raises
``UnsupportedTTIR`` -- there is no fallback executor.

The result is a tree of ``Op`` objects; no semantics are attached here.
"""
import re
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


class UnsupportedTTIR(Exception):
    """The kernel uses a construct outside the structured subset this backend executes."""


@dataclass(frozen=True)
class Type:
    """Scalar (shape == ()) or tensor type; ``elem`` is e.g. 'f32', 'i32', 'ptr<f16>'."""
    shape: Tuple[int, ...]
    elem: str

    @property
    def is_ptr(self):
        return self.elem.startswith("ptr<")

    @property
    def pointee(self):
        return self.elem[4:-1]

    @property
    def is_tensor(self):
        return len(self.shape) > 0 or self._tensor

    _tensor: bool = False


def parse_type(s: str) -> Type:
    s = s.strip()
    if s.startswith("tensor<"):
        inner = s[len("tensor<"):-1]
        dims = []
        while True:
            m = re.match(r"(\d+)x", inner)
            if not m:
                break
            dims.append(int(m.group(1)))
            inner = inner[m.end():]
        return Type(tuple(dims), _elem(inner), True)
    return Type((), _elem(s), False)


def _elem(s: str) -> str:
    s = s.strip()
    if s.startswith("!tt.ptr<"):
        inner = s[len("!tt.ptr<"):-1]
        # drop an address space such as "f32, 1"
        inner = inner.split(",")[0].strip()
        if inner.startswith("tensor<") or inner.startswith("!tt.ptr"):
            raise UnsupportedTTIR(f"pointer to non-scalar type: {s}")
        return f"ptr<{inner}>"
    if s == "index":
        return "i64"
    return s


@dataclass
class Block:
    args: List[Tuple[str, Type]] = field(default_factory=list)
    ops: List["Op"] = field(default_factory=list)


@dataclass
class Op:
    name: str
    results: List[Tuple[str, Type]]
    operands: List[str]
    attrs: Dict[str, object]
    regions: List[Block] = field(default_factory=list)
    text: str = ""


@dataclass
class Function:
    name: str
    args: List[Tuple[str, Type]]
    body: Block
    blocks: Dict[str, Block] = field(default_factory=dict)  # labelled successor blocks (^bb1, ...) of the body


_SSA = r"%[A-Za-z0-9_.$#-]+"


def _split_top(s: str, sep: str = ",") -> List[str]:
    """Split on `sep` outside of <>, (), [], {}."""
    out, depth, cur = [], 0, []
    for ch in s:
        if ch in "<([{":
            depth += 1
        elif ch in ">)]}":
            depth -= 1
        if ch == sep and depth == 0:
            out.append("".join(cur).strip())
            cur = []
        else:
            cur.append(ch)
    tail = "".join(cur).strip()
    if tail:
        out.append(tail)
    return out


def _parse_attr_dict(s: str) -> Dict[str, object]:
    """`{axis = 1 : i32, end = 1024 : i32}` (or the `<{...}>` property form)."""
    s = s.strip()
    if s.startswith("<"):
        s = s[1:-1].strip()
    s = s[1:-1]
    out = {}
    for item in _split_top(s):
        if "=" not in item:
            out[item.strip()] = True
            continue
        k, v = item.split("=", 1)
        out[k.strip()] = _parse_attr_value(v.strip())
    return out


def _parse_attr_value(v: str):
    m = re.match(r"^(-?\d+)\s*:\s*i\d+$", v)
    if m:
        return int(m.group(1))
    m = re.match(r"^array<i\d+(?::\s*(.*))?>$", v)
    if m:
        return [int(x) for x in m.group(1).split(",")] if m.group(1) else []
    if v in ("true", "false"):
        return v == "true"
    return v


def _find_trailing_type(s: str) -> Tuple[str, str]:
    """Split `... : type-part` at the last top-level ' : '."""
    depth = 0
    idx = -1
    for i, ch in enumerate(s):
        if ch in "<([{":
            depth += 1
        elif ch in ">)]}":
            depth -= 1
        elif ch == ":" and depth == 0 and s[i - 1:i] == " " and s[i + 1:i + 2] == " ":
            idx = i
    if idx < 0:
        return s, ""
    return s[:idx].rstrip(), s[idx + 1:].strip()


class _Lines:
    def __init__(self, text: str):
        # a trailing `// pred: ^bb0` comment follows block labels
        self.lines = [re.sub(r"\s+//.*$", "", l.rstrip()) for l in text.splitlines()]
        self.i = 0

    def peek(self) -> Optional[str]:
        while self.i < len(self.lines) and not self.lines[self.i].strip():
            self.i += 1
        return self.lines[self.i].strip() if self.i < len(self.lines) else None

    def next(self) -> str:
        l = self.peek()
        self.i += 1
        return l


def parse_module(text: str) -> Function:
    """Parse a module holding exactly one public tt.func."""
    L = _Lines(text)
    fn = None
    while L.peek() is not None:
        line = L.next()
        if line.startswith("tt.func"):
            if "private" in line.split("@")[0]:
                raise UnsupportedTTIR("non-inlined private function in module")
            if fn is not None:
                raise UnsupportedTTIR("more than one function in module")
            fn = _parse_func(line, L)
    if fn is None:
        raise UnsupportedTTIR("no tt.func found")
    return fn


def _parse_func(line: str, L: _Lines) -> Function:
    m = re.match(r"tt\.func\s+(?:public\s+)?@([\w$.]+)\((.*)\)\s*(?:attributes\s*\{.*\}\s*)?\{$", line)
    if not m:
        raise UnsupportedTTIR(f"cannot parse function header: {line}")
    args = []
    for a in _split_top(m.group(2)):
        if not a:
            continue
        am = re.match(rf"({_SSA})\s*:\s*(.*)$", a)
        ty = am.group(2)
        # strip an argument attribute dict such as {tt.divisibility = 16 : i32}
        ty = re.sub(r"\s*\{[^}]*\}\s*$", "", ty)
        args.append((am.group(1), parse_type(ty)))
    labels: Dict[str, Block] = {}
    body = _parse_block_body(L, labels=labels)
    return Function(m.group(1), args, body, labels)


def _parse_block_body(L: _Lines, block: Optional[Block] = None, labels: Optional[Dict[str, Block]] = None) -> Block:
    """Parse ops until the closing '}' (left for the caller). Returns the (entry) block.  A label
    before the first op names the block's own arguments (region bodies); later labels start the
    successor blocks of a function body, collected into `labels`."""
    entry = blk = block or Block()
    while True:
        line = L.peek()
        if line is None:
            raise UnsupportedTTIR("unexpected end of module")
        if line.startswith("}"):
            return entry  # caller inspects/consumes the closing line
        L.next()
        if line.startswith("^bb"):
            m = re.match(r"(\^bb\d+)(?:\((.*)\))?:$", line)
            if not m:
                raise UnsupportedTTIR(f"cannot parse block label: {line}")
            if blk is entry and not blk.ops and not blk.args and labels is None:
                target = blk
            else:
                if labels is None:
                    raise UnsupportedTTIR("control flow between blocks inside a region")
                target = blk = labels.setdefault(m.group(1), Block())
            for a in _split_top(m.group(2) or ""):
                am = re.match(rf"({_SSA})\s*:\s*(.*)$", a)
                target.args.append((am.group(1), parse_type(am.group(2))))
            continue
        blk.ops.append(_parse_op(line, L))


def _results_of(lhs: str, types: List[Type]) -> List[Tuple[str, Type]]:
    lhs = lhs.strip()
    m = re.match(rf"({_SSA}):(\d+)$", lhs)
    if m:
        n = int(m.group(2))
        assert n == len(types), (lhs, types)
        return [(f"{m.group(1)}#{k}", types[k]) for k in range(n)]
    names = [x.strip() for x in lhs.split(",")]
    assert len(names) == len(types), (lhs, types)
    return list(zip(names, types))


def _parse_op(line: str, L: _Lines) -> Op:
    lhs = None
    rest = line
    m = re.match(rf"^((?:{_SSA}(?::\d+)?)(?:\s*,\s*{_SSA})*)\s*=\s*(.*)$", line)
    if m:
        lhs, rest = m.group(1), m.group(2)
    # generic form with regions: "tt.reduce"(%x) <{axis = 0 : i32}> ({
    if rest.startswith('"'):
        return _parse_generic(lhs, rest, L, line)
    name = rest.split()[0] if " " in rest else rest
    body = rest[len(name):].strip()
    if name == "scf.for":
        return _parse_for(lhs, body, L, line)
    if name == "scf.if":
        return _parse_if(lhs, body, L, line)
    return _parse_simple(lhs, name, body, line)


def _parse_generic(lhs, rest, L: _Lines, line) -> Op:
    m = re.match(r'^"([\w.]+)"\((.*?)\)\s*(<\{.*?\}>)?\s*\(\{$', rest)
    if not m:
        raise UnsupportedTTIR(f"cannot parse generic op: {line}")
    name = m.group(1)
    operands = [x.strip() for x in _split_top(m.group(2))] if m.group(2).strip() else []
    attrs = _parse_attr_dict(m.group(3)) if m.group(3) else {}
    regions = []
    blk = _parse_block_body(L)
    regions.append(blk)
    closing = L.next()
    while closing.startswith("}, {"):
        regions.append(_parse_block_body(L))
        closing = L.next()
    cm = re.match(r"^\}\)\s*(\{.*\})?\s*:\s*\((.*)\)\s*->\s*(.*)$", closing)
    if not cm:
        raise UnsupportedTTIR(f"cannot parse end of generic op: {closing}")
    if cm.group(1):
        attrs.update(_parse_attr_dict(cm.group(1)))
    res_s = cm.group(3).strip()
    if res_s.startswith("("):
        res_s = res_s[1:-1]
    rtypes = [parse_type(t) for t in _split_top(res_s)] if res_s else []
    results = _results_of(lhs, rtypes) if lhs else []
    attrs["operand_types"] = [parse_type(t) for t in _split_top(cm.group(2))]
    return Op(name, results, operands, attrs, regions, line)


def _parse_for(lhs, body, L: _Lines, line) -> Op:
    m = re.match(rf"^({_SSA})\s*=\s*({_SSA})\s+to\s+({_SSA})\s+step\s+({_SSA})\s*(?:iter_args\((.*)\)\s*->\s*\((.*)\))?\s*(?::\s*(\w+))?\s*\{{$", body)
    if not m:
        raise UnsupportedTTIR(f"cannot parse scf.for: {line}")
    iv, lb, ub, step = m.group(1), m.group(2), m.group(3), m.group(4)
    iter_names, inits, rtypes = [], [], []
    if m.group(5):
        for it in _split_top(m.group(5)):
            a, b = it.split("=")
            iter_names.append(a.strip())
            inits.append(b.strip())
        rtypes = [parse_type(t) for t in _split_top(m.group(6))]
    iv_ty = parse_type(m.group(7) or "index")
    blk = Block(args=[(iv, iv_ty)] + list(zip(iter_names, rtypes)))
    _parse_block_body(L, blk)
    closing = L.next()
    attrs = {}
    cm = re.match(r"^\}\s*(\{.*\})?$", closing)
    if cm and cm.group(1):
        attrs = _parse_attr_dict(cm.group(1))
    results = _results_of(lhs, rtypes) if lhs else []
    return Op("scf.for", results, [lb, ub, step] + inits, attrs, [blk], line)


def _parse_if(lhs, body, L: _Lines, line) -> Op:
    m = re.match(rf"^({_SSA})\s*(?:->\s*\((.*)\))?\s*\{{$", body)
    if not m:
        raise UnsupportedTTIR(f"cannot parse scf.if: {line}")
    rtypes = [parse_type(t) for t in _split_top(m.group(2))] if m.group(2) else []
    then_blk = _parse_block_body(L)
    closing = L.next()
    regions = [then_blk]
    if closing.startswith("} else {"):
        regions.append(_parse_block_body(L))
        closing = L.next()
    results = _results_of(lhs, rtypes) if lhs else []
    return Op("scf.if", results, [m.group(1)], {}, regions, line)


_CMP_OPS = {"arith.cmpi", "arith.cmpf"}


def _parse_simple(lhs, name, body, line) -> Op:
    attrs: Dict[str, object] = {}
    if name in ("cf.cond_br", "cf.br"):
        parts = _split_top(body)
        operands = [x for x in parts if re.match(rf"^{_SSA}$", x)]
        dests = [x for x in parts if x.startswith("^")]
        if any("(" in d for d in dests) or len(dests) != (2 if name == "cf.cond_br" else 1):
            raise UnsupportedTTIR(f"branch with block arguments: {line}")
        return Op(name, [], operands, {"dests": dests}, [], line)
    if name in ("tt.return", "scf.yield", "tt.reduce.return", "tt.scan.return"):
        head, tys = _find_trailing_type(body)
        operands = [x.strip() for x in _split_top(head)] if head.strip() else []
        return Op(name, [], operands, attrs, [], line)
    head, tys = _find_trailing_type(body)
    # attribute dicts: either leading `{...}` (make_range) or trailing ones
    dicts = re.findall(r"\{[^{}]*\}", head)
    for d in dicts:
        attrs.update(_parse_attr_dict(d))
        head = head.replace(d, " ")
    head = head.strip()
    if name == "arith.constant":
        ty = parse_type(tys)
        attrs["value"] = head.strip()
        return Op(name, _results_of(lhs, [ty]), [], attrs, [], line)
    if name in ("tt.get_program_id", "tt.get_num_programs"):
        attrs["axis"] = {"x": 0, "y": 1, "z": 2}[head.strip()]
        return Op(name, _results_of(lhs, [parse_type(tys)]), [], attrs, [], line)
    if name in _CMP_OPS:
        parts = _split_top(head)
        attrs["predicate"] = parts[0]
        operands = parts[1:]
        opty = parse_type(tys)
        rty = Type(opty.shape, "i1", opty._tensor)
        attrs["operand_type"] = opty
        return Op(name, _results_of(lhs, [rty]), operands, attrs, [], line)
    # key = value attributes written inline (e.g. `inputPrecision = tf32`, `cacheModifier = ca`)
    parts = _split_top(head)
    operands = []
    for p in parts:
        if re.match(rf"^{_SSA}$", p):
            operands.append(p)
        elif "=" in p:
            k, v = p.split("=", 1)
            attrs[k.strip()] = _parse_attr_value(v.strip())
        elif p:
            attrs.setdefault("flags", []).append(p)
    rtypes = _result_types(name, tys, attrs)
    results = _results_of(lhs, rtypes) if lhs else []
    return Op(name, results, operands, attrs, [], line)


def _result_types(name: str, tys: str, attrs) -> List[Type]:
    """Result type(s) from the printed trailing type of each custom assembly format."""
    if not tys:
        return []
    if "->" in tys:
        # `a -> b` (splat, expand_dims, broadcast, dot, reshape, trans) : result after the arrow
        lhs_t, rhs_t = tys.rsplit("->", 1)
        attrs["operand_types"] = [parse_type(t) for t in _split_top(lhs_t.replace("*", ","))]
        return [parse_type(rhs_t)]
    if " to " in tys:
        a, b = tys.split(" to ")
        attrs["operand_types"] = [parse_type(a)]
        return [parse_type(b)]
    tlist = [parse_type(t) for t in _split_top(tys)]
    if name == "tt.addptr":
        attrs["operand_types"] = tlist
        return [tlist[0]]
    if name == "tt.load":
        p = tlist[0]
        return [Type(p.shape, p.pointee, p._tensor)]
    if name == "tt.store":
        attrs["operand_types"] = tlist
        return []
    if name == "arith.select":
        return [tlist[-1]]
    return [tlist[0]]
