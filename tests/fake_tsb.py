"""Host-memory stand-in for libtsb200.so, for CPU-only tests of the host logic.

TEST INFRASTRUCTURE.  It lets the plan compiler, the descriptor evaluation and
the program-range partitioning be exercised end to end without a GPU: the
Triton driver plugin runs unchanged, but the ctypes library object is replaced
by ``FakeLib`` whose entry points take the same arguments and execute on host
pointers.  ``tsb_elementwise`` is emulated in numpy from the descriptors (the
same definition as include/tsb200.h); the family entry points call the CPU
oracle with the arguments they were given.  Nothing here is reachable from the
product package.
"""
import ctypes

import numpy as np

import oracle
from triton_shared_b200.backend import runtime as rt

_SIZE = {0: 4, 1: 2, 2: 2, 3: 4, 4: 2, 5: 1, 6: 1, 7: 8, 9: 4, 10: 2, 11: 1}
_OPNAME = {v: k for k, v in rt.OPCODES.items()}
_CMPF = {v: k for k, v in rt.CMPF.items()}
_CMPI = {v: k for k, v in rt.CMPI.items()}


def _host_array(addr, nbytes):
    return np.ctypeslib.as_array((ctypes.c_uint8 * nbytes).from_address(addr))


def _bf16_to_f32(u16):
    return (u16.astype(np.uint32) << 16).view(np.float32)


def _f32_to_bf16(f):
    u = f.astype(np.float32).view(np.uint32)
    lsb = (u >> 16) & 1
    return ((u + 0x7fff + lsb) >> 16).astype(np.uint16)


def _round_to(f, dt):
    if dt == 1:
        return f.astype(np.float16).astype(np.float32)
    if dt == 2:
        return _bf16_to_f32(_f32_to_bf16(f))
    return f.astype(np.float32)


def _is_float(dt):
    return dt in (0, 1, 2)


class HostMemory:
    """Replacement for the driver's device-memory provider: plain host arrays."""
    host_pointers = True  # the stand-in executes on host memory: host tensors are what it wants

    def __init__(self):
        self._scratch = None
        self._tables = {}
        self._status = np.zeros(4, dtype=np.int32)

    def scratch(self, nbytes, stream=0):
        if self._scratch is None or self._scratch.size < nbytes:
            self._scratch = np.zeros(max(nbytes, 1024), dtype=np.uint8)
        return self._scratch.ctypes.data

    def table(self, key, host, stream=0):
        t = self._tables.get(key)
        if t is None:
            t = self._tables[key] = np.ascontiguousarray(host)
        return t.ctypes.data

    def status(self):
        return self._status.ctypes.data

    def read_status(self):
        return self._status.tolist()

    def clear_status(self):
        self._status[:] = 0


class _Regs(dict):
    """Register file of the elementwise VM: numbers, TSB_REG_ACC (-1, the previous result) and
    TSB_REG_IMM (-2, the op's imm2)."""

    def __init__(self, lanes):
        super().__init__()
        self.lanes, self.acc, self.imm = lanes, np.zeros(lanes, dtype=np.uint32), np.uint32(0)

    def __getitem__(self, r):
        if r == -1:
            return self.acc
        if r == -2:
            return np.full(self.lanes, self.imm, dtype=np.uint32)
        return dict.__getitem__(self, r)

    def write(self, r, v):
        self.acc = v
        if r >= 0:
            self[r] = v


class FakeLib:
    """Same entry points as libtsb200.so, executing on host memory."""

    def __init__(self):
        self.calls = []
        self._err = b""

    def tsb_last_error(self):
        return self._err

    def tsb_version(self):
        return 1000

    def tsb_sm_count(self):
        return 148

    # ---------------------------------------------------------------- generic engine
    def tsb_elementwise(self, accs, n_acc, ops, n_ops, grid, pid_lo, pid_hi, stream):
        self.calls.append(("tsb_elementwise", pid_lo, pid_hi))
        g = [max(int(grid[i]), 1) for i in range(3)]
        rank = accs[0].rank
        sizes = [int(accs[0].sizes[d]) for d in range(rank)]
        lanes = int(np.prod(sizes))
        idx = np.unravel_index(np.arange(lanes), sizes)
        import itertools
        body = [ops[k] for k in range(n_ops)]
        trips = []
        while body and _OPNAME[body[0].opcode] == "loop_begin":  # a perfect nest around the whole body
            assert _OPNAME[body[-1].opcode] == "loop_end" and body[-1].a == body[0].a == len(trips)
            trips.append(int(body[0].imm))
            body = body[1:-1]
        for prog in range(pid_lo, pid_hi):
            p = (prog % g[0], (prog // g[0]) % g[1], prog // (g[0] * g[1]))
            for its in itertools.product(*[range(t) for t in trips]):
                it = tuple(its) + (0,) * (4 - len(its))
                state = [self._acc_state(accs[a], p, rank, sizes, idx, lanes, it) for a in range(n_acc)]
                regs = _Regs(lanes)
                for o in body:
                    name = _OPNAME[o.opcode]
                    regs.imm = np.uint32(o.imm2)
                    if name == "load":
                        A = accs[o.a]
                        elem, valid = state[o.a]
                        if o.imm & rt.MEM_INDEX:
                            elem = elem + regs[o.b].view(np.int32).astype(np.int64)
                        if o.imm & rt.MEM_MASK:
                            valid = valid & ((regs[o.c] & 1) != 0)
                        if A.is_store == 2:
                            v = valid.astype(np.uint32)
                        elif A.is_store == 3:
                            v = elem.astype(np.int64).astype(np.uint32)
                        else:
                            v = self._load(A, elem, valid)
                        regs.write(o.dst, v)
                    elif name == "store":
                        A = accs[o.a]
                        elem, valid = state[o.a]
                        if o.imm & rt.MEM_INDEX:
                            elem = elem + regs[o.c].view(np.int32).astype(np.int64)
                        if o.imm & rt.MEM_MASK:
                            valid = valid & ((regs[o.dst] & 1) != 0)
                        self._store(A, elem, valid, regs[o.b])
                    elif name == "reduce":
                        # fold over all lanes of the program (left to right); every lane takes the total
                        comb = _OPNAME[o.imm]
                        src = regs[o.a]
                        op = type("O", (), {"type": o.type, "a": 0, "b": 1, "c": 0, "imm": 0, "imm2": 0})()
                        tot = src[0:1].copy()
                        for j in range(1, lanes):
                            tot = self._alu(comb, op, {0: tot, 1: src[j:j + 1]}, 1)
                        regs.write(o.dst, np.full(lanes, tot[0], dtype=np.uint32))
                    else:
                        regs.write(o.dst, self._alu(name, o, regs, lanes))
        return 0

    @staticmethod
    def _acc_state(A, p, rank, sizes, idx, lanes, it=(0, 0, 0, 0)):
        """(element index, validity) of every lane of the iteration space for program p (and loop counters it)."""
        off = A.offset0 + sum(A.offset_pid[k] * p[k] for k in range(3)) + sum(A.offset_loop[l] * it[l] for l in range(4))
        valid = np.ones(lanes, dtype=bool)
        elem = np.full(lanes, off, dtype=np.int64)
        for w in range(A.n_wrap):
            W = A.wrap[w]
            wo = W.offset0 + sum(W.offset_pid[k] * p[k] for k in range(3))
            inner = wo + idx[W.dim] * W.stride
            q = np.abs(inner) // W.modulus * np.sign(inner)
            elem = elem + W.scale * (inner - q * W.modulus)  # remainder with the dividend's sign
        for d in range(rank):
            elem = elem + idx[d] * A.strides[d]
            if A.masked[d]:
                st = A.mask_start0[d] + sum(A.mask_start_pid[d][k] * p[k] for k in range(3)) + \
                    sum(A.mask_start_loop[d][l] * it[l] for l in range(4))
                dim = max(min(st + sizes[d], A.mask_bound[d]), st) - st
                valid &= idx[d] < dim
        return elem, valid

    def tsb_block_program(self, accs, n_acc, ops, n_ops, reg_masks, n_regs, grid, pid_lo, pid_hi, stream):
        """Registers are numpy arrays of the iteration-space shape with absent dims collapsed to 1."""
        self.calls.append(("tsb_block_program", pid_lo, pid_hi))
        g = [max(int(grid[i]), 1) for i in range(3)]
        rank = accs[0].rank
        sizes = [int(accs[0].sizes[d]) for d in range(rank)]
        lanes = int(np.prod(sizes))
        idx = np.unravel_index(np.arange(lanes), sizes)
        shape_of = lambda m: tuple(sizes[d] if m & (1 << d) else 1 for d in range(rank))
        take = lambda full, m: full.reshape(sizes)[tuple(slice(None) if m & (1 << d) else slice(0, 1) for d in range(rank))]
        ident = {"addf": 0, "mulf": 0x3f800000, "maxnumf": 0xff800000, "maximumf": 0xff800000, "minnumf": 0x7f800000,
                 "minimumf": 0x7f800000, "muli": 1, "andi": 0xffffffff, "maxsi": 0x80000000, "minsi": 0x7fffffff,
                 "minui": 0xffffffff}
        for prog in range(pid_lo, pid_hi):
            p = (prog % g[0], (prog // g[0]) % g[1], prog // (g[0] * g[1]))
            R = {}
            it, trip, begin = [0] * 4, [0] * 4, [0] * 4
            k = 0
            while k < n_ops:
                o = ops[k]
                name = _OPNAME[o.opcode]
                if name == "loop_begin":
                    it[o.a], trip[o.a], begin[o.a] = 0, int(o.imm), k + 1
                    k = k + 1 if trip[o.a] > 0 else o.b
                    continue
                if name == "loop_end":
                    it[o.a] += 1
                    k = begin[o.a] if it[o.a] < trip[o.a] else k + 1
                    continue
                k += 1
                if name == "load":
                    A = accs[o.a]
                    elem, valid = self._acc_state(A, p, rank, sizes, idx, lanes, it)
                    bcast = lambda r: np.ascontiguousarray(np.broadcast_to(R[r], sizes)).reshape(-1)
                    if o.imm2 & rt.MEM_INDEX:
                        elem = elem + bcast(o.b).view(np.int32).astype(np.int64)
                    if o.imm2 & rt.MEM_MASK:
                        valid = valid & ((bcast(o.c) & 1) != 0)
                    if A.is_store == 2:
                        full = valid.astype(np.uint32)
                    elif A.is_store == 3:
                        full = elem.astype(np.uint32)
                    else:
                        full = self._load(A, elem, valid)
                    R[o.dst] = take(full, reg_masks[o.dst]).copy()
                elif name == "store":
                    A = accs[o.a]
                    elem, valid = self._acc_state(A, p, rank, sizes, idx, lanes, it)
                    bcast = lambda r: np.ascontiguousarray(np.broadcast_to(R[r], sizes)).reshape(-1)
                    if o.imm2 & rt.MEM_INDEX:
                        elem = elem + bcast(o.c).view(np.int32).astype(np.int64)
                    if o.imm2 & rt.MEM_MASK:
                        valid = valid & ((bcast(o.dst) & 1) != 0)
                    m = int(o.imm)
                    val = np.broadcast_to(R[o.b], shape_of(m))
                    sel = take(np.arange(lanes), m).reshape(-1)  # one lane per walked element
                    self._store(A, elem[sel], valid[sel], np.ascontiguousarray(val).reshape(-1))
                elif name == "argreduce":
                    d, want_max = int(o.imm2), int(o.imm) != 0
                    shp = tuple(max(a, b) for a, b in zip(R[o.a].shape, R[o.b].shape))
                    val = np.broadcast_to(R[o.a], shp).view(np.float32)
                    ind = np.broadcast_to(R[o.b], shp).view(np.int32)
                    # left-to-right fold from (-inf | +inf, -1): strictly better, or equal with a smaller index
                    n = val.shape[d]
                    bv = np.full(np.take(val, [0], axis=d).shape, -np.inf if want_max else np.inf, dtype=np.float32)
                    bi = np.full(bv.shape, -1, dtype=np.int32)
                    with np.errstate(invalid="ignore"):
                        for j in range(n):
                            v, ix = np.take(val, [j], axis=d), np.take(ind, [j], axis=d)
                            upd = ((v > bv) if want_max else (v < bv)) | ((v == bv) & (ix < bi))
                            bv, bi = np.where(upd, v, bv), np.where(upd, ix, bi)
                    R[o.dst] = np.ascontiguousarray(bv.astype(np.float32)).view(np.uint32).copy()
                    R[o.c] = np.ascontiguousarray(bi.astype(np.int32)).view(np.uint32)
                elif name == "scan":
                    src = R[o.a]
                    d = int(o.imm2)
                    if _OPNAME[o.imm] == "addf":
                        acc = np.cumsum(src.view(np.float32), axis=d, dtype=np.float32).view(np.uint32)
                    else:
                        acc = np.cumsum(src.view(np.int32).astype(np.int64), axis=d).astype(np.int32).view(np.uint32)
                    R[o.dst] = np.ascontiguousarray(acc)
                elif name == "reduce":
                    comb, d = _OPNAME[o.imm], int(o.imm2)
                    src = R[o.a]
                    acc = np.full(tuple(1 if i == d else n for i, n in enumerate(src.shape)), ident.get(comb, 0), dtype=np.uint32)
                    op = type("O", (), {"type": o.type, "a": 0, "b": 1, "c": 0, "imm": 0, "imm2": 0})()
                    for j in range(src.shape[d]):
                        sl = np.take(src, [j], axis=d)
                        flat = self._alu(comb, op, {0: np.ascontiguousarray(sl).reshape(-1), 1: acc.reshape(-1)}, sl.size)
                        acc = flat.reshape(acc.shape)
                    R[o.dst] = acc
                else:
                    shp = shape_of(reg_masks[o.dst])
                    n = int(np.prod(shp))
                    regs = {}
                    unary = {"exp", "exp2", "log", "log2", "sqrt", "rsqrt", "sin", "cos", "tanh", "erf", "absf", "negf",
                             "floor", "ceil", "absi", "cast", "bitcast", "mov"}
                    used = () if name == "const" else ((o.a,) if name in unary else
                                                      ((o.a, o.b, o.c) if name in ("select", "fma") else (o.a, o.b)))
                    for r in used:
                        regs[r] = np.ascontiguousarray(np.broadcast_to(R[r], shp)).reshape(-1)
                    R[o.dst] = self._alu(name, o, regs, n).reshape(shp)
        return 0

    def _load(self, A, elem, valid):
        es = _SIZE[A.dtype]
        out = np.zeros(elem.shape, dtype=np.uint32)
        fill = np.uint64(A.other_bits) if A.has_other else np.uint64(0)
        raw = np.zeros(elem.shape, dtype=np.uint64)
        for i in np.nonzero(valid)[0]:
            b = _host_array(A.base + int(elem[i]) * es, es)
            raw[i] = int.from_bytes(b.tobytes(), "little")
        raw[~valid] = fill
        return self._to_reg(raw, A.dtype)

    @staticmethod
    def _to_reg(raw, dt):
        if dt in (0, 3, 9):
            return raw.astype(np.uint32)
        if dt == 1:
            return raw.astype(np.uint16).view(np.float16).astype(np.float32).view(np.uint32)
        if dt == 2:
            return _bf16_to_f32(raw.astype(np.uint16)).view(np.uint32)
        if dt == 4:
            return raw.astype(np.uint16).view(np.int16).astype(np.int32).view(np.uint32)
        if dt == 5:
            return raw.astype(np.uint8).view(np.int8).astype(np.int32).view(np.uint32)
        return raw.astype(np.uint32)

    def _store(self, A, elem, valid, reg):
        es = _SIZE[A.dtype]
        dt = A.dtype
        if dt in (0, 3, 9):
            bits = reg.astype(np.uint32)
        elif dt == 1:
            bits = reg.view(np.float32).astype(np.float16).view(np.uint16)
        elif dt == 2:
            bits = _f32_to_bf16(reg.view(np.float32))
        elif dt == 6:
            bits = (reg & 1).astype(np.uint8)
        elif dt == 7:  # 64-bit integers are held as their low 32 bits and stored sign-extended
            bits = reg.view(np.int32).astype(np.int64).view(np.uint64)
        else:
            bits = reg.astype(np.uint32)
        for i in np.nonzero(valid)[0]:
            dst = _host_array(A.base + int(elem[i]) * es, es)
            dst[:] = np.frombuffer(int(bits[i]).to_bytes(8, "little")[:es], dtype=np.uint8)

    def _alu(self, name, o, R, lanes):
        dt = o.type
        f = lambda r: R[r].view(np.float32)
        i = lambda r: R[r].view(np.int32)
        u = lambda r: R[r]
        with np.errstate(all="ignore"):
            if name == "const":
                return np.full(lanes, o.imm, dtype=np.uint32)
            if name == "mov":
                return R[o.a].copy()
            fb = {"addf": np.add, "subf": np.subtract, "mulf": np.multiply, "divf": np.divide,
                  "maxnumf": np.fmax, "minnumf": np.fmin, "maximumf": np.maximum, "minimumf": np.minimum,
                  "remf": np.fmod}
            if name in fb:
                return _round_to(fb[name](f(o.a), f(o.b)).astype(np.float32), dt).view(np.uint32)
            fu = {"exp": np.exp, "exp2": np.exp2, "log": np.log, "log2": np.log2, "sqrt": np.sqrt,
                  "sin": np.sin, "cos": np.cos, "tanh": np.tanh, "absf": np.abs, "negf": np.negative,
                  "floor": np.floor, "ceil": np.ceil}
            if name in fu:
                return _round_to(fu[name](f(o.a)).astype(np.float32), dt).view(np.uint32)
            if name == "rsqrt":
                return _round_to((np.float32(1) / np.sqrt(f(o.a))).astype(np.float32), dt).view(np.uint32)
            if name == "erf":
                import math
                return _round_to(np.array([math.erf(x) for x in f(o.a)], dtype=np.float32), dt).view(np.uint32)
            if name == "fma":
                r = (f(o.a).astype(np.float64) * f(o.b).astype(np.float64) + f(o.c).astype(np.float64))
                return _round_to(r.astype(np.float32), dt).view(np.uint32)
            ib = {"addi": lambda a, b: a + b, "subi": lambda a, b: a - b, "muli": lambda a, b: a * b,
                  "andi": lambda a, b: a & b, "ori": lambda a, b: a | b, "xori": lambda a, b: a ^ b}
            if name in ib:
                return self._wrap(ib[name](u(o.a).astype(np.uint64), u(o.b).astype(np.uint64)).astype(np.uint32), dt)
            if name in ("divsi", "remsi", "minsi", "maxsi"):
                a, b = i(o.a).astype(np.int64), i(o.b).astype(np.int64)
                bz = np.where(b == 0, 1, b)
                q = np.abs(a) // np.abs(bz) * np.sign(a) * np.sign(bz)
                r = {"divsi": q, "remsi": a - q * bz, "minsi": np.minimum(a, b), "maxsi": np.maximum(a, b)}[name]
                return self._wrap(r.astype(np.int32).view(np.uint32), dt)
            if name in ("shli", "shrsi", "shrui", "divui", "remui", "minui", "maxui"):
                a64, b64 = u(o.a).astype(np.uint64), u(o.b).astype(np.uint64)
                sh = np.minimum(b64, 63)
                bz = np.where(b64 == 0, 1, b64)
                r = {"shli": np.where(b64 >= 32, 0, a64 << sh), "shrui": np.where(b64 >= 32, 0, a64 >> sh),
                     "shrsi": (i(o.a).astype(np.int64) >> np.minimum(b64, 31).astype(np.int64)).astype(np.uint64),
                     "divui": np.where(b64 == 0, 0, a64 // bz), "remui": np.where(b64 == 0, 0, a64 % bz),
                     "minui": np.minimum(a64, b64), "maxui": np.maximum(a64, b64)}[name]
                return self._wrap((r & 0xffffffff).astype(np.uint32), dt)
            if name == "absi":
                return self._wrap(np.abs(i(o.a)).view(np.uint32), dt)
            if name == "cmpf":
                a, b = f(o.a), f(o.b)
                un = np.isnan(a) | np.isnan(b)
                pred = _CMPF[o.imm]
                base = {"eq": a == b, "gt": a > b, "ge": a >= b, "lt": a < b, "le": a <= b, "ne": a != b,
                        "rd": np.ones_like(un), "no": np.zeros_like(un)}[pred[1:]]
                r = (~un & base) if pred[0] == "o" else (un | base)
                if pred == "ord":
                    r = ~un
                if pred == "uno":
                    r = un
                return r.astype(np.uint32)
            if name == "cmpi":
                pred = _CMPI[o.imm]
                a, b = (i(o.a), i(o.b)) if pred[0] == "s" or pred in ("eq", "ne") else (u(o.a), u(o.b))
                r = {"eq": a == b, "ne": a != b, "lt": a < b, "le": a <= b, "gt": a > b, "ge": a >= b}[pred[-2:]]
                return r.astype(np.uint32)
            if name == "select":
                return np.where((R[o.a] & 1) != 0, R[o.b], R[o.c])
            if name == "bitcast":
                return R[o.a].copy()
            if name == "cast":
                src, mode = int(o.imm), int(o.imm2)
                if _is_float(src) and _is_float(dt):
                    return _round_to(f(o.a), dt).view(np.uint32)
                if not _is_float(src) and _is_float(dt):
                    v = u(o.a).astype(np.float64) if (mode == 1 or src in (9, 10, 11, 6)) else i(o.a).astype(np.float64)
                    return _round_to(v.astype(np.float32), dt).view(np.uint32)
                if _is_float(src) and not _is_float(dt):
                    return self._wrap(np.trunc(f(o.a)).astype(np.int64).astype(np.uint32), dt)
                v = u(o.a)
                if mode == 1:
                    v = v & {1: 0xff, 2: 0xffff, 4: 0xffffffff}[_SIZE[src]]
                    if src == 6:
                        v = v & 1
                return self._wrap(v.astype(np.uint32), dt)
        raise NotImplementedError(name)

    @staticmethod
    def _wrap(x, dt):
        x = x.astype(np.uint32)
        if dt == 4:
            return x.astype(np.uint16).view(np.int16).astype(np.int32).view(np.uint32)
        if dt == 10:
            return x & 0xffff
        if dt == 5:
            return x.astype(np.uint8).view(np.int8).astype(np.int32).view(np.uint32)
        if dt == 11:
            return x & 0xff
        if dt == 6:
            return x & 1
        return x

    def tsb_block_copy(self, src, dst, grid, pid_lo, pid_hi, stream):
        raise NotImplementedError

    # ---------------------------------------------------------------- families -> oracle
    def tsb_softmax_rows(self, inp, out, dtype, is_, os_, n_cols, block, row_lo, row_hi, stream):
        self.calls.append(("tsb_softmax_rows", row_lo, row_hi))
        oracle.lib().orc_softmax(out, inp, is_, os_, n_cols, block, row_lo, row_hi, 1)
        return 0

    def tsb_layernorm_fwd(self, x, y, w, b, mean, rstd, dt, xs, ys, n, eps, row_lo, row_hi, stream):
        self.calls.append(("tsb_layernorm_fwd", row_lo, row_hi))
        assert xs == ys
        oracle.lib().orc_layernorm_fwd(x, y, w, b, mean, rstd, xs, n, eps, 1024, {0: 0, 1: 1, 2: 2}[dt], row_lo, row_hi, 1)
        return 0

    def tsb_reduce_rows_scratch_bytes(self, n_rows, n_valid, sm, sn):
        return 4 * n_rows if sm == 1 else 0

    def tsb_reduce_rows(self, x, out, sm, sn, out_stride, n_valid, row_lo, row_hi, scratch, stream):
        self.calls.append(("tsb_reduce_rows", row_lo, row_hi))
        assert out_stride == 1
        oracle.lib().orc_reduce_rows(x, out, row_hi, n_valid, sm, sn, 1, 64, row_lo, row_hi, 1)
        return 0

    def tsb_reduce_all(self, x, out, n, stride, stream):
        self.calls.append(("tsb_reduce_all", 0, 1))
        assert stride == 1
        oracle.lib().orc_reduce_all(x, out, n, 1024)
        return 0

    def tsb_gemm(self, a, b, c, dt, M, N, K, sam, sak, sbk, sbn, scm, scn, bm, bn, bk, tiles, n_prog, lo, hi,
                 status, stream):
        self.calls.append(("tsb_gemm", lo, hi))
        if dt == 0:  # fp32 operands: the oracle's matmul is 16-bit only; numpy per tile
            t = np.ctypeslib.as_array((ctypes.c_int32 * (2 * n_prog)).from_address(tiles)).reshape(-1, 2)
            elem = lambda base, n: np.ctypeslib.as_array((ctypes.c_float * n).from_address(int(base)))
            for pid in range(lo, hi):
                r0, c0 = int(t[pid][0]) * bm, int(t[pid][1]) * bn
                r1, c1 = min(r0 + bm, M), min(c0 + bn, N)
                if r1 <= r0 or c1 <= c0:
                    continue
                ri, ci, ki = np.arange(r0, r1), np.arange(c0, c1), np.arange(K)
                Af = np.array([[elem(a + 4 * (r * sam + k * sak), 1)[0] for k in ki] for r in ri], dtype=np.float32)
                Bf = np.array([[elem(b + 4 * (k * sbk + cc * sbn), 1)[0] for cc in ci] for k in ki], dtype=np.float32)
                Cf = Af @ Bf
                for i, r in enumerate(ri):
                    for j, cc in enumerate(ci):
                        elem(c + 4 * (r * scm + cc * scn), 1)[0] = Cf[i, j]
            return 0
        oracle.lib().orc_matmul(a, b, c, {1: 1, 2: 2}[dt], M, N, K, sam, sak, sbk, sbn, scm, scn, bm, bn, bk,
                                tiles, lo, hi, 1)
        return 0


    def _gemm_paired(self, a, b, c, dt, M, N, K, sam, sak, sbk, sbn, scm, scn, bm, bn, bk, pairs, n_pairs, status, stream):
        self.calls.append(("tsb_gemm_paired", 0, n_pairs))
        if sak != 1 or sam % 8 or (sbn == 1 and (sbk % 8 or bn % 128)) or (sbn != 1 and (sbk != 1 or sbn % 8)) or bm != 128:
            return -2
        pr = np.ctypeslib.as_array((ctypes.c_int32 * (2 * n_pairs)).from_address(pairs)).reshape(-1, 2)
        tiles = []
        for tm, tn in pr:
            tiles += [(tm, tn), (tm + 1, tn)]
        t = np.ascontiguousarray(np.asarray(tiles, dtype=np.int32))
        oracle.lib().orc_matmul(a, b, c, {1: 1, 2: 2}[dt], M, N, K, sam, sak, sbk, sbn, scm, scn, bm, bn, bk,
                                t.ctypes.data, 0, len(tiles), 1)
        return 0

    tsb_gemm_paired = _gemm_paired


class fake_device:
    """Context manager: route the driver plugin to FakeLib + host memory."""

    def __enter__(self):
        from triton_shared_b200.backend.driver import B200Launcher
        self._old_lib, self._old_mem = rt._lib, B200Launcher.memory
        self.lib = rt._lib = FakeLib()
        B200Launcher.memory = HostMemory()
        return self.lib

    def __exit__(self, *exc):
        from triton_shared_b200.backend.driver import B200Launcher
        rt._lib, B200Launcher.memory = self._old_lib, self._old_mem
        return False
