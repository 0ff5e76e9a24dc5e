"""TEST INFRASTRUCTURE, NOT PRODUCT CODE.

ctypes binding of the CPU oracle (``tsb_oracle.cpp``): a restatement of what the
reference CPU backend of triton-shared computes for a lowered kernel.  Only
``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py``
may import this package; nothing under the product package does.

All wrappers take and return numpy arrays (host memory).
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = None

F32, F16, BF16 = 0, 1, 2


def build(reference_root=None):
    """Compile liborc.so; also the reference's own memrefCopy when a checkout of the reference is named
    (argument, or the environment variable TSB_REFERENCE_ROOT)."""
    subprocess.check_call(["make", "-s", "-C", HERE, "liborc.so"])
    ref = reference_root or os.environ.get("TSB_REFERENCE_ROOT", "")
    if ref and os.path.exists(os.path.join(ref, "backend/include/ExecutionEngine/CRunnerUtils.cpp")):
        subprocess.check_call(["make", "-s", "-C", HERE, "ref", f"REF={ref}"],
                              stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(HERE, "liborc.so")
        if not os.path.exists(path):
            build()
        L = ctypes.CDLL(path)
        i64, vp, ci = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
        L.orc_mask_dim.restype = i64
        L.orc_mask_dim.argtypes = [i64, i64, i64]
        L.orc_strided_copy.argtypes = [i64, ci, vp, vp, vp, vp, vp]
        L.orc_block_load.argtypes = [vp, i64, ci, vp, vp, i64, vp, vp, vp]
        L.orc_block_store.argtypes = [vp, i64, ci, vp, vp, i64, vp, vp]
        L.orc_vec_add.argtypes = [vp, vp, vp, i64, i64, i64, i64, ci]
        L.orc_softmax.argtypes = [vp, vp, i64, i64, i64, i64, i64, i64, ci]
        L.orc_layernorm_fwd.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, ctypes.c_float, i64, ci, i64, i64, ci]
        L.orc_matmul.argtypes = [vp, vp, vp, ci] + [i64] * 12 + [vp, i64, i64, ci]
        L.orc_reduce_rows.argtypes = [vp, vp] + [i64] * 8 + [ci]
        L.orc_reduce_all.argtypes = [vp, vp, i64, i64]
        L.orc_max_threads.restype = ci
        for f in (L.orc_strided_copy, L.orc_block_load, L.orc_block_store, L.orc_vec_add, L.orc_softmax,
                  L.orc_layernorm_fwd, L.orc_matmul, L.orc_reduce_rows, L.orc_reduce_all):
            f.restype = None
        _LIB = L
    return _LIB


def ref_lib():
    """The reference's own CRunnerUtils (memrefCopy) if it was compiled, else None."""
    global _REF
    if _REF is None:
        path = os.path.join(HERE, "_ref", "libcrunnerutils.so")
        if not os.path.exists(path):
            return None
        _REF = ctypes.CDLL(path)
        _REF.memrefCopy.restype = None
        _REF.memrefCopy.argtypes = [ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]
    return _REF


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _i64(seq):
    return np.asarray(list(seq), dtype=np.int64)


def max_threads():
    return int(lib().orc_max_threads())


def mask_dim(start, size, bound):
    return int(lib().orc_mask_dim(start, size, bound))


def block_load(base, sizes, strides, offset, dims=None, other=None):
    """Dense block (numpy array of shape `sizes`) read from the 1-D array `base`."""
    base = np.ascontiguousarray(base)
    out = np.empty(tuple(sizes), dtype=base.dtype)
    s, st = _i64(sizes), _i64(strides)
    d = _i64(dims) if dims is not None else None
    o = np.asarray([other], dtype=base.dtype) if other is not None else None
    lib().orc_block_load(_p(base), base.itemsize, len(sizes), _p(s), _p(st), offset, _p(d), _p(o), _p(out))
    return out


def block_store(base, sizes, strides, offset, value, dims=None):
    """Write `value` (shape `sizes`) into the 1-D array `base` in place."""
    assert base.flags.c_contiguous
    value = np.ascontiguousarray(value, dtype=base.dtype)
    s, st = _i64(sizes), _i64(strides)
    d = _i64(dims) if dims is not None else None
    lib().orc_block_store(_p(base), base.itemsize, len(sizes), _p(s), _p(st), offset, _p(d), _p(value))


def strided_copy(esize, sizes, src, src_strides, dst, dst_strides):
    s, a, b = _i64(sizes), _i64(src_strides), _i64(dst_strides)
    lib().orc_strided_copy(esize, len(sizes), _p(s), _p(src), _p(a), _p(dst), _p(b))


def vec_add(x, y, n=None, block=1024, pid_lo=0, pid_hi=None, threads=1, out=None):
    n = x.size if n is None else n
    grid = (n + block - 1) // block
    z = np.zeros_like(x) if out is None else out
    lib().orc_vec_add(_p(x), _p(y), _p(z), n, block, pid_lo, grid if pid_hi is None else pid_hi, threads)
    return z


def softmax(x, block, n_cols=None, row_lo=0, row_hi=None, threads=1, out=None):
    """x: 2-D float32 array whose row stride may exceed n_cols."""
    rows, cols = x.shape
    n_cols = cols if n_cols is None else n_cols
    assert x.strides[1] == 4
    y = np.zeros_like(x) if out is None else out
    lib().orc_softmax(_p(y), _p(x), x.strides[0] // 4, y.strides[0] // 4, n_cols, block, row_lo,
                      rows if row_hi is None else row_hi, threads)
    return y


def _dt(a):
    if a.dtype == np.float32:
        return F32
    if a.dtype == np.float16:
        return F16
    raise TypeError("bf16 arrays are passed as uint16 with dtype=BF16 given explicitly")


def layernorm_fwd(x, w, b, eps, block=1024, dtype=None, row_lo=0, row_hi=None, threads=1):
    """x: [M,N] (float16, float32, or uint16 holding bf16 with dtype=BF16). Returns y, mean, rstd."""
    M, N = x.shape
    dt = _dt(x) if dtype is None else dtype
    y = np.zeros_like(x)
    mean = np.zeros(M, dtype=np.float32)
    rstd = np.zeros(M, dtype=np.float32)
    lib().orc_layernorm_fwd(_p(x), _p(y), _p(w), _p(b), _p(mean), _p(rstd), x.strides[0] // x.itemsize, N,
                            eps, block, dt, row_lo, M if row_hi is None else row_hi, threads)
    return y, mean, rstd


def grouped_tiles(M, N, BM, BN, group_m):
    """(tile_m, tile_n) per program for the grouped ordering of python/examples/test_matmul.py:57-65."""
    num_m, num_n = -(-M // BM), -(-N // BN)
    pid = np.arange(num_m * num_n, dtype=np.int64)
    in_group = group_m * num_n
    gid = pid // in_group
    first = gid * group_m
    gsz = np.minimum(num_m - first, group_m)
    tm = first + (pid % gsz)
    tn = (pid % in_group) // gsz
    return np.stack([tm, tn], axis=1).astype(np.int32)


def matmul(a, b, dtype, BM=128, BN=256, BK=64, group_m=8, pid_lo=0, pid_hi=None, threads=1, tiles=None):
    """a: [M,K], b: [K,N] as uint16 bit patterns (or float16 arrays); returns c as the same kind."""
    M, K = a.shape
    K2, N = b.shape
    assert K == K2
    c = np.zeros((M, N), dtype=a.dtype)
    tiles = grouped_tiles(M, N, BM, BN, group_m) if tiles is None else tiles
    tiles = np.ascontiguousarray(tiles, dtype=np.int32)
    es = a.itemsize
    lib().orc_matmul(_p(a), _p(b), _p(c), dtype, M, N, K, a.strides[0] // es, a.strides[1] // es,
                     b.strides[0] // es, b.strides[1] // es, c.strides[0] // es, c.strides[1] // es,
                     BM, BN, BK, _p(tiles), pid_lo, len(tiles) if pid_hi is None else pid_hi, threads)
    return c


def reduce_rows(x_flat, M, n_valid, stride_m, stride_n, BM, BN, pid_lo=0, pid_hi=None, threads=1):
    out = np.zeros(M, dtype=np.float32)
    grid = -(-M // BM)
    lib().orc_reduce_rows(_p(x_flat), _p(out), M, n_valid, stride_m, stride_n, BM, BN, pid_lo,
                          grid if pid_hi is None else pid_hi, threads)
    return out


def reduce_all(x, block=1024):
    out = np.zeros(1, dtype=np.float32)
    x = np.ascontiguousarray(x, dtype=np.float32)
    lib().orc_reduce_all(_p(x), _p(out), x.size, block)
    return out[0]


# --------------------------------------------------------------------------------------------------
# Restatements in numpy of the lowered forms beyond the five configured workloads.  Every fold runs
# left to right over the reduced axis (one numpy operation per step, vectorised over the other
# axes), which is the order of the reference's linalg.reduce loops.

_F32 = np.float32


def fold(x, axis, comb):
    """tt.reduce with a single-op combiner: acc = comb(x_i, acc) from the combiner's identity, i
    ascending (ReduceConverter, ConversionPatterns.hpp:1203-1440; identities 1227-1278)."""
    x = np.asarray(x)
    fl = x.dtype.kind == "f"
    ident = {"addf": 0.0, "mulf": 1.0, "maxnumf": -np.inf, "maximumf": -np.inf, "minnumf": np.inf, "minimumf": np.inf,
             "addi": 0, "muli": 1, "andi": -1, "ori": 0, "xori": 0, "maxsi": np.iinfo(np.int32).min,
             "minsi": np.iinfo(np.int32).max}[comb]
    op = {"addf": np.add, "mulf": np.multiply, "maxnumf": np.fmax, "minnumf": np.fmin, "maximumf": np.maximum,
          "minimumf": np.minimum, "addi": np.add, "muli": np.multiply, "andi": np.bitwise_and, "ori": np.bitwise_or,
          "xori": np.bitwise_xor, "maxsi": np.maximum, "minsi": np.minimum}[comb]
    acc = np.full(np.take(x, 0, axis=axis).shape, ident, dtype=x.dtype)
    with np.errstate(all="ignore"):
        for i in range(x.shape[axis]):
            acc = op(np.take(x, i, axis=axis), acc).astype(x.dtype)
    return acc if fl else acc.astype(x.dtype)


def argfold(x, axis, want_max):
    """tl.argmax / tl.argmin: fold of (value, index) pairs from (-inf | +inf, -1); an element replaces the
    running pair when it is strictly better, or equal with a smaller index, so NaNs never win and a
    line of only -inf (+inf) keeps index -1 (ArgMinMaxBaseConverter, ConversionPatterns.hpp:1442-1769)."""
    x = np.asarray(x, dtype=_F32)
    shape = np.take(x, 0, axis=axis).shape
    bv = np.full(shape, -np.inf if want_max else np.inf, dtype=_F32)
    bi = np.full(shape, -1, dtype=np.int32)
    with np.errstate(invalid="ignore"):
        for i in range(x.shape[axis]):
            v = np.take(x, i, axis=axis)
            upd = ((v > bv) if want_max else (v < bv)) | ((v == bv) & (i < bi))
            bv, bi = np.where(upd, v, bv), np.where(upd, np.int32(i), bi)
    return bv, bi


def cumsum(x, axis):
    """tl.cumsum -> ttx.cumsum: out[i] = out[i-1] + x[i] along the axis, in the element type
    (CumSumConverter, ConversionPatterns.hpp:1941-2007)."""
    x = np.asarray(x)
    out = np.empty_like(x)
    run = np.zeros(np.take(x, 0, axis=axis).shape, dtype=x.dtype)
    idx = [slice(None)] * x.ndim
    for i in range(x.shape[axis]):
        run = (run + np.take(x, i, axis=axis)).astype(x.dtype)
        idx[axis] = i
        out[tuple(idx)] = run
    return out


def layernorm_bwd_dx(x, dy, w, mean, rstd):
    """Row-wise input gradient of LayerNorm in fp32 with separately rounded products, sums folded left
    to right: xhat = (x - mean) * rstd; wdy = w * dy; c1 = sum(xhat * wdy) / N; c2 = sum(wdy) / N;
    dx = (wdy - (xhat * c1 + c2)) * rstd (the dx kernel of the LayerNorm tutorial the reference's
    examples follow, without its lock-protected partial accumulation)."""
    x, dy, w = (np.asarray(a, dtype=_F32) for a in (x, dy, w))
    n = _F32(x.shape[1])
    xhat = ((x - mean[:, None]).astype(_F32) * rstd[:, None]).astype(_F32)
    wdy = (w[None, :] * dy).astype(_F32)
    c1 = (fold((xhat * wdy).astype(_F32), 1, "addf") / n).astype(_F32)
    c2 = (fold(wdy, 1, "addf") / n).astype(_F32)
    inner = ((xhat * c1[:, None]).astype(_F32) + c2[:, None]).astype(_F32)
    return ((wdy - inner).astype(_F32) * rstd[:, None]).astype(_F32)


def layernorm_bwd_dwdb(dw_part, db_part, block_m):
    """Column sums of the partial weight / bias gradients: lane accumulators over row blocks of
    `block_m`, then a left-to-right fold over the block's rows
    (test/Conversion/StructuredToMemref/kernel-05-layer-norm-dwdb.mlir)."""
    out = []
    for part in (dw_part, db_part):
        part = np.asarray(part, dtype=_F32)
        m = part.shape[0]
        acc = np.zeros((block_m, part.shape[1]), dtype=_F32)
        for r0 in range(0, m, block_m):
            blk = np.zeros_like(acc)
            blk[: min(block_m, m - r0)] = part[r0:r0 + block_m]
            acc = (acc + blk).astype(_F32)
        out.append(fold(acc, 0, "addf"))
    return out
