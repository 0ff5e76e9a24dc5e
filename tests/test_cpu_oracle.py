"""CPU tests of the oracle: pinned against the reference's own strided-copy routine
(when it was compiled from the reference checkout), against the exact known answers of
the reference's tests, and against golden vectors produced by the reference's example
kernels under Triton's interpreter."""
import ctypes
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def gold():
    return np.load(os.path.join(HERE, "golden", "reference_kernels.npz"))


# ---- the element-by-element strided copy vs the reference's memrefCopy --------------------
class _Memref(ctypes.Structure):
    """StridedMemRefType<char, 3>: basePtr, data, offset, sizes[3], strides[3]."""
    _fields_ = [("base", ctypes.c_void_p), ("data", ctypes.c_void_p), ("offset", ctypes.c_int64),
                ("sizes", ctypes.c_int64 * 3), ("strides", ctypes.c_int64 * 3)]


class _Unranked(ctypes.Structure):
    _fields_ = [("rank", ctypes.c_int64), ("desc", ctypes.c_void_p)]


def _memref(arr, rank, offset, sizes, strides):
    # sizes then strides are laid out contiguously after `offset` for the given rank
    buf = (ctypes.c_int64 * (3 + 2 * rank))()
    buf[0] = arr.ctypes.data
    buf[1] = arr.ctypes.data
    buf[2] = offset
    for d in range(rank):
        buf[3 + d] = sizes[d]
        buf[3 + rank + d] = strides[d]
    return buf


def test_strided_copy_matches_reference_memrefcopy(oracle_lib):
    ref = oracle_lib.ref_lib()
    if ref is None:
        pytest.skip("reference checkout not present: oracle/_ref was not built")
    rng = np.random.default_rng(0)
    for case in range(60):
        rank = int(rng.integers(1, 4))
        esize = int(rng.choice([1, 2, 4, 8]))
        sizes = [int(rng.integers(0 if case % 7 == 0 else 1, 6)) for _ in range(rank)]
        sstr = [int(rng.integers(1, 9)) for _ in range(rank)]
        dstr = [int(rng.integers(1, 9)) for _ in range(rank)]
        span_s = sum(max(s - 1, 0) * st for s, st in zip(sizes, sstr)) + 8
        span_d = sum(max(s - 1, 0) * st for s, st in zip(sizes, dstr)) + 8
        src = rng.integers(0, 255, size=span_s * esize, dtype=np.uint8)
        d1 = np.full(span_d * esize, 7, dtype=np.uint8)
        d2 = d1.copy()
        so, do = int(rng.integers(0, 4)), int(rng.integers(0, 4))
        ms, md = _memref(src, rank, so, sizes, sstr), _memref(d1, rank, do, sizes, dstr)
        us, ud = _Unranked(rank, ctypes.addressof(ms)), _Unranked(rank, ctypes.addressof(md))
        ref.memrefCopy(esize, ctypes.byref(us), ctypes.byref(ud))
        oracle_lib.strided_copy(esize, sizes, src[so * esize:], sstr, d2[do * esize:], dstr)
        assert np.array_equal(d1, d2), (rank, esize, sizes, sstr, dstr)


# ---- mask dims and the fill rule ------------------------------------------------------------
def test_mask_dim_formula(oracle_lib):
    """dims = max(min(start + size, bound), start) - start (lib/Analysis/MaskAnalysis.cpp:583-585)."""
    md = oracle_lib.mask_dim
    assert md(96 * 1024, 1024, 98_432) == 128  # last of the 97 programs of the vec-add config
    assert md(0, 1024, 98_432) == 1024
    assert md(100, 4, 4) == 0  # fully masked: start beyond the bound
    assert md(0, 1024, 781) == 781
    assert md(5, 8, -3) == 0  # negative bound clamps to empty
    assert md(-4, 8, 2) == 6  # signed arithmetic, lower bound implicit


def test_block_load_fill_rule(oracle_lib):
    """`other` fills the block only when a dim is short (StructuredToMemref.cpp:192-224, 809-813)."""
    base = np.arange(40, dtype=np.int32)
    full = oracle_lib.block_load(base, (4,), (1,), 3, dims=(4,), other=-1)
    assert full.tolist() == [3, 4, 5, 6]
    short = oracle_lib.block_load(base, (4,), (1,), 3, dims=(2,), other=-1)
    assert short.tolist() == [3, 4, -1, -1]
    empty = oracle_lib.block_load(base, (4,), (1,), 100, dims=(0,), other=-1)
    assert empty.tolist() == [-1, -1, -1, -1]  # python/examples/test_mask.py:39
    blk = oracle_lib.block_load(base, (2, 4), (8, 2), 1, dims=(2, 3), other=0)
    assert blk.tolist() == [[1, 3, 5, 0], [9, 11, 13, 0]]


def test_block_store_clips(oracle_lib):
    out = np.full(8, -2, dtype=np.int32)
    oracle_lib.block_store(out, (8,), (1,), 0, np.arange(8, dtype=np.int32), dims=(4,))
    assert out.tolist() == [0, 1, 2, 3, -2, -2, -2, -2]  # python/examples/test_mask.py:58 shape


def test_known_answer_2x_plus_1(oracle_lib):
    """python/examples/test_load_2d_tensor_block.py:76-78: out = 2*x + 1 on arange, block by block."""
    x = np.arange(6 * 8, dtype=np.int32)
    out = np.zeros_like(x)
    for pm in range(3):
        for pn in range(2):
            off = pm * 2 * 8 + pn * 4
            blk = oracle_lib.block_load(x, (2, 4), (8, 1), off)
            oracle_lib.block_store(out, (2, 4), (8, 1), off, 2 * blk + 1)
    assert np.array_equal(out, 2 * x + 1)


# ---- kernels vs golden vectors from the reference's example kernels --------------------------
def test_vec_add_golden_bit_exact(oracle_lib, gold):
    z = oracle_lib.vec_add(gold["add_x"], gold["add_y"], 5000, 1024)
    assert np.array_equal(z.view(np.uint32), gold["add_out"].view(np.uint32))


def test_vec_add_config_and_threads(oracle_lib):
    """Configured workload 1: n = 98,432, 97 programs, last block 128 valid; thread count does not change results."""
    rng = np.random.default_rng(0)
    x, y = rng.random(98_432, dtype=np.float32), rng.random(98_432, dtype=np.float32)
    z1 = oracle_lib.vec_add(x, y, 98_432, 1024, threads=1)
    z4 = oracle_lib.vec_add(x, y, 98_432, 1024, threads=4)
    assert np.array_equal(z1, x + y) and np.array_equal(z1, z4)
    part = np.zeros_like(x)
    oracle_lib.vec_add(x, y, 98_432, 1024, pid_lo=0, pid_hi=48, out=part)
    oracle_lib.vec_add(x, y, 98_432, 1024, pid_lo=48, pid_hi=97, out=part)
    assert np.array_equal(part, z1)


def test_softmax_golden(oracle_lib, gold):
    y = oracle_lib.softmax(gold["sm_x"], 1024)
    np.testing.assert_allclose(y, gold["sm_out"], rtol=2e-6, atol=1e-9)
    np.testing.assert_allclose(y.sum(axis=1), 1.0, rtol=1e-5)


def test_layernorm_golden(oracle_lib, gold):
    y, mean, rstd = oracle_lib.layernorm_fwd(gold["ln_x"], gold["ln_w"], gold["ln_b"], 1e-5, 1024)
    np.testing.assert_allclose(mean, gold["ln_mean"], rtol=1e-5, atol=1e-7)
    np.testing.assert_allclose(rstd, gold["ln_rstd"], rtol=1e-5)
    # outputs are fp16: allow one unit in the last place where the fp32 mean/rstd differ in the last bit
    d = np.abs(y.astype(np.float32) - gold["ln_y"].astype(np.float32))
    assert d.max() <= 2e-3 and (d > 0).mean() < 0.02


def test_matmul_golden(oracle_lib, gold):
    c = oracle_lib.matmul(gold["mm_a"].view(np.uint16), gold["mm_b"].view(np.uint16), oracle_lib.F16, 32, 32, 16, 8)
    got = c.view(np.float16).astype(np.float32)
    ref = gold["mm_c"].astype(np.float32)
    np.testing.assert_allclose(got, ref, rtol=2e-3, atol=2e-3)


def test_reduce_rows_and_total(oracle_lib):
    """Configured workload 5, CPU-check size: 512 x 768 viewed with strides [1, 512], ragged to 740 columns."""
    rng = np.random.default_rng(4)
    flat = rng.standard_normal(512 * 768).astype(np.float32)
    rows = oracle_lib.reduce_rows(flat, 512, 740, 1, 512, 64, 64)
    ref = flat.reshape(768, 512)[:740].astype(np.float64).sum(axis=0)
    scale = np.abs(flat.reshape(768, 512)[:740]).sum(axis=0)
    assert np.all(np.abs(rows - ref) <= 1e-5 * scale)
    tot = oracle_lib.reduce_all(rows, 1024)
    assert abs(tot - ref.sum()) <= 1e-5 * np.abs(ref).sum()
    # block shape does not change which elements are summed
    rows2 = oracle_lib.reduce_rows(flat, 512, 740, 1, 512, 32, 128)
    assert np.all(np.abs(rows - rows2) <= 1e-5 * scale)
