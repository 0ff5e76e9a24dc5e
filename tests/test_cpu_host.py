"""CPU tests of the host side: TTIR -> launch plan, descriptor evaluation at launch, the
driver plugin surface and program-range partitioning.  Launches run through the real
Triton JIT and the real driver plugin; only the ctypes library object is replaced by a
host-memory stand-in (tests/fake_tsb.py), so no GPU is needed."""
import json
import os
import re

import numpy as np
import pytest
import torch
import triton
from triton.backends.compiler import GPUTarget
from triton.compiler import ASTSource

import kernels as K
import triton_shared_b200 as tsb
from fake_tsb import fake_device

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TARGET = GPUTarget(tsb.BACKEND_NAME, 100, 32)


@pytest.fixture(scope="module", autouse=True)
def _driver():
    tsb.activate()
    yield


def _family(fn, sig, ce):
    k = triton.compile(ASTSource(fn, sig, ce), target=TARGET)
    return json.loads(k.asm["plan"])["family"], k


PTR3 = {"a_ptr": "*bf16", "b_ptr": "*bf16", "c_ptr": "*bf16"}
MM_SIG = dict(PTR3, **{k: "i32" for k in ["M", "N", "K", "stride_am", "stride_bk", "stride_cm"]},
              **{k: "constexpr" for k in ["stride_ak", "stride_bn", "stride_cn", "BLOCK_M", "BLOCK_N", "BLOCK_K", "GROUP_M"]})
MM_CE = {"stride_ak": 1, "stride_bn": 1, "stride_cn": 1, "BLOCK_M": 128, "BLOCK_N": 256, "BLOCK_K": 64, "GROUP_M": 8}


@pytest.mark.parametrize("fn,sig,ce,family", [
    (K.add_kernel, {"x_ptr": "*fp32", "y_ptr": "*fp32", "out_ptr": "*fp32", "n_elements": "i32", "BLOCK_SIZE": "constexpr"},
     {"BLOCK_SIZE": 1024}, "elementwise"),
    (K.softmax_kernel, {"out_ptr": "*fp32", "in_ptr": "*fp32", "in_row_stride": "i32", "out_row_stride": "i32",
                        "n_cols": "i32", "BLOCK_SIZE": "constexpr"}, {"BLOCK_SIZE": 1024}, "softmax"),
    (K.layernorm_fwd_kernel, {"X": "*fp16", "Y": "*fp16", "W": "*fp16", "B": "*fp16", "Mean": "*fp32", "Rstd": "*fp32",
                              "stride": "i32", "N": "i32", "eps": "fp32", "BLOCK_SIZE": "constexpr"}, {"BLOCK_SIZE": 1024},
     "layernorm"),
    (K.matmul_kernel, MM_SIG, MM_CE, "gemm"),
    (K.matmul_wrap_kernel, MM_SIG, MM_CE, "gemm"),
    (K.row_sum_kernel, {"x_ptr": "*fp32", "out_ptr": "*fp32", "M": "i32", "N": "i32", "stride_m": "constexpr",
                        "stride_n": "i32", "BLOCK_M": "constexpr", "BLOCK_N": "constexpr"},
     {"stride_m": 1, "BLOCK_M": 64, "BLOCK_N": 64}, "reduce_rows"),
    (K.total_kernel, {"x_ptr": "*fp32", "out_ptr": "*fp32", "n": "i32", "BLOCK": "constexpr"}, {"BLOCK": 1024}, "reduce_all"),
    (K.gelu_bias_kernel, {"x_ptr": "*fp16", "b_ptr": "*fp16", "out_ptr": "*fp16", "n_cols": "i32", "BLOCK": "constexpr"},
     {"BLOCK": 256}, "elementwise"),
])
def test_kernel_maps_to_family(fn, sig, ce, family):
    fam, k = _family(fn, sig, ce)
    assert fam == family
    assert k.metadata.name == fn.fn.__name__ if hasattr(fn, "fn") else True


def test_vec_add_descriptor_matches_reference_lowering():
    """offsets [pid*1024], sizes [1024], strides [1], mask dim from n: the tts.make_tptr / tts.load of
    test/Conversion/StructuredToMemref/kernel-01-vector-add.mlir:29-52."""
    _, k = _family(K.add_kernel, {"x_ptr": "*fp32", "y_ptr": "*fp32", "out_ptr": "*fp32", "n_elements": "i32",
                                  "BLOCK_SIZE": "constexpr"}, {"BLOCK_SIZE": 1024})
    params = json.loads(k.asm["plan"])["params"]
    assert params["tree"] == [["seg", 0]] and len(params["segments"]) == 1
    p = params["segments"][0]
    assert p["space"] == [1024] and len(p["accs"]) == 3
    for acc, arg in zip(p["accs"], (0, 1, 2)):
        assert acc["arg"] == arg
        assert acc["offset"]["$poly"] == [[[["pid", 0]], 1024]]
        assert acc["strides"][0]["$poly"] == [[[], 1]]
        start, bound = acc["mask"][0]
        assert start["$poly"] == [[[["pid", 0]], 1024]] and bound["$poly"] == [[[["arg", 3]], 1]]
        assert acc["other"] is None
    assert [o[0] for o in p["ops"]] == ["load", "load", "addf", "store"]


def test_unsupported_kernel_is_rejected_at_compile_time():
    @triton.jit
    def gather_kernel(x_ptr, idx_ptr, out_ptr, BLOCK: tl_constexpr):
        # atomics have no counterpart in the reference's lowering either
        offs = tl.arange(0, BLOCK)
        idx = tl.load(idx_ptr + offs)
        tl.atomic_add(out_ptr + idx, tl.load(x_ptr + offs))

    with pytest.raises(Exception) as e:
        triton.compile(ASTSource(gather_kernel, {"x_ptr": "*fp32", "idx_ptr": "*i32", "out_ptr": "*fp32", "BLOCK": "constexpr"},
                                 {"BLOCK": 64}), target=TARGET)
    assert "structured" in str(e.value) or "fits no" in str(e.value)


import triton.language as tl  # noqa: E402  (used by the jit kernel above at compile time)
tl_constexpr = tl.constexpr


# ------------------------------------------------------------------ launches on the host stand-in
def test_vec_add_end_to_end(oracle_lib):
    n = 98_432
    torch.manual_seed(0)
    x, y = torch.rand(n), torch.rand(n)
    out = torch.full((n + 32,), -7.0)
    with fake_device() as lib:
        K.add_kernel[(97,)](x, y, out, n, BLOCK_SIZE=1024)
    ref = oracle_lib.vec_add(x.numpy(), y.numpy(), n, 1024)
    assert np.array_equal(out.numpy()[:n].view(np.uint32), ref.view(np.uint32))
    assert torch.all(out[n:] == -7.0)
    assert lib.calls == [("tsb_elementwise", 0, 97)]


def test_partitioned_ranges_cover_grid_exactly(oracle_lib):
    n = 20_000
    torch.manual_seed(0)
    x, y = torch.rand(n), torch.rand(n)
    full = torch.zeros(n)
    parts = torch.zeros(n)
    drv = tsb.B200Driver.current
    with fake_device() as lib:
        K.add_kernel[(20,)](x, y, full, n, BLOCK_SIZE=1024)
        for r in range(3):
            with drv.partition(r, 3):
                K.add_kernel[(20,)](x, y, parts, n, BLOCK_SIZE=1024)
    assert torch.equal(full, parts)
    ranges = [(lo, hi) for name, lo, hi in lib.calls[1:]]
    assert ranges == [(0, 7), (7, 14), (14, 20)]


@pytest.mark.parametrize("total,world", [(97, 2), (97, 8), (5, 8), (2048, 8), (0, 4), (1 << 20, 8)])
def test_partition_range_properties(total, world):
    spans = [tsb.partition_range(total, r, world) for r in range(world)]
    assert spans[0][0] == 0 and spans[-1][1] == total
    for (a, b), (c, d) in zip(spans, spans[1:]):
        assert b == c and a <= b
    sizes = [b - a for a, b in spans]
    assert max(sizes) - min(sizes) <= 1


def test_known_answers_through_the_plugin():
    """Exact vectors of python/examples/test_mask.py:39,58,64 and the 2x+1 answer of
    test_load_2d_tensor_block.py:76-78, produced by plan + descriptors (host stand-in)."""
    inp = torch.arange(0, 8, dtype=torch.int32)
    with fake_device():
        out = torch.full((8,), -2, dtype=torch.int32)
        K.masked_other_kernel[(1,)](inp, out)
        assert out.tolist() == [-1, -1, -1, -1, -2, -2, -2, -2]
        out = torch.full((8,), -2, dtype=torch.int32)
        K.scalar_conj_mask_kernel[(1,)](inp, out, 4, 3)
        assert out.tolist() == [0, 1, 2, 3, -1, -1, -1, -1]
        out = torch.full((8,), -2, dtype=torch.int32)
        K.scalar_conj_mask_kernel[(1,)](inp, out, 4, 8)
        assert out.tolist() == [-1] * 8
        M, N = 13, 21
        x = torch.arange(M * N, dtype=torch.int32).reshape(M, N)
        o2 = torch.full((M, N), -3, dtype=torch.int32)
        K.affine_2d_kernel[(4, 3)](x, o2, N, 1, M, N, BLOCK_M=4, BLOCK_N=8)
        assert torch.equal(o2, 2 * x + 1)
        a = torch.arange(0, 256, dtype=torch.float32)
        b = torch.arange(1000, 1256, dtype=torch.float32)
        ae, be = b.clone(), a.clone()
        K.swap_kernel[(2,)](a, b, BLOCK=128)
        assert torch.equal(a, ae) and torch.equal(b, be)
        s = torch.zeros(1000)
        K.splat_kernel[(4,)](s, 2.5, 1000, BLOCK=256)
        assert torch.all(s == 2.5)


def test_gelu_chain_register_allocation():
    torch.manual_seed(5)
    x = torch.randn(5, 300).half()
    b = torch.randn(300).half()
    out = torch.zeros_like(x)
    with fake_device():
        K.gelu_bias_kernel[(5, 2)](x, b, out, 300, BLOCK=256)
    ref = torch.nn.functional.gelu(x.float() + b.float(), approximate="tanh")
    assert torch.allclose(out.float(), ref, rtol=2e-3, atol=2e-3)


def test_family_parameters_reach_the_c_abi(oracle_lib):
    """softmax / layernorm / reductions / matmul: the arguments the plans compute at launch are the
    ones the oracle needs to reproduce the kernels' results."""
    with fake_device() as lib:
        torch.manual_seed(1)
        base = torch.randn(40, 800)
        out = torch.full((40, 800), 5.0)
        K.softmax_kernel[(40,)](out, base, 800, 800, 781, BLOCK_SIZE=1024)
        np.testing.assert_allclose(out.numpy()[:, :781], oracle_lib.softmax(base.numpy()[:, :781], 1024), rtol=1e-6)
        assert torch.all(out[:, 781:] == 5.0)

        torch.manual_seed(2)
        x = torch.randn(6, 2500).half()
        w = (torch.rand(2500) + 0.5).half()
        b = (0.1 * torch.randn(2500)).half()
        y = torch.zeros_like(x)
        mean, rstd = torch.zeros(6), torch.zeros(6)
        K.layernorm_fwd_kernel[(6,)](x, y, w, b, mean, rstd, 2500, 2500, 1e-5, BLOCK_SIZE=1024)
        yr, mr, rr = oracle_lib.layernorm_fwd(x.numpy(), w.numpy(), b.numpy(), 1e-5, 1024)
        assert np.array_equal(y.numpy(), yr) and np.array_equal(mean.numpy(), mr) and np.array_equal(rstd.numpy(), rr)

        torch.manual_seed(4)
        flat = torch.randn(512 * 768)
        rs = torch.zeros(512)
        K.row_sum_kernel[(8,)](flat, rs, 512, 740, 1, 512, BLOCK_M=64, BLOCK_N=64)
        tot = torch.zeros(1)
        K.total_kernel[(1,)](rs, tot, 512, BLOCK=1024)
        ref = flat.numpy().reshape(768, 512)[:740].astype(np.float64).sum(axis=0)
        np.testing.assert_allclose(rs.numpy(), ref, rtol=1e-4, atol=1e-4)
        assert abs(tot.item() - ref.sum()) < 1e-2

        torch.manual_seed(3)
        a = (2 * torch.rand(200, 128) - 1).half()
        bm = (2 * torch.rand(128, 264) - 1).half()
        for kern in (K.matmul_kernel, K.matmul_wrap_kernel):
            c = torch.zeros(200, 264, dtype=torch.float16)
            kern[(2 * 2,)](a, bm, c, 200, 264, 128, 128, 1, 264, 1, 264, 1, BLOCK_M=128, BLOCK_N=256, BLOCK_K=64, GROUP_M=8)
            ref = a.float() @ bm.float()
            assert torch.allclose(c.float(), ref, rtol=1e-2, atol=1e-2)
    names = [c[0] for c in lib.calls]
    # 200 x 264 with 128 x 256 blocks: two vertically adjacent pairs of tiles, no single tile left over
    assert names == ["tsb_softmax_rows", "tsb_layernorm_fwd", "tsb_reduce_rows", "tsb_reduce_all",
                     "tsb_gemm_paired", "tsb_gemm_paired"]


# ------------------------------------------------------------------ plugin surface
def test_tile_pairing_for_the_two_cta_matmul():
    """Pairs are (even tile_m, tile_n) with (tile_m + 1, tile_n) present; every tile lands in exactly one place."""
    from triton_shared_b200.backend.plan import GemmPlan
    tiles = np.asarray(oracle_tiles(5 * 128, 3 * 256), dtype=np.int32)  # 5 x 3 tiles: the last tile row has no partner
    pairs, singles = GemmPlan.pair_tiles(tiles)
    assert len(pairs) == 2 * 3 and len(singles) == 3 and set(singles[:, 0]) == {4}
    covered = {(tm, tn) for tm, tn in pairs} | {(tm + 1, tn) for tm, tn in pairs} | {tuple(t) for t in singles}
    assert covered == {tuple(t) for t in tiles}
    # a partial range (what one of several GPUs gets) may cut a pair: the orphan becomes a single
    pairs, singles = GemmPlan.pair_tiles(tiles[1:8])
    covered = [(tm, tn) for tm, tn in pairs] + [(tm + 1, tn) for tm, tn in pairs] + [tuple(t) for t in singles]
    assert sorted(covered) == sorted(tuple(t) for t in tiles[1:8])


def oracle_tiles(M, N):
    import oracle
    return oracle.grouped_tiles(M, N, 128, 256, 8)


def test_driver_surface_matches_reference():
    """Method set of CPUDriver (backend/driver.py:420-464 in the reference) and launcher call shape."""
    d = tsb.B200Driver()
    for name in ["get_benchmarker", "get_device_capability", "get_current_stream", "get_current_device",
                 "set_current_device", "get_current_target", "get_active_torch_device", "assemble_tensormap_to_arg",
                 "map_python_to_cpp_type", "is_active"]:
        assert callable(getattr(d, name))
    assert d.is_active() is False
    assert d.binary_ext == "plan" and d.launcher_cls is tsb.B200Launcher
    assert d.map_python_to_cpp_type("*fp32") == "void*" and d.map_python_to_cpp_type("i32") == "int32_t"
    t = d.get_current_target()
    assert tsb.B200Backend.supports_target(t)
    from triton.backends import backends
    assert not backends["nvidia"].compiler.supports_target(t)
    props = d.utils.get_device_properties(0)
    assert "max_shared_mem" in props
    with pytest.raises(TypeError):
        from triton_shared_b200.backend.driver import LaunchArgs
        LaunchArgs(None, [("*fp32", object())]).pointer(0)


def test_c_abi_library_exports_every_declared_symbol():
    """The shared object loads without a GPU and exports exactly what include/tsb200.h declares."""
    hdr = open(os.path.join(ROOT, "include", "tsb200.h")).read()
    declared = set(re.findall(r"\b(tsb_[a-z_0-9]+)\s*\(", hdr))
    from triton_shared_b200.backend import runtime as rt
    import ctypes
    L = ctypes.CDLL(rt.LIB_PATH)
    for sym in declared:
        assert hasattr(L, sym), f"{sym} declared in tsb200.h but not exported"
    assert declared == set(rt.SYMBOLS)
    assert L.tsb_version() == 1000


def test_missing_library_fails_loudly(monkeypatch):
    from triton_shared_b200.backend import runtime as rt
    monkeypatch.setattr(rt, "_lib", None)
    monkeypatch.setattr(rt, "LIB_PATH", "/nonexistent/libtsb200.so")
    with pytest.raises(rt.TsbError, match="no fallback"):
        rt.lib()


# ------------------------------------------------------------------ loops and wrap-around
def _loop_and_wrap_cases(dev):
    """Shared by the CPU (host stand-in) and GPU variants: returns a list of (name, got, expected)."""
    out = []
    # grid-stride copy with a loop-carried index/mask
    x = torch.arange(0, 100, dtype=torch.float32, device=dev)
    y = torch.full((104,), -1.0, device=dev)
    K.grid_stride_copy_kernel[(3,)](y, x, 100, 5, BLOCK_SIZE=8)
    exp = torch.full((104,), -1.0)
    exp[:100] = 2.0 * torch.arange(0, 100, dtype=torch.float32)
    out.append(("grid_stride_copy", y.cpu(), exp))
    # nested tile walk
    a = torch.arange(0, 12 * 20, dtype=torch.float32, device=dev).reshape(12, 20)
    c = torch.zeros_like(a)
    K.tile_walk_kernel[(1,)](a, c, 20, 1, TM=4, TN=4, NI=3, NJ=5)
    out.append(("tile_walk", c.cpu(), a.cpu() + 1.0))
    # stacked wrap-around: the exact expected matrix of python/examples/test_modulo.py:45-50
    A = torch.arange(0, 32, dtype=torch.float32, device=dev).reshape(4, 8)
    C = torch.full((4, 8), 88888.0, device=dev)
    K.wrap_rows_kernel[(1,)](A, C, 4, 8, 1, 8, 1, START=2, BM=4, BN=4, STEPS=2)
    exp = torch.tensor([[16, 17, 18, 19, 20, 21, 22, 23], [24, 25, 26, 27, 28, 29, 30, 31],
                        [0, 1, 2, 3, 4, 5, 6, 7], [8, 9, 10, 11, 12, 13, 14, 15]], dtype=torch.float32)
    out.append(("wrap_rows", C.cpu(), exp))
    # side-by-side wrap-around: first row of the expected matrix of test_modulo.py:88-97
    A = torch.arange(0, 64, dtype=torch.float32, device=dev).reshape(8, 8)
    C = torch.full((8, 8), 88888.0, device=dev)
    K.wrap_cols_kernel[(1,)](A, C, 8, 7, 8, 1, 1, START=6, BN=4)
    exp = torch.full((8, 8), 88888.0)
    exp[0, :4] = torch.tensor([62.0, 63.0, 56.0, 57.0])
    out.append(("wrap_cols", C.cpu(), exp))
    return out


def test_loops_and_wraparound_on_host_stand_in():
    with fake_device() as lib:
        cases = _loop_and_wrap_cases("cpu")
    for name, got, exp in cases:
        assert torch.equal(got, exp), name
    # every loop nest here is perfect, so each kernel is one launch with the loops run on the device
    assert len(lib.calls) == 4


# ------------------------------------------------------------------ block programs (reductions in the body)
def _block_program_cases(dev):
    out = []
    torch.manual_seed(7)
    x = torch.randn(9, 300, device=dev)
    s = torch.zeros(9, device=dev)
    K.block_sum_kernel[(9,)](x, s, 300, 290, BLOCK_SIZE=512)
    import oracle as O
    npf = lambda t: t.detach().cpu().numpy()
    # left-to-right folds of the oracle; the GPU folds in a tree, so float sums agree within rounding
    out.append(("block_sum", s.cpu(), torch.from_numpy(O.fold(npf(x[:, :290]), 1, "addf")), 1e-4))
    # the reference's own block-pointer test: 32 programs of 16 elements (test_reduce.py:33-43, rtol 1e-3)
    xb = torch.rand(32, 16, device=dev)
    sb = torch.zeros(32, device=dev)
    K.block_ptr_sum_kernel[(32,)](xb, sb, 16, 16, BLOCK_SIZE=16)
    out.append(("block_ptr_sum", sb.cpu(), xb.sum(dim=1).cpu(), 1e-3))
    xh = torch.randn(5, 1000, device=dev).half()
    w = (torch.rand(1000, device=dev) + 0.5).half()
    y = torch.zeros_like(xh)
    K.rmsnorm_kernel[(5,)](xh, w, y, 1000, 1000, 1e-6, BLOCK=1024)
    xf = xh.float()
    ref = xf * torch.rsqrt((xf * xf).mean(dim=1, keepdim=True) + 1e-6) * w.float()
    out.append(("rmsnorm", y.float().cpu(), ref.cpu(), 2e-2))
    xi = torch.randint(-1000, 1000, (50, 24), dtype=torch.int32, device=dev)
    rmax = torch.full((50,), -7, dtype=torch.int32, device=dev)
    cmin = torch.full((4 * 32,), -7, dtype=torch.int32, device=dev)
    K.tile_max_kernel[(4,)](xi, rmax, cmin, 24, 50, 24, BM=16, BN=32)
    # masked lanes load other = 0 and take part in the fold (the reference reduces the whole filled block)
    blk_rows = np.zeros((50, 32), dtype=np.int32)
    blk_rows[:, :24] = npf(xi)
    out.append(("tile_rowmax", rmax.cpu(), torch.from_numpy(O.fold(blk_rows, 1, "maxsi")), 0))
    exp_cmin = torch.full((4, 32), -7, dtype=torch.int32)
    xc = xi.cpu()
    for pid in range(4):
        blk = torch.zeros(16, 32, dtype=torch.int32)
        rows = xc[pid * 16:(pid + 1) * 16]
        blk[:rows.shape[0], :24] = rows
        exp_cmin[pid, :24] = torch.from_numpy(O.fold(blk.numpy(), 0, "minsi"))[:24]
    out.append(("tile_colmin", cmin.cpu().reshape(4, 32), exp_cmin, 0))
    # argmax / argmin: ties go to the smaller index
    xa = torch.randint(0, 5, (6, 100), device=dev).float()  # many ties
    av = torch.zeros(6, device=dev)
    ai = torch.zeros(6, dtype=torch.int32, device=dev)
    K.row_argmax_kernel[(6,)](xa, av, ai, 100, 90, BLOCK=128)
    xa[1, 3] = float("nan")      # a NaN never wins the reference's fold
    xa[2, :] = float("-inf")     # a line without any winner keeps index -1
    K.row_argmax_kernel[(6,)](xa, av, ai, 100, 90, BLOCK=128)
    padded = np.full((6, 128), -np.inf, dtype=np.float32)  # the kernel loads other = -inf beyond n
    padded[:, :90] = npf(xa[:, :90])
    ov, oi = O.argfold(padded, 1, True)
    out.append(("argmax_val", av.cpu(), torch.from_numpy(ov), 0))
    out.append(("argmax_idx", ai.cpu(), torch.from_numpy(oi), 0))
    xt = torch.randn(32, 16, device=dev)
    ti = torch.zeros(32, dtype=torch.int32, device=dev)
    K.tile_argmin_kernel[(4,)](xt, ti, 16, BM=8, BN=16)
    out.append(("argmin_axis1", ti.cpu(), torch.from_numpy(O.argfold(npf(xt), 1, False)[1]), 0))
    # loops that carry block values (device-side loops of the block-program kernel)
    xr = torch.randn(7, 1000, device=dev)
    rs = torch.zeros(7, device=dev)
    rm = torch.zeros(7, device=dev)
    K.row_stats_kernel[(7,)](xr, rs, rm, 1000, 900, BLOCK=256)
    out.append(("row_stats_sum", rs.cpu(), torch.from_numpy(O.fold(npf(xr[:, :900]), 1, "addf")), 1e-4))
    out.append(("row_stats_max", rm.cpu(), torch.from_numpy(O.fold(npf(xr[:, :900]), 1, "maxnumf")), 0))
    xs = torch.randn(6, 2500, device=dev)
    os_ = torch.full((6, 2500), -1.0, device=dev)
    K.wide_softmax_kernel[(6,)](os_, xs, 2500, 2400, BLOCK=512)
    exp = torch.full((6, 2500), -1.0)
    exp[:, :2400] = torch.softmax(xs[:, :2400].cpu(), dim=1)
    out.append(("wide_softmax", os_.cpu(), exp, 1e-5))
    # running sums (tl.cumsum): float rows with a ragged tail, and an int32 tile along axis 1 (exact)
    xc_ = torch.randn(5, 300, device=dev)
    yc = torch.full((5, 300), -3.0, device=dev)
    K.row_cumsum_kernel[(5,)](xc_, yc, 300, 260, BLOCK=512)
    expc = torch.full((5, 300), -3.0)
    expc[:, :260] = torch.from_numpy(O.cumsum(npf(xc_[:, :260]), 1))
    out.append(("row_cumsum", yc.cpu(), expc, 1e-4))
    ti_ = torch.randint(-50, 50, (16, 32), dtype=torch.int32, device=dev)
    to = torch.zeros_like(ti_)
    K.tile_cumsum_kernel[(2,)](ti_, to, 32, BM=8, BN=32)
    out.append(("tile_cumsum_int", to.cpu(), torch.from_numpy(O.cumsum(npf(ti_), 1)), 0))
    # LayerNorm backward: input gradient per row, and the column sums of the partial dw / db
    Mb, Nb = 6, 200
    xb_ = torch.randn(Mb, Nb, device=dev)
    dyb = torch.randn(Mb, Nb, device=dev)
    wb = torch.rand(Nb, device=dev) + 0.5
    mean = xb_.mean(dim=1)
    rstd = 1.0 / torch.sqrt(xb_.var(dim=1, unbiased=False) + 1e-5)
    dxb = torch.zeros_like(xb_)
    K.layernorm_bwd_dx_kernel[(Mb,)](dxb, dyb, xb_, wb, mean, rstd, Nb, Nb, BLOCK_N=256)
    out.append(("ln_bwd_dx", dxb.cpu(), torch.from_numpy(O.layernorm_bwd_dx(npf(xb_), npf(dyb), npf(wb), npf(mean), npf(rstd))), 1e-4))
    dwp, dbp = torch.randn(70, 300, device=dev), torch.randn(70, 300, device=dev)
    fdw, fdb = torch.zeros(300, device=dev), torch.zeros(300, device=dev)
    K.layernorm_bwd_dwdb_kernel[(3,)](dwp, dbp, fdw, fdb, 70, 300, BLOCK_SIZE_M=32, BLOCK_SIZE_N=128)
    edw, edb = O.layernorm_bwd_dwdb(npf(dwp), npf(dbp), 32)
    out.append(("ln_bwd_dw", fdw.cpu(), torch.from_numpy(edw), 1e-4))
    out.append(("ln_bwd_db", fdb.cpu(), torch.from_numpy(edb), 1e-4))
    return out


def test_block_programs_on_host_stand_in():
    with fake_device() as lib:
        cases = _block_program_cases("cpu")
    for name, got, exp, tol in cases:
        if tol == 0:
            assert torch.equal(got, exp), name
        else:
            assert torch.allclose(got, exp, rtol=tol, atol=tol), name
    # argmax runs twice (before and after the NaN / -inf rows); the RMS norm and the LayerNorm input
    # gradient (full folds of the one block they store) run on the elementwise engine
    names = [c[0] for c in lib.calls]
    assert names.count("tsb_block_program") == 11 and names.count("tsb_elementwise") == 2 and len(names) == 13


# ------------------------------------------------------------------ a spread of elementwise ops
def _mixed_op_cases(dev):
    out = []
    torch.manual_seed(11)
    n = 3000
    x = torch.randn(n, device=dev)
    y = torch.randn(n, device=dev)
    o1, o2, o3 = (torch.zeros(n, device=dev) for _ in range(3))
    K.mixed_float_kernel[(3,)](x, y, o1, o2, o3, n, 0.1, BLOCK=1024)
    out.append(("leaky", o1.cpu(), torch.where(x > 0, x, 0.1 * x).cpu(), 1e-6))
    sig = 1.0 / (1.0 + torch.exp(-x))
    ref2 = torch.maximum(sig, torch.minimum(y.abs(), torch.tensor(0.75, device=dev))) + x.abs().sqrt() * torch.log(y.abs() + 1.0)
    out.append(("sigmoid_mix", o2.cpu(), ref2.cpu(), 1e-5))
    out.append(("floor_trig", o3.cpu(), (torch.floor(x * 4.0) + torch.cos(y) * torch.sin(x)).cpu(), 1e-5))
    a = torch.randint(0, 1000, (n,), dtype=torch.int32, device=dev)
    b = torch.randint(1, 1000, (n,), dtype=torch.int32, device=dev)
    i1, i2, i3 = (torch.zeros(n, dtype=torch.int32, device=dev) for _ in range(3))
    K.mixed_int_kernel[(3,)](a, b, i1, i2, i3, n, BLOCK=1024)
    out.append(("int_arith", i1.cpu(), ((a * 3 + b) // 7 + (a % 5) - torch.minimum(a, b)).cpu(), 0))
    out.append(("int_bits", i2.cpu(), (((a & b) | (a ^ 21)) + (b << 2) + (a >> 1)).cpu(), 0))
    offs = torch.arange(n, device=dev)
    out.append(("int_float_int", i3.cpu(), (a.float() * 0.5 + offs.float()).to(torch.int32).cpu(), 0))
    u = torch.randint(0, 256, (n,), dtype=torch.uint8, device=dev)
    uo = torch.zeros(n, dtype=torch.uint8, device=dev)
    K.bytes_kernel[(3,)](u, uo, n, BLOCK=1024)
    out.append(("bytes", uo.cpu(), torch.clamp(u.int() * 2 + 10, max=255).to(torch.uint8).cpu(), 0))
    return out


def test_mixed_ops_on_host_stand_in():
    with fake_device():
        cases = _mixed_op_cases("cpu")
    for name, got, exp, tol in cases:
        if tol == 0:
            assert torch.equal(got, exp), name
        else:
            assert torch.allclose(got, exp, rtol=tol, atol=tol), name


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.int16, torch.uint8], ids=lambda d: str(d)[6:])
@pytest.mark.parametrize("n_cols", [1000, 1001, 3])
def test_padded_scale_2d_on_host_stand_in(dtype, n_cols):
    """The plan of the padded scale kernel (masked loads with a fill, unmasked store) on the host
    stand-in: the same cases the GPU suite runs through the lean and general accessors."""
    BLOCK, rows = 256, 5
    nb = (n_cols + BLOCK - 1) // BLOCK
    g = torch.Generator().manual_seed(n_cols)
    x = torch.randint(0, 20, (rows, n_cols), generator=g).to(dtype)
    b = torch.randint(0, 20, (n_cols,), generator=g).to(dtype)
    out = torch.full((rows + 1, nb * BLOCK), 99, dtype=dtype)
    with fake_device():
        K.pad_scale_kernel[(rows, nb)](x, b, out, n_cols, nb * BLOCK, BLOCK=BLOCK)
    exp = torch.full((rows, nb * BLOCK), 9, dtype=torch.int64)
    exp[:, :n_cols] = x.to(torch.int64) * 2 + b.to(torch.int64)
    assert torch.equal(out[:rows].to(torch.int64), exp)
    assert torch.all(out[rows] == 99)


@pytest.mark.parametrize("block", [16, 128])
def test_row_folds_on_host_stand_in(block):
    """Full folds of the stored block lower to the elementwise family (TSB_OP_REDUCE)."""
    rows, n_cols = 5, block - 3
    x = torch.randint(-50, 1000, (rows, block), generator=torch.Generator().manual_seed(block), dtype=torch.int32)
    y = torch.full_like(x, -7)
    with fake_device() as lib:
        K.row_center_kernel[(rows,)](x, y, block, n_cols, BLOCK=block)
    assert [c[0] for c in lib.calls] == ["tsb_elementwise"]
    xv = x[:, :n_cols].long()
    exp = xv - torch.clamp(xv.max(dim=1, keepdim=True).values, min=0) + xv.sum(dim=1, keepdim=True)
    assert torch.equal(y[:, :n_cols].long(), exp)
    assert torch.all(y[:, n_cols:] == -7)


def test_launch_hooks_are_called():
    """launch_enter_hook / launch_exit_hook around every launch, as the reference launcher does
    (backend/driver.py:197-218 there)."""
    from triton import knobs
    seen = []
    old_enter, old_exit = knobs.runtime.launch_enter_hook, knobs.runtime.launch_exit_hook
    knobs.runtime.launch_enter_hook = lambda md: seen.append(("enter", md.get()["name"] if hasattr(md, "get") else md))
    knobs.runtime.launch_exit_hook = lambda md: seen.append(("exit", md.get()["name"] if hasattr(md, "get") else md))
    try:
        x = torch.arange(0, 64, dtype=torch.float32)
        y = torch.ones(64)
        out = torch.zeros(64)
        with fake_device():
            K.add_kernel[(1,)](x, y, out, 64, BLOCK_SIZE=64)
    finally:
        knobs.runtime.launch_enter_hook, knobs.runtime.launch_exit_hook = old_enter, old_exit
    assert [s[0] for s in seen] == ["enter", "exit"] and seen[0][1] == "add_kernel"
    assert torch.equal(out, x + 1)


def test_tile_tables_are_keyed_by_content():
    """Two specialisations of one kernel (same name, scalars and grid, different GROUP_M) must not
    share an uploaded pid -> tile table, also under a partial program range."""
    import kernels as K
    M = N = 512
    Kd = 128
    torch.manual_seed(5)
    A = (2 * torch.rand(M, Kd) - 1).half()
    B = (2 * torch.rand(Kd, N) - 1).half()
    ref = (A.float() @ B.float())
    outs = []
    with fake_device():
        drv = tsb.activate()
        for gm in (8, 1):
            C = torch.zeros(M, N, dtype=torch.float16)
            with drv.program_range(0, 5):  # 5 of the 8 programs: which tiles those are depends on GROUP_M
                K.matmul_kernel[(8,)](A, B, C, M, N, Kd, Kd, 1, N, 1, N, 1, BLOCK_M=128, BLOCK_N=256, BLOCK_K=64, GROUP_M=gm)
            outs.append(C)
    tiles_of = {8: [(0, 0), (1, 0), (2, 0), (3, 0), (0, 1)], 1: [(0, 0), (0, 1), (1, 0), (1, 1), (2, 0)]}
    for gm, C in zip((8, 1), outs):
        for tm in range(4):
            for tn in range(2):
                blk = C[tm * 128:(tm + 1) * 128, tn * 256:(tn + 1) * 256].float()
                want = ref[tm * 128:(tm + 1) * 128, tn * 256:(tn + 1) * 256] if (tm, tn) in tiles_of[gm] else torch.zeros(128, 256)
                assert torch.allclose(blk, want, rtol=1e-2, atol=1e-2), (gm, tm, tn)


def test_driver_check_reports_a_device_side_timeout():
    """B200Driver.check() turns the status word a timed-out device wait leaves behind into an exception."""
    from triton_shared_b200.backend.driver import B200Launcher
    from triton_shared_b200.backend.runtime import TsbError
    with fake_device():
        drv = tsb.activate()
        drv.check()  # nothing recorded: passes
        B200Launcher.memory._status[:] = [-4, 1, 17, 3]
        with pytest.raises(TsbError, match="tile 17"):
            drv.check()
        drv.check()  # the word was cleared


def test_c_plan_evaluator_parses_every_family():
    """tsb_plan_create reads the plan text of each kernel family (no GPU needed: nothing is launched)."""
    import json
    import kernels as K
    from triton_shared_b200 import runtime as rt
    L = rt.lib()
    cases = [
        (K.add_kernel, {"x_ptr": "*fp32", "y_ptr": "*fp32", "out_ptr": "*fp32", "n_elements": "i32", "BLOCK_SIZE": "constexpr"},
         {"BLOCK_SIZE": 1024}),
        (K.softmax_kernel, {"out_ptr": "*fp32", "in_ptr": "*fp32", "in_row_stride": "i32", "out_row_stride": "i32",
                            "n_cols": "i32", "BLOCK_SIZE": "constexpr"}, {"BLOCK_SIZE": 1024}),
        (K.layernorm_fwd_kernel, {"X": "*fp16", "Y": "*fp16", "W": "*fp16", "B": "*fp16", "Mean": "*fp32", "Rstd": "*fp32",
                                  "stride": "i32", "N": "i32", "eps": "fp32", "BLOCK_SIZE": "constexpr"}, {"BLOCK_SIZE": 1024}),
        (K.row_sum_kernel, {"x_ptr": "*fp32", "out_ptr": "*fp32", "M": "i32", "N": "i32", "stride_m": "i32", "stride_n": "i32",
                            "BLOCK_M": "constexpr", "BLOCK_N": "constexpr"}, {"BLOCK_M": 64, "BLOCK_N": 64}),
        (K.total_kernel, {"x_ptr": "*fp32", "out_ptr": "*fp32", "n": "i32", "BLOCK": "constexpr"}, {"BLOCK": 1024}),
        (K.rmsnorm_kernel, {"x_ptr": "*fp16", "w_ptr": "*fp16", "y_ptr": "*fp16", "stride": "i32", "n_cols": "i32", "eps": "fp32",
                            "BLOCK": "constexpr"}, {"BLOCK": 1024}),
        (K.row_stats_kernel, {"x_ptr": "*fp32", "sum_ptr": "*fp32", "max_ptr": "*fp32", "stride": "i32", "N": "i32",
                              "BLOCK": "constexpr"}, {"BLOCK": 1024}),
    ]
    seen = set()
    for fn, sig, ce in cases:
        text = triton.compile(ASTSource(fn, sig, ce), target=TARGET).asm["plan"]
        h = L.tsb_plan_create(text, len(text))
        assert h, L.tsb_last_error()
        assert L.tsb_plan_family(h).decode() == json.loads(text)["family"]
        seen.add(L.tsb_plan_family(h).decode())
        L.tsb_plan_destroy(h)
    assert seen == {"elementwise", "softmax", "layernorm", "reduce_rows", "reduce_all", "block_program"}
    assert not L.tsb_plan_create(b"[1, 2", -1) and b"JSON" in L.tsb_last_error()


# ------------------------------------------------------------------ the reference's own example tests
def _reference_cases():
    import reference_examples as R
    # the host stand-in executes lanes in numpy: keep to the cases it finishes in seconds
    return [c for c in R.cases() if "b=2048" not in c[0] and "b=4096" not in c[0] and "h=5120" not in c[0]
            and "h=7680" not in c[0] and "h=8192" not in c[0] and "(128, 2, 4)" not in c[0] and "(64, 2, 4)" not in c[0]]


_REF = _reference_cases()


@pytest.mark.skipif(not _REF, reason="TSB_REFERENCE_EXAMPLES does not name a directory of reference examples")
@pytest.mark.parametrize("case", _REF or [None], ids=[c[0] for c in _REF] or ["none"])
def test_reference_example_on_host_stand_in(case):
    """python/examples of the reference, unmodified, with B200Driver for CPUDriver and the C library
    replaced by its host stand-in (plan compilation and descriptor evaluation are the real ones)."""
    import reference_examples as R
    import triton_shared_b200
    triton_shared_b200.activate()
    _, path, name, kw = case
    with fake_device():
        R.run_case(path, name, kw, "cpu")
