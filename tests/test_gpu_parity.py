"""GPU parity tests: the CUDA path (through the Triton driver plugin and through
the C ABI directly) against the CPU oracle on the same seeded inputs.

Tolerances are the ones stated for each workload: bit-exact for fp32 add and all
masking/indexing; rel 1e-5 for fp32 reductions and softmax; 1e-2 on fp16/bf16
outputs with fp32 accumulation; 1e-5 on LayerNorm mean/rstd.
"""
import ctypes

import numpy as np
import pytest
import torch

import kernels as K

pytestmark = pytest.mark.gpu


def _cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")


@pytest.fixture(scope="module")
def drv(tsb_driver):
    _cuda()
    return tsb_driver


def _loaded_native():
    """The product library must be the thing that ran."""
    with open("/proc/self/maps") as f:
        return "libtsb200.so" in f.read()


# ---------------------------------------------------------------- config 1: vec add
@pytest.mark.parametrize("n", [98_432, 1, 1023, 1024, 1025, 4096, 1_000_003])
def test_vec_add_bit_exact(drv, oracle_lib, n):
    torch.manual_seed(0)
    x = torch.rand(n, dtype=torch.float32)
    y = torch.rand(n, dtype=torch.float32)
    ref = oracle_lib.vec_add(x.numpy(), y.numpy(), n, 1024)
    xd, yd = x.cuda(), y.cuda()
    out = torch.full((n + 64,), -7.0, device="cuda")  # guard band behind the masked tail
    grid = (triton_cdiv(n, 1024),)
    K.add_kernel[grid](xd, yd, out, n, BLOCK_SIZE=1024)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    assert np.array_equal(got[:n].view(np.uint32), ref.view(np.uint32))
    assert np.all(got[n:] == -7.0), "stored beyond the mask"
    assert _loaded_native()


def triton_cdiv(a, b):
    return (a + b - 1) // b


def test_vec_add_unaligned_views(drv, oracle_lib):
    """Base pointers that are not 16-byte aligned take the scalar path; results stay bit-exact."""
    n = 5000
    torch.manual_seed(0)
    xb = torch.rand(n + 3, dtype=torch.float32)
    yb = torch.rand(n + 1, dtype=torch.float32)
    x, y = xb[3:], yb[1:]
    ref = oracle_lib.vec_add(np.ascontiguousarray(x.numpy()), np.ascontiguousarray(y.numpy()), n, 1024)
    xd, yd = xb.cuda()[3:], yb.cuda()[1:]
    out = torch.zeros(n + 2, device="cuda")[2:]
    K.add_kernel[(triton_cdiv(n, 1024),)](xd, yd, out, n, BLOCK_SIZE=1024)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), ref.view(np.uint32))


def test_vec_add_large_property(drv):
    """Full-size property check (n = 2^30, 16 GB on the device): equals torch's x+y exactly."""
    n = 1 << 30
    torch.manual_seed(0)
    x = torch.rand(n, device="cuda")
    y = torch.rand(n, device="cuda")
    out = torch.empty_like(x)
    K.add_kernel[(triton_cdiv(n, 1024),)](x, y, out, n, BLOCK_SIZE=1024)
    assert torch.equal(out, x + y)


# ---------------------------------------------------------------- config 2: softmax
@pytest.mark.parametrize("rows,cols,block", [(1823, 781, 1024), (7, 1, 16), (64, 1024, 1024), (33, 4096, 4096),
                                             (5, 3000, 4096), (3, 9000, 16384)])
def test_softmax_vs_oracle(drv, oracle_lib, rows, cols, block):
    torch.manual_seed(1)
    x = torch.randn(rows, cols, dtype=torch.float32)
    ref = oracle_lib.softmax(x.numpy(), block)
    xd = x.cuda()
    out = torch.empty_like(xd)
    K.softmax_kernel[(rows,)](out, xd, xd.stride(0), out.stride(0), cols, BLOCK_SIZE=block)
    got = out.cpu().numpy()
    np.testing.assert_allclose(got, ref, rtol=1e-5, atol=1e-8)
    np.testing.assert_allclose(got.sum(axis=1), 1.0, rtol=1e-5)


def test_softmax_padded_rows(drv, oracle_lib):
    """Row stride larger than n_cols; the padding must stay untouched."""
    torch.manual_seed(1)
    base = torch.randn(100, 800, dtype=torch.float32)
    x = base[:, :781]
    ref = oracle_lib.softmax(base.numpy()[:, :781], 1024)
    xd = base.cuda()
    out = torch.full((100, 800), 5.0, device="cuda")
    K.softmax_kernel[(100,)](out, xd, xd.stride(0), out.stride(0), 781, BLOCK_SIZE=1024)
    got = out.cpu().numpy()
    np.testing.assert_allclose(got[:, :781], ref, rtol=1e-5, atol=1e-8)
    assert np.all(got[:, 781:] == 5.0)


def test_softmax_full_size_property(drv):
    rows, cols = 65_536, 4_096
    torch.manual_seed(1)
    x = torch.randn(rows, cols, device="cuda")
    out = torch.empty_like(x)
    K.softmax_kernel[(rows,)](out, x, x.stride(0), out.stride(0), cols, BLOCK_SIZE=4096)
    s = out.sum(dim=1)
    assert torch.allclose(s, torch.ones_like(s), rtol=1e-5)
    assert torch.allclose(out, torch.softmax(x, dim=1), rtol=1e-5, atol=1e-8)


# ---------------------------------------------------------------- config 3: layernorm
@pytest.mark.parametrize("M,N,dtype", [(256, 1024, torch.float16), (17, 8192, torch.float16), (5, 1000, torch.float16),
                                       (9, 77, torch.float16), (12, 2048, torch.float32), (6, 3000, torch.bfloat16)])
def test_layernorm_vs_oracle(drv, oracle_lib, M, N, dtype):
    torch.manual_seed(2)
    x = torch.randn(M, N).to(dtype)
    w = (torch.rand(N) + 0.5).to(dtype)
    b = (0.1 * torch.randn(N)).to(dtype)
    eps = 1e-5
    if dtype == torch.bfloat16:
        as_np = lambda t: t.view(torch.uint16).numpy()
        yr, mr, rr = oracle_lib.layernorm_fwd(as_np(x), as_np(w), as_np(b), eps, 1024, dtype=oracle_lib.BF16)
        yr = torch.from_numpy(yr.view(np.int16)).view(torch.bfloat16).float().numpy()
    else:
        yr, mr, rr = oracle_lib.layernorm_fwd(x.numpy(), w.numpy(), b.numpy(), eps, 1024)
        yr = yr.astype(np.float32)
    xd, wd, bd = x.cuda(), w.cuda(), b.cuda()
    y = torch.empty_like(xd)
    mean = torch.empty(M, dtype=torch.float32, device="cuda")
    rstd = torch.empty(M, dtype=torch.float32, device="cuda")
    K.layernorm_fwd_kernel[(M,)](xd, y, wd, bd, mean, rstd, xd.stride(0), N, eps, BLOCK_SIZE=1024)
    np.testing.assert_allclose(mean.cpu().numpy(), mr, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(rstd.cpu().numpy(), rr, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(y.float().cpu().numpy(), yr, rtol=1e-2, atol=1e-2)


def test_layernorm_full_size_property(drv):
    M, N = 4096, 8192
    torch.manual_seed(2)
    x = torch.randn(M, N, device="cuda").half()
    w = (torch.rand(N, device="cuda") + 0.5).half()
    b = (0.1 * torch.randn(N, device="cuda")).half()
    y = torch.empty_like(x)
    mean = torch.empty(M, dtype=torch.float32, device="cuda")
    rstd = torch.empty(M, dtype=torch.float32, device="cuda")
    K.layernorm_fwd_kernel[(M,)](x, y, w, b, mean, rstd, x.stride(0), N, 1e-5, BLOCK_SIZE=1024)
    ref = torch.nn.functional.layer_norm(x.float(), (N,), w.float(), b.float(), 1e-5)
    assert torch.allclose(y.float(), ref, rtol=1e-2, atol=1e-2)
    assert torch.allclose(mean, x.float().mean(dim=1), rtol=1e-5, atol=1e-6)


# ---------------------------------------------------------------- config 5: strided reduce
@pytest.mark.parametrize("M,N_total,N_valid,BM,BN", [(512, 768, 740, 64, 64), (100, 50, 37, 32, 16), (8192, 300, 300, 128, 64)])
def test_strided_reduce_vs_oracle(drv, oracle_lib, M, N_total, N_valid, BM, BN):
    torch.manual_seed(4)
    flat = torch.randn(M * N_total, dtype=torch.float32)
    ref = oracle_lib.reduce_rows(flat.numpy(), M, N_valid, 1, M, BM, BN)
    ref_total = oracle_lib.reduce_all(ref, 1024)
    xd = flat.cuda()
    out = torch.empty(M, dtype=torch.float32, device="cuda")
    K.row_sum_kernel[(triton_cdiv(M, BM),)](xd, out, M, N_valid, 1, M, BLOCK_M=BM, BLOCK_N=BN)
    tot = torch.zeros(1, dtype=torch.float32, device="cuda")
    K.total_kernel[(1,)](out, tot, M, BLOCK=1024)
    got = out.cpu().numpy()
    _assert_sum_close(got, ref, flat.numpy().reshape(N_total, M)[:N_valid].T)
    assert abs(tot.cpu().numpy()[0] - ref_total) <= 1e-5 * np.abs(ref).sum()


def _assert_sum_close(got, ref, terms, rel=1e-5):
    """Sums that cancel cannot be compared relative to their own value: both the oracle's
    left-to-right fold and the GPU's tree differ from the exact sum by O(eps * sum|x|).
    The stated tolerance (rel 1e-5) is therefore applied to the sum of magnitudes."""
    scale = np.abs(terms).sum(axis=1)
    bad = np.abs(got - ref) > rel * scale
    assert not bad.any(), f"{bad.sum()} row sums off by more than {rel} * sum|x|"


def test_row_major_reduce_vs_oracle(drv, oracle_lib):
    """Same kernel with the reduced dim contiguous (strides [N, 1])."""
    M, N = 300, 1000
    torch.manual_seed(4)
    x = torch.randn(M, N, dtype=torch.float32)
    ref = oracle_lib.reduce_rows(x.numpy().reshape(-1), M, N - 7, N, 1, 32, 128)
    out = torch.empty(M, dtype=torch.float32, device="cuda")
    K.row_sum_kernel[(triton_cdiv(M, 32),)](x.cuda(), out, M, N - 7, N, 1, BLOCK_M=32, BLOCK_N=128)
    _assert_sum_close(out.cpu().numpy(), ref, x.numpy()[:, :N - 7])


def test_strided_reduce_full_size_property(drv):
    M, N, NV = 8192, 12288, 12000
    torch.manual_seed(4)
    flat = torch.randn(M * N, device="cuda")
    out = torch.empty(M, device="cuda")
    K.row_sum_kernel[(M // 64,)](flat, out, M, NV, 1, M, BLOCK_M=64, BLOCK_N=64)
    ref = flat.view(N, M)[:NV].double().sum(dim=0)
    scale = flat.view(N, M)[:NV].abs().double().sum(dim=0)
    assert torch.all((out.double() - ref).abs() <= 1e-5 * scale)
    tot = torch.zeros(1, device="cuda")
    K.total_kernel[(1,)](out, tot, M, BLOCK=1024)
    assert abs(tot.item() - ref.sum().item()) <= 1e-5 * ref.abs().sum().item()


# ---------------------------------------------------------------- generic engine: known answers
def test_affine_2d_known_answer(drv, oracle_lib):
    """2x+1 on arange, the known answer of python/examples/test_load_2d_tensor_block.py:76-78, here with ragged masks."""
    M, N = 13, 21
    x = torch.arange(M * N, dtype=torch.int32).reshape(M, N)
    out = torch.full((M, N), -3, dtype=torch.int32, device="cuda")
    xd = x.cuda()
    K.affine_2d_kernel[(triton_cdiv(M, 4), triton_cdiv(N, 8))](xd, out, N, 1, M, N, BLOCK_M=4, BLOCK_N=8)
    assert torch.equal(out.cpu(), 2 * x + 1)
    # the oracle's block load/store agrees on one ragged block
    blk = oracle_lib.block_load(x.numpy().reshape(-1), (4, 8), (N, 1), 12 * N + 16, dims=(1, 5), other=0)
    assert np.array_equal(blk[0, :5], x.numpy()[12, 16:21]) and np.all(blk[1:] == 0) and np.all(blk[0, 5:] == 0)


def test_swap_known_answer(drv):
    x = torch.arange(0, 256, dtype=torch.float32, device="cuda")
    y = torch.arange(1000, 1256, dtype=torch.float32, device="cuda")
    xe, ye = y.clone(), x.clone()
    K.swap_kernel[(2,)](x, y, BLOCK=128)
    assert torch.equal(x, xe) and torch.equal(y, ye)


def test_mask_known_answers(drv):
    """Exact vectors of python/examples/test_mask.py:39,58,64."""
    inp = torch.arange(0, 8, dtype=torch.int32, device="cuda")
    out = torch.full((8,), -2, dtype=torch.int32, device="cuda")
    K.masked_other_kernel[(1,)](inp, out)
    assert out.cpu().tolist() == [-1, -1, -1, -1, -2, -2, -2, -2]
    out = torch.full((8,), -2, dtype=torch.int32, device="cuda")
    K.scalar_conj_mask_kernel[(1,)](inp, out, 4, 3)
    assert out.cpu().tolist() == [0, 1, 2, 3, -1, -1, -1, -1]
    out = torch.full((8,), -2, dtype=torch.int32, device="cuda")
    K.scalar_conj_mask_kernel[(1,)](inp, out, 4, 8)
    assert out.cpu().tolist() == [-1] * 8


def test_splat_and_float_arg(drv):
    out = torch.zeros(1000, device="cuda")
    K.splat_kernel[(4,)](out, 2.5, 1000, BLOCK=256)
    assert torch.all(out == 2.5)


def test_gelu_bias_fp16(drv):
    """A 25-op elementwise chain with fp16 I/O and broadcast bias through the register VM."""
    torch.manual_seed(5)
    rows, cols = 37, 1000
    x = torch.randn(rows, cols, device="cuda").half()
    b = torch.randn(cols, device="cuda").half()
    out = torch.zeros_like(x)
    K.gelu_bias_kernel[(rows, triton_cdiv(cols, 256))](x, b, out, cols, BLOCK=256)
    v = x.float() + b.float()
    ref = torch.nn.functional.gelu(v, approximate="tanh")
    assert torch.allclose(out.float(), ref, rtol=2e-3, atol=2e-3)


# ---------------------------------------------------------------- C ABI directly
def test_c_abi_softmax_and_errors(oracle_lib):
    _cuda()
    from triton_shared_b200 import runtime as rt
    L = rt.lib()
    torch.manual_seed(1)
    x = torch.randn(50, 781, device="cuda")
    out = torch.empty_like(x)
    rc = L.tsb_softmax_rows(x.data_ptr(), out.data_ptr(), 0, 781, 781, 781, 1024, 0, 50, 0)
    assert rc == 0, L.tsb_last_error()
    torch.cuda.synchronize()
    ref = oracle_lib.softmax(x.cpu().numpy(), 1024)
    np.testing.assert_allclose(out.cpu().numpy(), ref, rtol=1e-5, atol=1e-8)
    # errors are codes + text, never exceptions or faults
    assert L.tsb_softmax_rows(None, out.data_ptr(), 0, 781, 781, 781, 1024, 0, 50, 0) == -1
    assert b"null" in L.tsb_last_error()
    assert L.tsb_softmax_rows(x.data_ptr(), out.data_ptr(), 0, 781, 781, 10 ** 6, 1 << 20, 0, 50, 0) == -2


def test_c_abi_block_copy_strided(oracle_lib):
    """tsb_block_copy against the oracle's strided copy on a transposing descriptor."""
    _cuda()
    from triton_shared_b200 import runtime as rt
    L = rt.lib()
    src = torch.arange(64 * 48, dtype=torch.float32)
    dst = torch.full((64 * 48,), -1.0)
    a, b = rt.Access(), rt.Access()
    sd, dd = src.cuda(), dst.cuda()
    for acc, base, strides in ((a, sd, (48, 1)), (b, dd, (1, 64))):
        acc.base = base.data_ptr()
        acc.dtype = 0
        acc.rank = 2
        acc.sizes[0], acc.sizes[1] = 16, 16
        acc.strides[0], acc.strides[1] = strides
        acc.masked[0] = acc.masked[1] = 1
        acc.mask_bound[0], acc.mask_bound[1] = 60, 45  # ragged: 64x48 tile space cut to 60x45
        acc.mask_start_pid[0][0] = 16  # rows follow program_id(0)
        acc.mask_start_pid[1][1] = 16  # cols follow program_id(1)
    a.offset_pid[0], a.offset_pid[1] = 16 * 48, 16
    b.offset_pid[0], b.offset_pid[1] = 16, 16 * 64
    grid = (ctypes.c_int32 * 3)(4, 3, 1)
    assert L.tsb_block_copy(ctypes.byref(a), ctypes.byref(b), grid, 0, 12, 0) == 0, L.tsb_last_error()
    torch.cuda.synchronize()
    exp = dst.numpy().copy()
    s = src.numpy()
    for pm in range(4):
        for pn in range(3):
            dims = (oracle_lib.mask_dim(16 * pm, 16, 60), oracle_lib.mask_dim(16 * pn, 16, 45))
            blk = oracle_lib.block_load(s, (16, 16), (48, 1), pm * 16 * 48 + pn * 16, dims=dims)
            oracle_lib.block_store(exp, (16, 16), (1, 64), pm * 16 + pn * 16 * 64, blk, dims=dims)
    assert np.array_equal(dd.cpu().numpy(), exp)


def test_partitioned_launch_matches_full(drv, oracle_lib):
    """Two disjoint program ranges (what two GPUs would run) reproduce the single launch bit for bit."""
    n = 98_432
    torch.manual_seed(0)
    x = torch.rand(n, device="cuda")
    y = torch.rand(n, device="cuda")
    full = torch.empty_like(x)
    K.add_kernel[(97,)](x, y, full, n, BLOCK_SIZE=1024)
    parts = torch.zeros_like(x)
    for rank in range(2):
        with drv.partition(rank, 2):
            K.add_kernel[(97,)](x, y, parts, n, BLOCK_SIZE=1024)
    assert torch.equal(full, parts)


def test_loops_and_wraparound_known_answers(drv):
    """Loops without carried data (walked on the host) and wrap-around offsets, against the exact
    expected matrices of python/examples/test_modulo.py:45-50 and :88-97 and plain copies."""
    from test_cpu_host import _loop_and_wrap_cases
    for name, got, exp in _loop_and_wrap_cases("cuda"):
        assert torch.equal(got, exp), name


def test_wraparound_large_blocks(drv):
    """Row wrap-around on vector-width blocks: rows (START + i) % M, 16-byte path on the columns."""
    M, N = 48, 256
    A = torch.randn(M, N, device="cuda")
    C = torch.zeros(64, N, device="cuda")
    K.wrap_rows_kernel[(1,)](A, C, M, N, 1, N, 1, START=40, BM=64, BN=64, STEPS=4)
    rows = (40 + torch.arange(64, device="cuda")) % M
    assert torch.equal(C, A[rows])


def test_block_programs(drv):
    """Bodies with tt.reduce (sum to scalar, RMS norm, axis-0 and axis-1 integer max/min): block-program kernel."""
    from test_cpu_host import _block_program_cases
    for name, got, exp, tol in _block_program_cases("cuda"):
        if tol == 0:
            assert torch.equal(got, exp), name
        else:
            assert torch.allclose(got, exp, rtol=tol, atol=tol), name


def test_mixed_elementwise_ops(drv):
    """where / exp / sqrt / log / trig / floor, integer division, remainder, shifts and bit ops,
    int <-> float casts and uint8 I/O through the register VM, against torch."""
    from test_cpu_host import _mixed_op_cases
    for name, got, exp, tol in _mixed_op_cases("cuda"):
        if tol == 0:
            assert torch.equal(got, exp), name
        else:
            assert torch.allclose(got, exp, rtol=tol, atol=tol), name


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.uint8])
@pytest.mark.parametrize("M,N", [(1000, 1000), (130, 72), (64, 128)])
def test_block_copy_2d(drv, dtype, M, N):
    """Masked strided 2-D block copy: aligned rows take the lean 16-byte kernel, a transposed
    destination and odd pitches the general one; nothing outside the mask is written."""
    torch.manual_seed(9)
    src = (torch.rand(M, N, device="cuda") * 200).to(dtype)
    grid = ((M + 63) // 64, (N + 127) // 128)
    # row-major -> row-major inside a padded buffer (guard columns must stay untouched)
    pad = torch.full((M, N + 16), 7, dtype=dtype, device="cuda")
    K.copy_2d_kernel[grid](src, pad, M, N, N, 1, N + 16, 1, BM=64, BN=128)
    assert torch.equal(pad[:, :N], src) and torch.all(pad[:, N:] == 7)
    # row-major -> column-major (transposing store: unit stride along rows)
    dst_t = torch.zeros(N, M, dtype=dtype, device="cuda")
    K.copy_2d_kernel[grid](src, dst_t, M, N, N, 1, 1, M, BM=64, BN=128)
    assert torch.equal(dst_t.t(), src)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("rows,cols,src_rows", [(1000, 520, 777), (64, 100, 64)])
def test_gather_rows_known_answer(drv, dtype, rows, cols, src_rows):
    """Row gather through a loaded index (int64, as torch produces it): exact against indexing,
    ragged against the 16 x 128 tiles, nothing written outside the mask."""
    import kernels as K
    torch.manual_seed(9)
    x = torch.randn(src_rows, cols, device="cuda").to(dtype)
    idx = torch.randint(0, src_rows, (rows,), device="cuda")
    out = torch.full((rows + 3, cols + 5), -5.0, device="cuda", dtype=dtype)
    K.gather_rows_kernel[((rows + 15) // 16, (cols + 127) // 128)](x, idx, out, rows, cols, x.stride(0), out.stride(0),
                                                                   BLOCK_M=16, BLOCK_N=128)
    torch.cuda.synchronize()
    assert torch.equal(out[:rows, :cols], x[idx])
    assert torch.all(out[rows:] == -5.0) and torch.all(out[:, cols:] == -5.0)


# ---------------------------------------------------------------- packed VM kernel: accessor modes
_PAD_DTYPES = [torch.float32, torch.float16, torch.bfloat16, torch.int32, torch.int16, torch.int8, torch.uint8]


@pytest.mark.parametrize("dtype", _PAD_DTYPES, ids=lambda d: str(d)[6:])
@pytest.mark.parametrize("n_cols", [1024, 1000, 1001, 4, 3])
def test_padded_scale_2d_exact(drv, dtype, n_cols):
    """x*2 + b over a (row, column block) grid with masked loads filled by 3 and an unmasked store.
    n_cols a multiple of 4 keeps every vector aligned (lean accessors, ragged last sub-items);
    odd n_cols makes rows unaligned (general accessors).  Small integers: every type computes exactly."""
    BLOCK, rows = 256, 37
    nb = (n_cols + BLOCK - 1) // BLOCK
    g = torch.Generator().manual_seed(n_cols)
    x = torch.randint(0, 20, (rows, n_cols), generator=g).to(dtype)
    b = torch.randint(0, 20, (n_cols,), generator=g).to(dtype)
    out = torch.full((rows + 1, nb * BLOCK), 99, dtype=dtype, device="cuda")  # one guard row
    K.pad_scale_kernel[(rows, nb)](x.cuda(), b.cuda(), out, n_cols, nb * BLOCK, BLOCK=BLOCK)
    torch.cuda.synchronize()
    exp = torch.full((rows, nb * BLOCK), 3 * 2 + 3, dtype=torch.int64)
    exp[:, :n_cols] = x.to(torch.int64) * 2 + b.to(torch.int64)
    assert torch.equal(out[:rows].cpu().to(torch.int64), exp)
    assert torch.all(out[rows] == 99), "stored outside the grid's blocks"
    assert _loaded_native()


def test_bias_add_beyond_32bit_offsets(drv):
    """A 2-D body whose element offsets pass 2^31 (and whose byte offsets pass 2^32): program and
    block offsets are 64-bit, only the offset inside one block is 32-bit."""
    rows, cols = 66_000, 32_768  # 2.16e9 elements of fp16 = 4.3 GB per tensor
    x = torch.empty(rows, cols, dtype=torch.float16, device="cuda")
    x.copy_((torch.arange(rows, device="cuda") % 64).to(torch.float16)[:, None].expand(rows, cols))
    b = (torch.arange(cols, device="cuda") % 32).to(torch.float16)
    out = torch.empty_like(x)
    K.pad_scale_kernel[(rows, cols // 1024)](x, b, out, cols, cols, BLOCK=1024)
    torch.cuda.synchronize()
    for r in (0, 1, 65_535, 65_536, rows - 1):  # rows either side of the 2^31-element line
        exp = (r % 64) * 2.0 + (torch.arange(cols) % 32).to(torch.float32)
        assert torch.equal(out[r].float().cpu(), exp), r
    # checksum of the whole result: sum over rows of (2*(r%64)*cols + sum(b))
    total = out.double().sum().item()
    want = sum(2.0 * (r % 64) for r in range(rows)) * cols + rows * float((torch.arange(cols) % 32).sum())
    assert total == want


@pytest.mark.parametrize("block", [16, 64, 128, 512, 1024, 4096])
@pytest.mark.parametrize("dtype", [torch.int32, torch.float32], ids=["i32", "f32"])
def test_row_folds_on_the_elementwise_engine(drv, dtype, block):
    """x - max(x) + sum(x) per row for every size of thread group a program can have in the packed
    kernel (1 thread to the whole CTA), ragged rows (masked lanes take part with the fill value 0, as in
    the kernel text).  Integers exactly; floats against a float64 fold (rel 1e-5: the fold order differs)."""
    rows, n_cols = 53, block - 3
    g = torch.Generator().manual_seed(block)
    if dtype == torch.int32:
        x = torch.randint(-50, 1000, (rows, block), generator=g, dtype=torch.int32)
    else:
        x = torch.rand(rows, block, generator=g) + 0.5
    xd = x.cuda()
    y = torch.full_like(xd, -7)
    K.row_center_kernel[(rows,)](xd, y, block, n_cols, BLOCK=block)
    torch.cuda.synchronize()
    xv = x[:, :n_cols].double()
    mx = torch.clamp(xv.max(dim=1, keepdim=True).values, min=0.0)  # the masked lanes hold 0
    exp = xv - mx + xv.sum(dim=1, keepdim=True)
    got = y[:, :n_cols].cpu().double()
    if dtype == torch.int32:
        assert torch.equal(got, exp)
    else:
        assert torch.allclose(got, exp, rtol=1e-5, atol=0)
    assert torch.all(y[:, n_cols:] == -7), "stored beyond the mask"
