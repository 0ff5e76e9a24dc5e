"""tsb_plan_create / tsb_launch: a launch plan's JSON text is all a host needs to run a kernel.

These tests use nothing of the Python launch path: the plan text comes out of the Triton compile
pipeline (the `plan` stage), and from there on only the C ABI is called through ctypes, the way the
reference's generated C++ launcher would (backend/driver.py:102-246 of microsoft/triton-shared).
Results are compared with the CPU oracle.
"""
import ctypes

import numpy as np
import pytest
import torch
import triton
from triton.backends.compiler import GPUTarget
from triton.compiler import ASTSource

import kernels as K
import triton_shared_b200 as tsb
from triton_shared_b200 import runtime as rt

pytestmark = pytest.mark.gpu
TARGET = GPUTarget(tsb.BACKEND_NAME, 100, 32)


def _plan_text(fn, signature, constexprs):
    return triton.compile(ASTSource(fn, signature, constexprs), target=TARGET).asm["plan"]


def _launch(text, grid, ptrs, scalars, n_args, scratch_ok=True):
    """ptrs: {position: device address}; scalars: {position: int | float}."""
    L = rt.lib()
    h = L.tsb_plan_create(text, len(text))
    assert h, L.tsb_last_error()
    try:
        P = (ctypes.c_void_p * n_args)()
        S = (rt.Scalar * n_args)()
        for k, v in ptrs.items():
            P[k] = v
        for k, v in scalars.items():
            if isinstance(v, float):
                S[k].kind, S[k].f = 2, v
            else:
                S[k].kind, S[k].i = 1, v
        g = (ctypes.c_int32 * 3)(*grid)
        total = grid[0] * grid[1] * grid[2]
        need = L.tsb_launch_scratch_bytes(h, g, 0, total, S, n_args)
        assert need >= 0, L.tsb_last_error()
        scratch = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
        status = torch.zeros(4, dtype=torch.int32, device="cuda")
        rc = L.tsb_launch(h, g, 0, total, 0, P, S, n_args, scratch.data_ptr() if scratch_ok else None,
                          need if scratch_ok else 0, status.data_ptr())
        msg = L.tsb_last_error().decode()
        torch.cuda.synchronize()
        return rc, msg, L.tsb_plan_family(h).decode(), status.cpu().tolist()
    finally:
        L.tsb_plan_destroy(h)


def test_vec_add_from_plan_text(oracle_lib):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    n = 98_432
    text = _plan_text(K.add_kernel, {"x_ptr": "*fp32", "y_ptr": "*fp32", "out_ptr": "*fp32", "n_elements": "i32",
                                     "BLOCK_SIZE": "constexpr"}, {"BLOCK_SIZE": 1024})
    torch.manual_seed(0)
    x, y = torch.rand(n), torch.rand(n)
    xd, yd = x.cuda(), y.cuda()
    out = torch.full((n + 64,), -7.0, device="cuda")
    rc, msg, fam, _ = _launch(text, ((n + 1023) // 1024, 1, 1), {0: xd.data_ptr(), 1: yd.data_ptr(), 2: out.data_ptr()},
                              {3: n}, 4)
    assert rc == 0, msg
    assert fam == "elementwise"
    ref = oracle_lib.vec_add(x.numpy(), y.numpy(), n, 1024)
    assert np.array_equal(out[:n].cpu().numpy().view(np.uint32), ref.view(np.uint32))
    assert torch.all(out[n:] == -7.0)  # nothing stored beyond the mask


def test_matmul_from_plan_text(oracle_lib):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    M, N, Kd = 300, 520, 200  # ragged against 128 x 256 x 64 blocks
    sig = {"a_ptr": "*bf16", "b_ptr": "*bf16", "c_ptr": "*bf16", "M": "i32", "N": "i32", "K": "i32", "stride_am": "i32",
           "stride_ak": "i32", "stride_bk": "i32", "stride_bn": "i32", "stride_cm": "i32", "stride_cn": "i32",
           "BLOCK_M": "constexpr", "BLOCK_N": "constexpr", "BLOCK_K": "constexpr", "GROUP_M": "constexpr"}
    text = _plan_text(K.matmul_kernel, sig, {"BLOCK_M": 128, "BLOCK_N": 256, "BLOCK_K": 64, "GROUP_M": 8})
    torch.manual_seed(3)
    A = (2 * torch.rand(M, Kd) - 1).bfloat16()
    B = (2 * torch.rand(Kd, N) - 1).bfloat16()
    Ad, Bd = A.cuda(), B.cuda()
    C = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    grid = (-(-M // 128) * -(-N // 256), 1, 1)
    scal = {3: M, 4: N, 5: Kd, 6: Kd, 7: 1, 8: N, 9: 1, 10: N, 11: 1}
    rc, msg, fam, status = _launch(text, grid, {0: Ad.data_ptr(), 1: Bd.data_ptr(), 2: C.data_ptr()}, scal, 12)
    assert rc == 0, msg
    assert fam == "gemm" and status[0] == 0
    bits = lambda t: t.view(torch.int16).numpy().view(np.uint16)
    ref = oracle_lib.matmul(bits(A), bits(B), oracle_lib.BF16, 128, 256, 64, 8, threads=oracle_lib.max_threads())
    ref = torch.from_numpy(ref.view(np.int16).copy()).view(torch.bfloat16).float().numpy()
    np.testing.assert_allclose(C.float().cpu().numpy(), ref, rtol=1e-2, atol=1e-2 * np.abs(ref).max())


def test_launch_errors_are_return_codes():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    L = rt.lib()
    assert not L.tsb_plan_create(b"{not json", -1)
    assert b"JSON" in L.tsb_last_error()
    assert not L.tsb_plan_create(b'{"family": "nope", "name": "k", "params": {}}', -1)
    assert b"unknown kernel family" in L.tsb_last_error()
