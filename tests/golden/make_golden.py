"""Generates tests/golden/reference_kernels.npz.

Runs the reference's own example kernels (python/examples/test_vec_add.py,
test_softmax.py, test_layernorm.py, test_matmul.py of microsoft/triton-shared,
imported unmodified from a checkout) under Triton's CPU interpreter
(TRITON_INTERPRET=1) on small seeded inputs and stores inputs and outputs.  The
reference CPU backend itself cannot be built here (no MLIR/LLVM tools), so these
vectors pin the oracle to the kernels' Triton semantics rather than to the
backend's own binary output.

    TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/triton-shared
"""
import os
import sys
import types

assert os.environ.get("TRITON_INTERPRET") == "1", "run with TRITON_INTERPRET=1"
assert len(sys.argv) > 1, "usage: make_golden.py /path/to/triton-shared"
ref = sys.argv[1]

import numpy as np
import torch
import triton

# the example files import the reference's driver module, which needs MLIR tools; the
# interpreter never touches it
pkg = types.ModuleType("triton.backends.triton_shared")
pkg.__path__ = []
drv = types.ModuleType("triton.backends.triton_shared.driver")
drv.CPUDriver = object
sys.modules["triton.backends.triton_shared"] = pkg
sys.modules["triton.backends.triton_shared.driver"] = drv
sys.path.insert(0, os.path.join(ref, "python", "examples"))

import test_vec_add
import test_softmax
import test_layernorm
import test_matmul

out = {}

# vec-add: 5 programs of 1024, ragged tail of 904
torch.manual_seed(0)
n = 5000
x, y = torch.rand(n), torch.rand(n)
z = torch.empty(n)
test_vec_add.add_kernel[(triton.cdiv(n, 1024),)](x, y, z, n, BLOCK_SIZE=1024)
out.update(add_x=x.numpy(), add_y=y.numpy(), add_out=z.numpy())

# softmax: 16 rows of 781 columns, BLOCK 1024
torch.manual_seed(1)
a = torch.randn(16, 781)
o = torch.empty_like(a)
test_softmax.softmax_kernel[(16,)](o, a, a.stride(0), o.stride(0), 781, BLOCK_SIZE=1024)
out.update(sm_x=a.numpy(), sm_out=o.numpy())

# layernorm forward: 8 rows of 2500 fp16 columns, BLOCK 1024 (three chunks, ragged last)
torch.manual_seed(2)
M, N = 8, 2500
xh = torch.randn(M, N).half()
w = (torch.rand(N) + 0.5).half()
b = (0.1 * torch.randn(N)).half()
yh = torch.empty_like(xh)
mean = torch.empty(M, dtype=torch.float32)
rstd = torch.empty(M, dtype=torch.float32)
test_layernorm._layer_norm_fwd_fused[(M,)](xh, yh, w, b, mean, rstd, xh.stride(0), N, 1e-5, BLOCK_SIZE=1024)
out.update(ln_x=xh.numpy(), ln_w=w.numpy(), ln_b=b.numpy(), ln_y=yh.numpy(), ln_mean=mean.numpy(), ln_rstd=rstd.numpy())

# matmul: 96 x 72 @ 72 x 80 fp16, blocks 32/32/16, the reference kernel (offsets wrap modulo M, N)
torch.manual_seed(3)
A = (2 * torch.rand(96, 72) - 1).half()
B = (2 * torch.rand(72, 80) - 1).half()
C = torch.empty(96, 80, dtype=torch.float16)
grid = (triton.cdiv(96, 32) * triton.cdiv(80, 32),)
test_matmul.matmul_kernel[grid](A, B, C, 96, 80, 72, A.stride(0), A.stride(1), B.stride(0), B.stride(1),
                                C.stride(0), C.stride(1), BLOCK_SIZE_M=32, BLOCK_SIZE_N=32, BLOCK_SIZE_K=16,
                                GROUP_SIZE_M=8, ACTIVATION="")
out.update(mm_a=A.numpy(), mm_b=B.numpy(), mm_c=C.numpy())

path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_kernels.npz")
np.savez_compressed(path, **out)
print("wrote", path, {k: v.shape for k, v in out.items()})
