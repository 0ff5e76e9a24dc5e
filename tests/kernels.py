"""Triton kernels used by the tests, the smoke check and the benchmark.

They are written in the style of the reference's python/examples (one program per
block / row / tile, masked tails) and exercise exactly the lowered constructs the
backend executes: structured block loads and stores, elementwise bodies,
reductions and tt.dot.
"""
import triton
import triton.language as tl


@triton.jit
def add_kernel(x_ptr, y_ptr, out_ptr, n_elements, BLOCK_SIZE: tl.constexpr):
    pid = tl.program_id(axis=0)
    offsets = pid * BLOCK_SIZE + tl.arange(0, BLOCK_SIZE)
    mask = offsets < n_elements
    x = tl.load(x_ptr + offsets, mask=mask)
    y = tl.load(y_ptr + offsets, mask=mask)
    tl.store(out_ptr + offsets, x + y, mask=mask)


@triton.jit
def softmax_kernel(out_ptr, in_ptr, in_row_stride, out_row_stride, n_cols, BLOCK_SIZE: tl.constexpr):
    row = tl.program_id(0)
    cols = tl.arange(0, BLOCK_SIZE)
    x = tl.load(in_ptr + row * in_row_stride + cols, mask=cols < n_cols, other=-float('inf'))
    z = x - tl.max(x, axis=0)
    num = tl.exp(z)
    den = tl.sum(num, axis=0)
    tl.store(out_ptr + row * out_row_stride + cols, num / den, mask=cols < n_cols)


@triton.jit
def layernorm_fwd_kernel(X, Y, W, B, Mean, Rstd, stride, N, eps, BLOCK_SIZE: tl.constexpr):
    row = tl.program_id(0)
    Y += row * stride
    X += row * stride
    acc = tl.zeros([BLOCK_SIZE], dtype=tl.float32)
    for off in range(0, N, BLOCK_SIZE):
        cols = off + tl.arange(0, BLOCK_SIZE)
        acc += tl.load(X + cols, mask=cols < N, other=0.).to(tl.float32)
    mean = tl.sum(acc, axis=0) / N
    acc2 = tl.zeros([BLOCK_SIZE], dtype=tl.float32)
    for off in range(0, N, BLOCK_SIZE):
        cols = off + tl.arange(0, BLOCK_SIZE)
        x = tl.load(X + cols, mask=cols < N, other=0.).to(tl.float32)
        x = tl.where(cols < N, x - mean, 0.)
        acc2 += x * x
    var = tl.sum(acc2, axis=0) / N
    rstd = 1 / tl.sqrt(var + eps)
    tl.store(Mean + row, mean)
    tl.store(Rstd + row, rstd)
    for off in range(0, N, BLOCK_SIZE):
        cols = off + tl.arange(0, BLOCK_SIZE)
        mask = cols < N
        w = tl.load(W + cols, mask=mask)
        b = tl.load(B + cols, mask=mask)
        x = tl.load(X + cols, mask=mask, other=0.).to(tl.float32)
        y = (x - mean) * rstd * w + b
        tl.store(Y + cols, y, mask=mask)


@triton.jit
def matmul_kernel(a_ptr, b_ptr, c_ptr, M, N, K, stride_am, stride_ak, stride_bk, stride_bn, stride_cm,
                  stride_cn, BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr,
                  GROUP_M: tl.constexpr):
    """C = A @ B with masked M/N/K tails and the grouped program order."""
    pid = tl.program_id(axis=0)
    num_pid_m = tl.cdiv(M, BLOCK_M)
    num_pid_n = tl.cdiv(N, BLOCK_N)
    num_pid_in_group = GROUP_M * num_pid_n
    group_id = pid // num_pid_in_group
    first_pid_m = group_id * GROUP_M
    group_size_m = min(num_pid_m - first_pid_m, GROUP_M)
    pid_m = first_pid_m + (pid % group_size_m)
    pid_n = (pid % num_pid_in_group) // group_size_m
    offs_m = pid_m * BLOCK_M + tl.arange(0, BLOCK_M)
    offs_n = pid_n * BLOCK_N + tl.arange(0, BLOCK_N)
    offs_k = tl.arange(0, BLOCK_K)
    a_ptrs = a_ptr + (offs_m[:, None] * stride_am + offs_k[None, :] * stride_ak)
    b_ptrs = b_ptr + (offs_k[:, None] * stride_bk + offs_n[None, :] * stride_bn)
    acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float32)
    for k in range(0, tl.cdiv(K, BLOCK_K)):
        a = tl.load(a_ptrs, mask=(offs_m[:, None] < M) & (offs_k[None, :] < K - k * BLOCK_K), other=0.0)
        b = tl.load(b_ptrs, mask=(offs_k[:, None] < K - k * BLOCK_K) & (offs_n[None, :] < N), other=0.0)
        acc = tl.dot(a, b, acc)
        a_ptrs += BLOCK_K * stride_ak
        b_ptrs += BLOCK_K * stride_bk
    c = acc.to(c_ptr.dtype.element_ty)
    c_ptrs = c_ptr + stride_cm * offs_m[:, None] + stride_cn * offs_n[None, :]
    tl.store(c_ptrs, c, mask=(offs_m[:, None] < M) & (offs_n[None, :] < N))


@triton.jit
def row_sum_kernel(x_ptr, out_ptr, M, N, stride_m, stride_n, BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr):
    """out[i] = sum_j x[i*stride_m + j*stride_n] for j < N: ragged 2-D blocks, sum along axis 1."""
    pid = tl.program_id(0)
    offs_m = pid * BLOCK_M + tl.arange(0, BLOCK_M)
    acc = tl.zeros([BLOCK_M], dtype=tl.float32)
    for n0 in range(0, N, BLOCK_N):
        offs_n = n0 + tl.arange(0, BLOCK_N)
        ptrs = x_ptr + offs_m[:, None] * stride_m + offs_n[None, :] * stride_n
        mask = (offs_m[:, None] < M) & (offs_n[None, :] < N)
        x = tl.load(ptrs, mask=mask, other=0.0)
        acc += tl.sum(x, axis=1)
    tl.store(out_ptr + offs_m, acc, mask=offs_m < M)


@triton.jit
def total_kernel(x_ptr, out_ptr, n, BLOCK: tl.constexpr):
    """out[0] = sum of x[0:n]; a single program."""
    acc = tl.zeros([BLOCK], dtype=tl.float32)
    for off in range(0, n, BLOCK):
        offs = off + tl.arange(0, BLOCK)
        acc += tl.load(x_ptr + offs, mask=offs < n, other=0.0)
    tl.store(out_ptr, tl.sum(acc, axis=0))


# ---- small kernels covering the generic structured-access engine -----------------

@triton.jit
def affine_2d_kernel(x_ptr, out_ptr, stride_m, stride_n, M, N, BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr):
    """out = 2*x + 1 on masked 2-D blocks (2-D program grid)."""
    pm = tl.program_id(0)
    pn = tl.program_id(1)
    offs_m = pm * BLOCK_M + tl.arange(0, BLOCK_M)
    offs_n = pn * BLOCK_N + tl.arange(0, BLOCK_N)
    mask = (offs_m[:, None] < M) & (offs_n[None, :] < N)
    offs = offs_m[:, None] * stride_m + offs_n[None, :] * stride_n
    x = tl.load(x_ptr + offs, mask=mask, other=0)
    tl.store(out_ptr + offs, 2 * x + 1, mask=mask)


@triton.jit
def swap_kernel(x_ptr, y_ptr, BLOCK: tl.constexpr):
    offs = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)
    x = tl.load(x_ptr + offs)
    y = tl.load(y_ptr + offs)
    tl.store(x_ptr + offs, y)
    tl.store(y_ptr + offs, x)


@triton.jit
def masked_other_kernel(in_ptr, out_ptr):
    """Fully masked-off load: every lane takes `other`."""
    offs = 100 + tl.arange(0, 4)
    a = tl.load(in_ptr + offs, mask=offs < 4, other=-1)
    tl.store(out_ptr + tl.arange(0, 4), a)


@triton.jit
def scalar_conj_mask_kernel(in_ptr, out_ptr, bound, value):
    offs = tl.arange(0, 8)
    a = tl.load(in_ptr + offs, mask=(value < 5) & (offs < bound), other=-1)
    tl.store(out_ptr + offs, a)


@triton.jit
def splat_kernel(out_ptr, fill, n, BLOCK: tl.constexpr):
    offs = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)
    v = tl.full([BLOCK], 0, dtype=tl.float32) + fill
    tl.store(out_ptr + offs, v, mask=offs < n)


@triton.jit
def gelu_bias_kernel(x_ptr, b_ptr, out_ptr, n_cols, BLOCK: tl.constexpr):
    """Row-broadcast bias + tanh-GELU in fp16 I/O with fp32 math (2-D grid: row, column block)."""
    row = tl.program_id(0)
    cols = tl.program_id(1) * BLOCK + tl.arange(0, BLOCK)
    m = cols < n_cols
    x = tl.load(x_ptr + row * n_cols + cols, mask=m, other=0.0).to(tl.float32)
    b = tl.load(b_ptr + cols, mask=m, other=0.0).to(tl.float32)
    v = x + b
    inner = 0.7978845608028654 * (v + 0.044715 * v * v * v)
    e = tl.exp(2.0 * inner)
    t = 1.0 - 2.0 / (e + 1.0)
    y = 0.5 * v * (1.0 + t)
    tl.store(out_ptr + row * n_cols + cols, y.to(tl.float16), mask=m)


@triton.jit
def matmul_wrap_kernel(a_ptr, b_ptr, c_ptr, M, N, K, stride_am, stride_ak, stride_bk, stride_bn, stride_cm,
                       stride_cn, BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr,
                       GROUP_M: tl.constexpr):
    """Same product, but the row/column offsets of A and B wrap modulo M and N instead of
    being masked (the form of python/examples/test_matmul.py: split pointers in the reference)."""
    pid = tl.program_id(axis=0)
    num_pid_m = tl.cdiv(M, BLOCK_M)
    num_pid_n = tl.cdiv(N, BLOCK_N)
    num_pid_in_group = GROUP_M * num_pid_n
    group_id = pid // num_pid_in_group
    first_pid_m = group_id * GROUP_M
    group_size_m = min(num_pid_m - first_pid_m, GROUP_M)
    pid_m = first_pid_m + (pid % group_size_m)
    pid_n = (pid % num_pid_in_group) // group_size_m
    offs_am = (pid_m * BLOCK_M + tl.arange(0, BLOCK_M)) % M
    offs_bn = (pid_n * BLOCK_N + tl.arange(0, BLOCK_N)) % N
    offs_k = tl.arange(0, BLOCK_K)
    a_ptrs = a_ptr + (offs_am[:, None] * stride_am + offs_k[None, :] * stride_ak)
    b_ptrs = b_ptr + (offs_k[:, None] * stride_bk + offs_bn[None, :] * stride_bn)
    acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float32)
    for k in range(0, tl.cdiv(K, BLOCK_K)):
        a = tl.load(a_ptrs, mask=offs_k[None, :] < K - k * BLOCK_K, other=0.0)
        b = tl.load(b_ptrs, mask=offs_k[:, None] < K - k * BLOCK_K, other=0.0)
        acc = tl.dot(a, b, acc)
        a_ptrs += BLOCK_K * stride_ak
        b_ptrs += BLOCK_K * stride_bk
    c = acc.to(c_ptr.dtype.element_ty)
    offs_cm = pid_m * BLOCK_M + tl.arange(0, BLOCK_M)
    offs_cn = pid_n * BLOCK_N + tl.arange(0, BLOCK_N)
    c_ptrs = c_ptr + stride_cm * offs_cm[:, None] + stride_cn * offs_cn[None, :]
    tl.store(c_ptrs, c, mask=(offs_cm[:, None] < M) & (offs_cn[None, :] < N))


# ---- loops without carried data, and wrap-around (modulo) offsets ---------------------------

@triton.jit
def grid_stride_copy_kernel(y_ptr, x_ptr, size, iterations, BLOCK_SIZE: tl.constexpr):
    """Each program copies `iterations` blocks, striding by the whole grid; the index tensor and
    therefore the mask start are loop-carried (the form of python/examples/test_mask_loop_iter_arg.py)."""
    idx = tl.program_id(0) * BLOCK_SIZE + tl.arange(0, BLOCK_SIZE)
    stride = tl.num_programs(0) * BLOCK_SIZE
    for it in range(iterations):
        mask = idx < size
        x = tl.load(x_ptr + idx, mask=mask)
        tl.store(y_ptr + idx, x * 2.0, mask=mask)
        idx += stride


@triton.jit
def tile_walk_kernel(in_ptr, out_ptr, stride_m, stride_n, TM: tl.constexpr, TN: tl.constexpr,
                     NI: tl.constexpr, NJ: tl.constexpr):
    """Two nested loops walking NI x NJ tiles of TM x TN with loop-carried pointers."""
    offs_m = tl.arange(0, TM)
    offs_n = tl.arange(0, TN)
    a_ptrs = in_ptr + offs_m[:, None] * stride_m + offs_n[None, :] * stride_n
    c_ptrs = out_ptr + offs_m[:, None] * stride_m + offs_n[None, :] * stride_n
    for i in range(0, NI):
        a_row = a_ptrs
        c_row = c_ptrs
        for j in range(0, NJ):
            tl.store(c_row, tl.load(a_row) + 1.0)
            a_row += TN * stride_n
            c_row += TN * stride_n
        a_ptrs += TM * stride_m
        c_ptrs += TM * stride_m


@triton.jit
def wrap_rows_kernel(a_ptr, c_ptr, M, stride_am, stride_an, stride_cm, stride_cn, START: tl.constexpr,
                     BM: tl.constexpr, BN: tl.constexpr, STEPS: tl.constexpr):
    """Rows (START + i) % M of A, column block by column block, into rows i of C: the row index
    wraps around the matrix ("stacked" wrap-around of python/examples/test_modulo.py:7-52)."""
    offs_am = (START + tl.arange(0, BM)) % M
    offs_n = tl.arange(0, BN)
    a_ptrs = a_ptr + offs_am[:, None] * stride_am + offs_n[None, :] * stride_an
    c_ptrs = c_ptr + tl.arange(0, BM)[:, None] * stride_cm + offs_n[None, :] * stride_cn
    for k in range(0, STEPS):
        tl.store(c_ptrs, tl.load(a_ptrs))
        a_ptrs += BN * stride_an
        c_ptrs += BN * stride_cn


@triton.jit
def wrap_cols_kernel(a_ptr, c_ptr, N, row, stride_am, stride_an, stride_cn, START: tl.constexpr, BN: tl.constexpr):
    """Columns (START + j) % N of one row: the wrap is on the innermost dim
    ("side-by-side", python/examples/test_modulo.py:55-99)."""
    offs_an = (START + tl.arange(0, BN)) % N
    a = tl.load(a_ptr + row * stride_am + offs_an[None, :] * stride_an)
    tl.store(c_ptr + tl.arange(0, BN)[None, :] * stride_cn, a)


# ---- bodies with block reductions but no loop-carried accumulator ------------------------------

@triton.jit
def block_sum_kernel(x_ptr, out_ptr, stride, n_elements, BLOCK_SIZE: tl.constexpr):
    """One masked 1-D block per program, summed to a scalar (the shape of python/examples/test_reduce.py:9-30)."""
    pid = tl.program_id(0)
    offs = tl.arange(0, BLOCK_SIZE)
    x = tl.load(x_ptr + pid * stride + offs, mask=offs < n_elements, other=0.0)
    tl.store(out_ptr + pid, tl.sum(x, axis=0))


@triton.jit
def rmsnorm_kernel(x_ptr, w_ptr, y_ptr, stride, n_cols, eps, BLOCK: tl.constexpr):
    """y = x * rsqrt(mean(x^2) + eps) * w for one row per program (row fits one block)."""
    row = tl.program_id(0)
    cols = tl.arange(0, BLOCK)
    m = cols < n_cols
    x = tl.load(x_ptr + row * stride + cols, mask=m, other=0.0).to(tl.float32)
    w = tl.load(w_ptr + cols, mask=m, other=0.0).to(tl.float32)
    ms = tl.sum(x * x, axis=0) / n_cols
    y = x * (1.0 / tl.sqrt(ms + eps)) * w
    tl.store(y_ptr + row * stride + cols, y.to(y_ptr.dtype.element_ty), mask=m)


@triton.jit
def tile_max_kernel(x_ptr, rowmax_ptr, colmin_ptr, stride_m, M, N, BM: tl.constexpr, BN: tl.constexpr):
    """Row maxima and column minima of one ragged int32 tile per program (axis 1 and axis 0 reductions)."""
    pid = tl.program_id(0)
    offs_m = pid * BM + tl.arange(0, BM)
    offs_n = tl.arange(0, BN)
    mask = (offs_m[:, None] < M) & (offs_n[None, :] < N)
    x = tl.load(x_ptr + offs_m[:, None] * stride_m + offs_n[None, :], mask=mask, other=0)
    tl.store(rowmax_ptr + offs_m, tl.max(x, axis=1), mask=offs_m < M)
    tl.store(colmin_ptr + pid * BN + offs_n, tl.min(x, axis=0), mask=offs_n < N)


@triton.jit
def block_ptr_sum_kernel(x_ptr, out_ptr, stride, n_elements, BLOCK_SIZE: tl.constexpr):
    """Block-pointer form of a per-program 1-D sum with a boundary check
    (python/examples/test_reduce.py:9-30): Triton rewrites the block pointer into 64-bit offset
    arithmetic with a `>= 0` and a `< bound` mask."""
    pid = tl.program_id(0)
    bp = tl.make_block_ptr(base=x_ptr, shape=[n_elements * tl.num_programs(0)], strides=[1],
                           offsets=[stride * pid], block_shape=[BLOCK_SIZE], order=[0])
    x = tl.load(bp, boundary_check=[0])
    tl.store(out_ptr + pid, tl.sum(x, axis=0))


# ---- a spread of elementwise ops for the register VM ------------------------------------------

@triton.jit
def mixed_float_kernel(x_ptr, y_ptr, o1_ptr, o2_ptr, o3_ptr, n, slope, BLOCK: tl.constexpr):
    offs = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)
    m = offs < n
    x = tl.load(x_ptr + offs, mask=m, other=0.0)
    y = tl.load(y_ptr + offs, mask=m, other=1.0)
    leaky = tl.where(x > 0, x, slope * x)
    tl.store(o1_ptr + offs, leaky, mask=m)
    sig = 1.0 / (1.0 + tl.exp(-x))
    tl.store(o2_ptr + offs, tl.maximum(sig, tl.minimum(tl.abs(y), 0.75)) + tl.sqrt(tl.abs(x)) * tl.log(tl.abs(y) + 1.0), mask=m)
    tl.store(o3_ptr + offs, tl.floor(x * 4.0) + tl.cos(y) * tl.sin(x), mask=m)


@triton.jit
def mixed_int_kernel(a_ptr, b_ptr, o1_ptr, o2_ptr, o3_ptr, n, BLOCK: tl.constexpr):
    offs = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)
    m = offs < n
    a = tl.load(a_ptr + offs, mask=m, other=1)
    b = tl.load(b_ptr + offs, mask=m, other=1)
    tl.store(o1_ptr + offs, (a * 3 + b) // 7 + (a % 5) - tl.minimum(a, b), mask=m)
    tl.store(o2_ptr + offs, ((a & b) | (a ^ 21)) + (b << 2) + (a >> 1), mask=m)
    tl.store(o3_ptr + offs, (a.to(tl.float32) * 0.5 + offs.to(tl.float32)).to(tl.int32), mask=m)


@triton.jit
def bytes_kernel(x_ptr, o_ptr, n, BLOCK: tl.constexpr):
    """uint8 in, uint8 out: saturating brighten (narrow integer I/O through the 32-bit lanes)."""
    offs = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)
    m = offs < n
    x = tl.load(x_ptr + offs, mask=m, other=0).to(tl.int32)
    tl.store(o_ptr + offs, tl.minimum(x * 2 + 10, 255).to(tl.uint8), mask=m)


@triton.jit
def copy_2d_kernel(src_ptr, dst_ptr, M, N, s_sm, s_sn, d_sm, d_sn, BM: tl.constexpr, BN: tl.constexpr):
    """Masked strided 2-D block copy (one tile per program, 2-D grid): the lowered form is exactly
    reinterpret_cast + subview + memref.copy on both sides."""
    offs_m = tl.program_id(0) * BM + tl.arange(0, BM)
    offs_n = tl.program_id(1) * BN + tl.arange(0, BN)
    mask = (offs_m[:, None] < M) & (offs_n[None, :] < N)
    x = tl.load(src_ptr + offs_m[:, None] * s_sm + offs_n[None, :] * s_sn, mask=mask)
    tl.store(dst_ptr + offs_m[:, None] * d_sm + offs_n[None, :] * d_sn, x, mask=mask)


# ---- loops that carry block values, outside the dedicated families -----------------------------

@triton.jit
def row_stats_kernel(x_ptr, sum_ptr, max_ptr, stride, N, BLOCK: tl.constexpr):
    """Per row: sum and maximum over column chunks, two lane accumulators carried through the loop."""
    row = tl.program_id(0)
    s_acc = tl.zeros([BLOCK], dtype=tl.float32)
    m_acc = tl.full([BLOCK], -float("inf"), dtype=tl.float32)
    for off in range(0, N, BLOCK):
        cols = off + tl.arange(0, BLOCK)
        x = tl.load(x_ptr + row * stride + cols, mask=cols < N, other=0.0)
        s_acc += x
        m_acc = tl.maximum(m_acc, tl.where(cols < N, x, -float("inf")))
    tl.store(sum_ptr + row, tl.sum(s_acc, axis=0))
    tl.store(max_ptr + row, tl.max(m_acc, axis=0))


@triton.jit
def wide_softmax_kernel(out_ptr, in_ptr, stride, N, BLOCK: tl.constexpr):
    """Softmax of rows wider than one block: three loops over column chunks (max, sum, write)."""
    row = tl.program_id(0)
    m_acc = tl.full([BLOCK], -float("inf"), dtype=tl.float32)
    for off in range(0, N, BLOCK):
        cols = off + tl.arange(0, BLOCK)
        m_acc = tl.maximum(m_acc, tl.load(in_ptr + row * stride + cols, mask=cols < N, other=-float("inf")))
    m = tl.max(m_acc, axis=0)
    s_acc = tl.zeros([BLOCK], dtype=tl.float32)
    for off in range(0, N, BLOCK):
        cols = off + tl.arange(0, BLOCK)
        x = tl.load(in_ptr + row * stride + cols, mask=cols < N, other=-float("inf"))
        s_acc += tl.exp(x - m)
    s = tl.sum(s_acc, axis=0)
    for off in range(0, N, BLOCK):
        cols = off + tl.arange(0, BLOCK)
        x = tl.load(in_ptr + row * stride + cols, mask=cols < N, other=-float("inf"))
        tl.store(out_ptr + row * stride + cols, tl.exp(x - m) / s, mask=cols < N)


@triton.jit
def row_argmax_kernel(x_ptr, val_ptr, idx_ptr, stride, n, BLOCK: tl.constexpr):
    """Per row: the maximum and the index of its first occurrence."""
    row = tl.program_id(0)
    offs = tl.arange(0, BLOCK)
    x = tl.load(x_ptr + row * stride + offs, mask=offs < n, other=-float("inf"))
    tl.store(val_ptr + row, tl.max(x, axis=0))
    tl.store(idx_ptr + row, tl.argmax(x, axis=0))


@triton.jit
def tile_argmin_kernel(x_ptr, idx_ptr, stride_m, BM: tl.constexpr, BN: tl.constexpr):
    """Index of the smallest element of every row of a BM x BN tile (argmin along axis 1)."""
    offs_m = tl.program_id(0) * BM + tl.arange(0, BM)
    offs_n = tl.arange(0, BN)
    x = tl.load(x_ptr + offs_m[:, None] * stride_m + offs_n[None, :])
    tl.store(idx_ptr + offs_m, tl.argmin(x, axis=1))


@triton.jit
def row_cumsum_kernel(x_ptr, y_ptr, stride, n, BLOCK: tl.constexpr):
    """Inclusive running sum of each row (tl.cumsum -> tt.scan with an add region)."""
    row = tl.program_id(0)
    cols = tl.arange(0, BLOCK)
    m = cols < n
    x = tl.load(x_ptr + row * stride + cols, mask=m, other=0.0)
    tl.store(y_ptr + row * stride + cols, tl.cumsum(x, axis=0), mask=m)


@triton.jit
def tile_cumsum_kernel(x_ptr, y_ptr, stride_m, BM: tl.constexpr, BN: tl.constexpr):
    """Running sum along axis 1 of a 2-D int32 tile per program."""
    rows = tl.program_id(0) * BM + tl.arange(0, BM)
    cols = tl.arange(0, BN)
    offs = rows[:, None] * stride_m + cols[None, :]
    tl.store(y_ptr + offs, tl.cumsum(tl.load(x_ptr + offs), axis=1))


@triton.jit
def layernorm_bwd_dx_kernel(DX, DY, X, W, Mean, Rstd, stride, N, BLOCK_N: tl.constexpr):
    """Input gradient of LayerNorm, one row per program (the dx part of the tutorial's backward
    kernel; its lock-protected dw/db partial accumulation is not part of the reference's lowering)."""
    row = tl.program_id(0)
    cols = tl.arange(0, BLOCK_N)
    mask = cols < N
    x = tl.load(X + row * stride + cols, mask=mask, other=0).to(tl.float32)
    dy = tl.load(DY + row * stride + cols, mask=mask, other=0).to(tl.float32)
    w = tl.load(W + cols, mask=mask).to(tl.float32)
    mean = tl.load(Mean + row)
    rstd = tl.load(Rstd + row)
    xhat = (x - mean) * rstd
    wdy = w * dy
    xhat = tl.where(mask, xhat, 0.)
    wdy = tl.where(mask, wdy, 0.)
    c1 = tl.sum(xhat * wdy, axis=0) / N
    c2 = tl.sum(wdy, axis=0) / N
    dx = (wdy - (xhat * c1 + c2)) * rstd
    tl.store(DX + row * stride + cols, dx, mask=mask)


@triton.jit
def layernorm_bwd_dwdb_kernel(DW, DB, FINAL_DW, FINAL_DB, M, N, BLOCK_SIZE_M: tl.constexpr, BLOCK_SIZE_N: tl.constexpr):
    """Column sums of the partial weight / bias gradients (python/examples/test_layernorm.py's
    _layer_norm_bwd_dwdb; lowered form in kernel-05-layer-norm-dwdb.mlir)."""
    pid = tl.program_id(0)
    cols = pid * BLOCK_SIZE_N + tl.arange(0, BLOCK_SIZE_N)
    dw = tl.zeros((BLOCK_SIZE_M, BLOCK_SIZE_N), dtype=tl.float32)
    db = tl.zeros((BLOCK_SIZE_M, BLOCK_SIZE_N), dtype=tl.float32)
    for i in range(0, M, BLOCK_SIZE_M):
        rows = i + tl.arange(0, BLOCK_SIZE_M)
        mask = (rows[:, None] < M) & (cols[None, :] < N)
        offs = rows[:, None] * N + cols[None, :]
        dw += tl.load(DW + offs, mask=mask, other=0.)
        db += tl.load(DB + offs, mask=mask, other=0.)
    sum_dw = tl.sum(dw, axis=0)
    sum_db = tl.sum(db, axis=0)
    tl.store(FINAL_DW + cols, sum_dw, mask=cols < N)
    tl.store(FINAL_DB + cols, sum_db, mask=cols < N)


@triton.jit
def gather_rows_kernel(x_ptr, idx_ptr, out_ptr, n_rows, n_cols, stride_x, stride_o, BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr):
    """out[r, :] = x[idx[r], :]: one unstructured dim (rows picked by a loaded index), contiguous rows
    (the row form of the reference's index_select examples, tts.make_gather_scatter_tptr)."""
    rows = tl.program_id(0) * BLOCK_M + tl.arange(0, BLOCK_M)
    cols = tl.program_id(1) * BLOCK_N + tl.arange(0, BLOCK_N)
    rmask = rows < n_rows
    idx = tl.load(idx_ptr + rows, mask=rmask, other=0)
    m = rmask[:, None] & (cols[None, :] < n_cols)
    v = tl.load(x_ptr + idx[:, None] * stride_x + cols[None, :], mask=m, other=0.0)
    tl.store(out_ptr + rows[:, None] * stride_o + cols[None, :], v, mask=m)


@triton.jit
def pad_scale_kernel(x_ptr, b_ptr, out_ptr, n_cols, out_stride, BLOCK: tl.constexpr):
    """out[row, c] = x[row, c] * 2 + b[c] with masked loads filled by 3; the store is NOT masked, so
    the padded lanes of the last column block land in the (block-padded) output too."""
    row = tl.program_id(0)
    cols = tl.program_id(1) * BLOCK + tl.arange(0, BLOCK)
    m = cols < n_cols
    x = tl.load(x_ptr + row * n_cols + cols, mask=m, other=3)
    b = tl.load(b_ptr + cols, mask=m, other=3)
    tl.store(out_ptr + row * out_stride + cols, x * 2 + b)


@triton.jit
def row_center_kernel(x_ptr, y_ptr, stride, n_cols, BLOCK: tl.constexpr):
    """y = x - max(x) + sum(x) per row: two full folds of the one block the kernel stores."""
    row = tl.program_id(0)
    cols = tl.arange(0, BLOCK)
    m = cols < n_cols
    x = tl.load(x_ptr + row * stride + cols, mask=m, other=0)
    y = x - tl.max(x, axis=0) + tl.sum(x, axis=0)
    tl.store(y_ptr + row * stride + cols, y, mask=m)


@triton.jit
def bias_chain_kernel(x_ptr, b_ptr, o_ptr, C, NIT: tl.constexpr, BLOCK: tl.constexpr):
    """(x + b) followed by NIT times (v * 1.0001 + b) over a (row, column block) grid: an elementwise
    body of 1 + 2 * NIT ops whose length is a parameter."""
    row = tl.program_id(0)
    cols = tl.program_id(1) * BLOCK + tl.arange(0, BLOCK)
    m = cols < C
    x = tl.load(x_ptr + row * C + cols, mask=m).to(tl.float32)
    b = tl.load(b_ptr + cols, mask=m).to(tl.float32)
    v = x + b
    for i in tl.static_range(NIT):
        v = v * 1.0001 + b
    tl.store(o_ptr + row * C + cols, v.to(o_ptr.dtype.element_ty), mask=m)
