"""tsb_reduce_rows_static: the reduction for callers that cannot allocate device memory.

Some hosts have no way to hand the library a scratch buffer: a bare C/ctypes launcher with no
allocator, a process whose device memory is wholly owned by another framework, or a loop that
cannot afford cudaMalloc's synchronisation.  This entry point keeps its partial sums in a fixed
array inside the library instead.  The test calls it through the C ABI, twice in a row on
different data (the array keeps the previous call's contents), and requires the results to be
identical to tsb_reduce_rows given ordinary scratch; it also checks that an oversized shape is
refused rather than served by a hidden allocation.  It runs last so that a failure here cannot
mask any other test.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from triton_shared_b200 import runtime as rt
    return rt.lib()


# few rows and many columns: the shapes whose column splits exceed one thread-block cluster, so the
# partial sums go through scratch memory (larger row counts are combined on chip and need none)
@pytest.mark.parametrize("rows,cols_total,cols_valid", [(256, 20480, 20000), (1000, 6500, 6400)])
def test_static_scratch_matches_caller_scratch_twice(rows, cols_total, cols_valid):
    L = _lib()
    for seed in (11, 12):  # second call finds the first call's partials in the array
        torch.manual_seed(seed)
        x = torch.randn(rows * cols_total, device="cuda")
        need = L.tsb_reduce_rows_scratch_bytes(rows, cols_valid, 1, rows)
        assert 0 < need <= (1 << 20), "shape chosen so that partial sums are used and fit the built-in array"
        scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
        ref = torch.full((rows,), float("nan"), device="cuda")
        got = torch.full((rows,), float("nan"), device="cuda")
        rc = L.tsb_reduce_rows(x.data_ptr(), ref.data_ptr(), 1, rows, 1, cols_valid, 0, rows, scratch.data_ptr(), 0)
        assert rc == 0, L.tsb_last_error()
        rc = L.tsb_reduce_rows_static(x.data_ptr(), got.data_ptr(), 1, rows, 1, cols_valid, 0, rows, 0)
        assert rc == 0, L.tsb_last_error()
        torch.cuda.synchronize()
        # same kernels, same split, same order of additions: the tolerance the other reduction tests
        # use (1e-5 of sum|x|) is met with zero difference
        assert torch.equal(got, ref)
        exact = x.view(cols_total, rows)[:cols_valid].double().sum(dim=0)
        scale = x.view(cols_total, rows)[:cols_valid].abs().double().sum(dim=0)
        assert torch.all((got.double() - exact).abs() <= 1e-5 * scale)


def test_static_scratch_refuses_oversized_shapes():
    L = _lib()
    rows, cols = 4608, 8192  # 36 row tiles x 66 column splits of 4,608 partial sums: 1.2 MB, above the built-in 1 MiB
    assert L.tsb_reduce_rows_scratch_bytes(rows, cols, 1, rows) > (1 << 20)
    x = torch.zeros(16, device="cuda")  # never dereferenced: the call is refused before any launch
    out = torch.zeros(16, device="cuda")
    rc = L.tsb_reduce_rows_static(x.data_ptr(), out.data_ptr(), 1, rows, 1, cols, 0, rows, 0)
    assert rc == -2
    msg = L.tsb_last_error().decode()
    assert "built-in array" in msg and "tsb_reduce_rows" in msg
    torch.cuda.synchronize()
