"""The reference project's own example tests, unmodified, through B200Driver on a GPU.

python/examples/conftest.py of microsoft/triton-shared activates ``CPUDriver`` and hands every test
``device = "cpu"``.  Here the same test functions run with ``B200Driver`` in that place and
``device = "cuda"``: the literal drop-in swap.  The examples are not part of this repository; point
TSB_REFERENCE_EXAMPLES at a checkout's python/examples directory to collect them (nothing is
collected without it).
"""
import pytest

import reference_examples as R

pytestmark = pytest.mark.gpu

_CASES = R.cases()


@pytest.mark.skipif(not _CASES, reason=f"{R.ENV} does not name a directory of reference examples")
@pytest.mark.parametrize("case", _CASES or [None], ids=[c[0] for c in _CASES] or ["none"])
def test_reference_example(case, tsb_driver):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    _, path, name, kw = case
    R.run_case(path, name, kw, "cuda")
    torch.cuda.synchronize()
    tsb_driver.check()
