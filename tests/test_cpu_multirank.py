"""World-size-2 test of the multi-GPU host logic on CPU ranks (gloo): every rank launches only its
contiguous program range (disjoint outputs, no data-path collective); the strided-reduction
workload combines one scalar with an all-reduce."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, HERE)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import kernels as K
    import triton_shared_b200 as tsb
    from fake_tsb import fake_device
    drv = tsb.activate()
    n = 10_000
    torch.manual_seed(0)  # same inputs on every rank
    x, y = torch.rand(n), torch.rand(n)
    mine = torch.zeros(n)
    flat = torch.randn(256 * 96)
    rows = torch.zeros(256)
    tot = torch.zeros(1)
    with fake_device() as lib:
        with drv.partition(rank, world):
            K.add_kernel[(10,)](x, y, mine, n, BLOCK_SIZE=1024)
            K.row_sum_kernel[(4,)](flat, rows, 256, 90, 1, 256, BLOCK_M=64, BLOCK_N=32)
        K.total_kernel[(1,)](rows, tot, 256, BLOCK=1024)  # this rank's partial scalar
    written = (mine != 0).to(torch.int32)
    dist.all_reduce(written)  # how many ranks wrote each element
    dist.all_reduce(mine)     # disjoint outputs: the sum is the concatenation
    dist.all_reduce(rows)
    dist.all_reduce(tot)      # the one collective of the reduction workload
    if rank == 0:
        q.put((written.numpy(), mine.numpy(), (x + y).numpy(), rows.numpy(), tot.item(),
               flat.numpy().reshape(96, 256)[:90].sum(axis=0), [c for c in lib.calls]))
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_ranks_disjoint_ranges_and_scalar_combine():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    written, got, ref, rows, tot, rows_ref, calls = q.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert np.all(written == 1), "an element was written by zero or by two ranks"
    assert np.array_equal(got, ref)
    np.testing.assert_allclose(rows, rows_ref, rtol=1e-4, atol=1e-4)
    assert abs(tot - rows_ref.sum()) < 1e-2
    assert calls[0] == ("tsb_elementwise", 0, 5) and calls[1] == ("tsb_reduce_rows", 0, 128)
