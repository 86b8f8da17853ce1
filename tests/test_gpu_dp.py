"""Data parallelism through the C ABI on 2 GPUs of one box (skipped with fewer): tests/dp_worker.py under
torch.distributed.run, one process per GPU."""
import pathlib
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = pathlib.Path(__file__).resolve().parent


@pytest.mark.parametrize("variant", ["flat", "hier"])
def test_dp_step_averages_gradients_eager_and_captured(variant):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import __graft_entry__ as ge
    ge.build()
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29531", str(HERE / "dp_worker.py"), variant]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("OK") == 2, r.stdout


def test_single_rank_communicator_collectives():
    # world size 1 on one GPU: the all-reduce is the identity, the all-gather a copy, the step equals the plain step
    import __graft_entry__ as ge
    ge.build()
    import pm_b200 as pm
    dp = pm.DataParallel(1, 0, pm.DataParallel.unique_id())
    try:
        assert dp.nranks == 1
        g = torch.Generator(device="cuda"); g.manual_seed(3)
        x = torch.randn(1000, device="cuda", generator=g)
        ref = x.clone()
        dp.all_reduce_async(x); dp.sync()
        send = torch.randn(257, 3, device="cuda", generator=g)
        recv = torch.zeros_like(send)
        dp.all_gather_async(send, recv); dp.sync()
        ids = torch.arange(64, device="cuda", dtype=torch.int64)
        ids_all = torch.zeros_like(ids)
        dp.all_gather_async(ids, ids_all); dp.sync()
        torch.cuda.synchronize()
        assert torch.equal(x, ref) and torch.equal(recv, send) and torch.equal(ids_all, ids)
        with pytest.raises(ValueError):
            dp.all_gather_async(send, torch.zeros(5, device="cuda"))
    finally:
        dp.close()
