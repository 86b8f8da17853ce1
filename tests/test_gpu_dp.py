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
