"""The allocation-free gated-RMSNorm backward (collected last on purpose).

Some hosts cannot call cudaMalloc at the point where they need a kernel: they handed the whole GPU to their
own memory pool at start-up, or they sit in a loop that must never enter the driver's allocator.  For them
the library offers one entry point whose scratch is a fixed 4 MiB array inside the library image.  This test
drives it through the C ABI with caller-owned inputs and outputs only, twice in a row (the array keeps the
previous call's contents), and compares with the workspace-taking entry point."""
import ctypes as C

import pytest
import torch

from util import FP32_TOL, assert_close, randn

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pm():
    import __graft_entry__ as ge
    ge.build()
    import pm_b200
    assert torch.cuda.is_available()
    return pm_b200


def _case(pm, rows, width, seed):
    y = randn((rows, width), seed).cuda()
    zfull = randn((rows, width + 8), seed + 1).cuda()
    z = zfull[:, :width]
    w = (1 + randn((width,), seed + 2, 0.1)).cuda()
    dout = randn((rows, width), seed + 3).cuda()
    _, rstd = pm.gated_rmsnorm_fwd(y, z, w, 1e-5)
    return dout, y, z, w, rstd


def test_static_scratch_variant_matches_workspace_variant_twice_in_a_row(pm):
    # second case is smaller than the first, so stale rows of the shared array lie beyond what it reads
    # the third case (width and row pitch not multiples of 4) takes the scalar kernels instead of the float4 ones
    for rows, width, seed in ((2048, 1536, 1), (300, 256, 7), (100, 250, 11)):
        args = _case(pm, rows, width, seed)
        ref = pm.gated_rmsnorm_bwd(*args)
        got = pm.gated_rmsnorm_bwd_static(*args)      # outputs are caller-owned; the scratch is the library's array
        torch.cuda.synchronize()
        for name, a, b in zip(("dy", "dz", "dw"), got, ref):
            assert_close(a, b, tol=FP32_TOL, what=f"{name} rows={rows}")
            assert torch.equal(a, b), f"{name}: same kernels and order, expected identical bits"


def test_static_scratch_limit_is_enforced(pm):
    limit = pm.lib.pmb_gated_rmsnorm_bwd_static_max_bytes()
    assert limit == 4 << 20
    rows, width = 4 * 1024 + 4, 1024             # ceil(rows/4) * width * 4 = 4 MiB + 4 KiB
    args = _case(pm, rows, width, 3)
    with pytest.raises(pm.PmbError) as ei:
        pm.gated_rmsnorm_bwd_static(*args)
    assert ei.value.status == 1 and "built-in" in str(ei.value)
    pm.gated_rmsnorm_bwd(*args)                   # the workspace-taking entry point still serves this size
