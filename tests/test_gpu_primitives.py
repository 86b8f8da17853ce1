"""The primitive ops behind the rest of pm_core::Ops against torch on the CPU (known answers of
crates/pm-candle/src/ops_impl.rs:464-572 are the model: silu, sigmoid, softplus, cumsum, matmul ...)."""
import pytest
import torch
import torch.nn.functional as F

from util import assert_close, randn

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pm():
    import __graft_entry__ as ge
    ge.build()
    import pm_b200
    assert torch.cuda.is_available()
    return pm_b200


def test_unary_and_binary(pm):
    x, y = randn((37, 50), 1), randn((37, 50), 2)
    ref = {"neg": -x, "exp": x.exp(), "sqrt": x.abs().sqrt(), "silu": F.silu(x), "sigmoid": x.sigmoid(), "softplus": F.softplus(x),
           "mul_scalar": x * 1.5, "add_scalar": x + 0.25, "copy": x}
    for op, r in ref.items():
        src = x.abs() if op == "sqrt" else x
        s = 1.5 if op == "mul_scalar" else 0.25
        assert_close(pm.unary(op, src.cuda(), s), r, tol=1e-6, what=op)
    for op, r in {"add": x + y, "sub": x - y, "mul": x * y, "div": x / y}.items():
        assert_close(pm.binary(op, x.cuda(), y.cuda()), r, tol=1e-6, what=op)
    with pytest.raises(pm.PmbError):
        pm.binary("add", x.cuda(), y[:, :10].contiguous().cuda())


def test_views_as_strided_copies(pm):
    x = randn((4, 6, 10), 3)
    xc = x.cuda()
    narrow = pm.strided_copy(xc, (4, 6, 3), (60, 10, 1), offset=5)                 # narrow(dim 2, start 5, len 3)
    assert torch.equal(narrow.cpu(), x[:, :, 5:8])
    tr = pm.strided_copy(xc, (4, 10, 6), (60, 1, 10))                              # transpose(1, 2)
    assert torch.equal(tr.cpu(), x.transpose(1, 2).contiguous())
    row = randn((1, 10), 4)
    bc = pm.strided_copy(row.cuda(), (7, 10), (0, 1))                              # broadcast_as((7, 10))
    assert torch.equal(bc.cpu(), row.expand(7, 10))


def test_embedding_gather_log_softmax_sum_cumsum(pm):
    table = randn((50, 16), 5)
    ids = torch.randint(0, 50, (3, 9))
    out, bad = pm.embedding(table.cuda(), ids.cuda())
    assert torch.equal(out.cpu(), table[ids]) and int(bad) == 0
    ids[0, 0] = 50
    out, bad = pm.embedding(table.cuda(), ids.cuda())
    assert int(bad) == 1 and float(out[0, 0].abs().sum()) == 0.0
    x = randn((33, 301), 6, 3.0)
    ls = pm.log_softmax(x.cuda())
    assert_close(ls, F.log_softmax(x.double(), -1), tol=1e-6, what="log_softmax")
    idx = torch.randint(0, 301, (33,))
    g, bad = pm.gather_last(ls, idx.cuda())
    assert_close(g, F.log_softmax(x.double(), -1).gather(1, idx[:, None])[:, 0], tol=1e-6, what="gather")
    assert int(bad) == 0
    big = randn((1000, 517), 7)
    assert_close(pm.sum_all(big.cuda()), big.double().sum().reshape(1), tol=1e-5, what="sum_all")
    assert_close(pm.sum_all(big.cuda(), mean=True), big.double().mean().reshape(1), tol=1e-5, what="mean_all")
    c = randn((3, 64, 5), 8)
    assert_close(pm.cumsum(c.cuda(), 1), c.double().cumsum(1), tol=1e-6, what="cumsum")
