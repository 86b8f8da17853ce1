"""GPU parity tests of the individual kernels against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import mamba2_oracle as orc
from util import GOLD, FP32_TOL, assert_close, rand, randn, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pm():
    import __graft_entry__ as ge
    ge.build()
    import pm_b200
    assert torch.cuda.is_available()
    return pm_b200


# ------------------------------------------------------------------------------------------------ GEMM
GEMM_SHAPES = [(256, 256, 128), (300, 200, 100), (128, 552, 128), (64, 40, 36), (1, 8, 4), (513, 129, 257)]


def _gemm_case(pm, M, N, K, ta, tb, engine, residual):
    a = randn((K, M) if ta else (M, K), 1)
    b = randn((N, K) if tb else (K, N), 2)
    r = randn((M, N), 3) if residual else None
    ref = (a.T if ta else a).double() @ (b.T if tb else b).double()
    if residual:
        ref = ref + r.double()
    out = pm.matmul(a.cuda(), b.cuda(), trans_a=ta, trans_b=tb, residual=None if r is None else r.cuda(), engine=engine)
    torch.cuda.synchronize()
    return rel_err(out, ref)


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_gemm_simt(pm, M, N, K, ta, tb):
    assert _gemm_case(pm, M, N, K, ta, tb, 1, residual=(M + ta) % 2 == 0) < 2e-6


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (300, 200, 100), (128, 552, 128), (64, 40, 36), (4, 8, 4),
                                   (516, 132, 260), (2048, 384, 768)])
@pytest.mark.parametrize("ta,tb", [(0, 1), (0, 0), (1, 0), (1, 1)])
@pytest.mark.parametrize("engine", [2, 3])      # 128x128 tiles / 128x64 tiles with two CTAs per SM
def test_gemm_tcgen05_3xtf32(pm, M, N, K, ta, tb, engine):
    e = _gemm_case(pm, M, N, K, ta, tb, engine, residual=(M + tb) % 2 == 0)
    assert pm.device_status() == 0
    assert e < 1e-5, e


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (304, 200, 104), (128, 552, 128), (64, 40, 32), (8, 8, 8),
                                   (520, 136, 264), (2048, 384, 768)])
@pytest.mark.parametrize("ta,tb", [(0, 1), (0, 0), (1, 0), (1, 1)])
@pytest.mark.parametrize("engine", [4, 5, 6])      # 128x128 single-CTA tiles / 256x256 / 256x128 CTA-pair tiles
def test_gemm_tcgen05_bf16_pairs(pm, M, N, K, ta, tb, engine):
    """fp32 operands split into (hi, lo) bf16 pairs, three kind::f16 MMAs per k-step: 16 mantissa bits per operand,
    so the error bound is ~2^-16 of the result's scale instead of the 3xTF32 kernel's ~2^-21."""
    e = _gemm_case(pm, M, N, K, ta, tb, engine, residual=(M + tb) % 2 == 0)
    assert pm.device_status() == 0
    assert e < 3e-5, e


@pytest.mark.parametrize("ta,tb", [(0, 1), (0, 0), (1, 0), (1, 1)])
def test_gemm_auto_takes_pair_tiles_for_many_tiles(pm, ta, tb):
    """17 x 18 = 306 tiles of 256x256 is above the threshold at which engine 0 switches to the CTA-pair kernel."""
    e = _gemm_case(pm, 4344, 4600, 136, ta, tb, 0, residual=bool(ta))
    assert pm.device_status() == 0
    assert e < 3e-5, e


def test_gemm_unaligned_is_refused_by_tc_and_taken_by_auto(pm):
    a, b = randn((33, 7), 1).cuda(), randn((7, 5), 2).cuda()
    with pytest.raises(pm.PmbError):
        pm.matmul(a, b, engine=2)
    out = pm.matmul(a, b, engine=0)
    assert rel_err(out, a.cpu().double() @ b.cpu().double()) < 3e-5    # auto: bf16 pairs through the library scratch


def test_gemm_inplace_residual(pm):
    a, b = randn((256, 128), 1).cuda(), randn((128, 256), 2).cuda()
    for eng in (1, 2):
        c = randn((256, 256), 3).cuda()
        ref = a.cpu().double() @ b.cpu().double() + c.cpu().double()
        pm.matmul(a, b, residual=c, out=c, engine=eng)
        assert rel_err(c, ref) < 1e-5


# ------------------------------------------------------------------------------------------------ conv
@pytest.mark.parametrize("B,T,H,P,N,G,K", [(2, 128, 8, 32, 16, 1, 4), (1, 37, 3, 5, 7, 3, 4), (2, 64, 4, 8, 8, 1, 2), (1, 300, 2, 16, 8, 1, 7)])
def test_conv_silu_dt_fwd_bwd(pm, B, T, H, P, N, G, K):
    cfg = pm.Mamba2Config(d_model=32, d_state=N, d_head=P, n_heads=H, n_groups=G, d_conv=K, block_len=T)
    I, X, J = cfg.d_inner, cfg.xbc_dim, cfg.in_proj_dim
    xzd = randn((B, T, J), 1).requires_grad_(True)
    w = randn((X, 1, K), 2, 0.5).requires_grad_(True)
    b = randn((X,), 3, 0.1).requires_grad_(True)
    dtb = randn((H,), 4)
    xbc = xzd[..., I:I + X].transpose(1, 2)
    conv = F.conv1d(xbc, w, None, padding=K - 1, groups=X) + b.reshape(-1, 1)
    act_ref = orc.silu(conv[..., :T].transpose(1, 2))
    dt_ref = orc.softplus(xzd[..., I + X:] + dtb)
    act, dt = pm.conv_silu_dt_fwd(cfg, xzd.detach().cuda(), w.detach().cuda(), b.detach().cuda(), dtb.cuda())
    assert_close(act, act_ref, what="act")
    assert_close(dt, dt_ref, what="dt")
    dact = randn((B, T, X), 5)
    (act_ref * dact).sum().backward()
    dxzd, dw, db = pm.conv_silu_bwd(cfg, xzd.detach().cuda(), w.detach().cuda(), b.detach().cuda(), dact.cuda())
    assert_close(dxzd[..., I:I + X], xzd.grad[..., I:I + X], what="dxbc")
    assert_close(dw, w.grad, what="dconv_w")
    assert_close(db, b.grad, what="dconv_b")


# ------------------------------------------------------------------------------------------------ gated RMSNorm
@pytest.mark.parametrize("rows,width", [(256, 256), (37, 1536), (5, 40)])
def test_gated_rmsnorm_fwd_bwd(pm, rows, width):
    y = randn((rows, width), 1).requires_grad_(True)
    zfull = randn((rows, width + 24), 2).requires_grad_(True)   # z lives inside a wider row (xzd)
    w = (1 + randn((width,), 3, 0.1)).requires_grad_(True)
    z = zfull[:, :width]
    ref = orc.rmsnorm(y * orc.silu(z), w, 1e-5)
    zc = zfull.detach().cuda()
    out, rstd = pm.gated_rmsnorm_fwd(y.detach().cuda(), zc[:, :width], w.detach().cuda(), 1e-5)
    assert_close(out, ref, what="normed")
    dout = randn((rows, width), 4)
    (ref * dout).sum().backward()
    dy, dz, dw = pm.gated_rmsnorm_bwd(dout.cuda(), y.detach().cuda(), zc[:, :width], w.detach().cuda(), rstd)
    assert_close(dy, y.grad, what="dy")
    assert_close(dz, zfull.grad[:, :width], what="dz")
    assert_close(dw, w.grad, what="dw")


# ------------------------------------------------------------------------------------------------ SSD scan
def test_ssd_reference_fixture(pm):
    # reference/fixtures/ssd_q64 (crates/pm-core/tests/ssd_fixture.rs:68-75 holds 5e-3)
    f = np.load(GOLD / "ssd_q64.npz")
    X, A, B, C = (torch.from_numpy(f[k]).cuda() for k in "XABC")
    scan = pm.SsdScan(X, A, B, C, 64)
    y, fs = scan.forward(want_final_state=True)
    assert np.abs(y.cpu().numpy() - f["Y"]).max() < 1e-4
    assert np.abs(fs.cpu().numpy().transpose(0, 1, 3, 2) - f["final_state"]).max() < 1e-4


def test_ssd_zero_a_running_sum(pm):
    # crates/pm-core/src/mamba2/ssd.rs:105-120
    b, t, h, p, n = 1, 4, 1, 2, 2
    x = torch.ones(b, t, h, p).cuda()
    a = torch.zeros(b, t, h).cuda()
    bb = (torch.arange(b * t * h * n, dtype=torch.float32) * 0.1).reshape(b, t, h, n).cuda()
    y = pm.ssd_scan(x, a, bb, bb.clone(), 4).cpu()
    expect = torch.tril(bb[0, :, 0].cpu() @ bb[0, :, 0].cpu().T).sum(-1)
    assert torch.allclose(y[0, :, 0, 0], expect, atol=1e-6) and torch.allclose(y[0, :, 0, 0], y[0, :, 0, 1])


SSD_CASES = [  # B, T, H, P, N, G, Q
    (2, 128, 8, 32, 16, 1, 64),     # single-block config dims
    (1, 128, 2, 8, 16, 2, 64),      # fixture dims, per-head B/C
    (2, 64, 4, 8, 8, 1, 16),        # many small chunks
    (1, 96, 3, 20, 12, 1, 96),      # one chunk, ragged tile sizes
    (1, 512, 4, 64, 64, 1, 256),    # production chunk length
    (2, 80, 2, 16, 8, 2, 40),       # chunk length not a multiple of the tile
    # shapes the tensor-core scan takes (block_len % 64 == 0, d_state % 32 == 0, d_head % 64 == 0)
    (2, 256, 4, 64, 32, 4, 64),     # per-head B/C, chunk shorter than the 128-row tile
    (1, 256, 2, 128, 128, 1, 128),  # wide head, large state
    (2, 512, 8, 64, 64, 1, 128),
    (1, 768, 3, 64, 64, 1, 256),    # three chunks of the production length
    (1, 1024, 2, 64, 32, 1, 512),   # chunk longer than one 256-thread round of the fused cumsum / row-sum kernels
]


@pytest.mark.parametrize("B,T,H,P,N,G,Q", SSD_CASES)
def test_ssd_fwd_bwd_vs_oracle(pm, B, T, H, P, N, G, Q):
    x = randn((B, T, H, P), 1).requires_grad_(True)
    a = (-rand((B, T, H), 2) * 0.5).requires_grad_(True)
    b = randn((B, T, G, N), 3, 0.5).requires_grad_(True)
    c = randn((B, T, G, N), 4, 0.5).requires_grad_(True)
    be, ce = (b.expand(B, T, H, N), c.expand(B, T, H, N)) if G == 1 else (b, c)
    y_ref = orc.ssd_scan_ops_default(x, a, be, ce, Q)
    dy = randn((B, T, H, P), 5)
    (y_ref * dy).sum().backward()
    scan = pm.SsdScan(x.detach().cuda(), a.detach().cuda(), b.detach().cuda(), c.detach().cuda(), Q)
    y = scan.forward()
    assert_close(y, y_ref, what="y")
    dx, da, db, dc = scan.backward(dy.cuda())
    assert_close(dx, x.grad, what="dx")
    assert_close(da, a.grad, what="da")
    assert_close(db, b.grad, what="db")
    assert_close(dc, c.grad, what="dc")


@pytest.mark.parametrize("P,N", [(16, 16), (64, 32)])   # FMA engine / tensor-core engine
def test_ssd_strong_decay_underflows_cleanly(pm, P, N):
    # A = -16, dt ~ 0.13, Q = 256: in-chunk sums reach about -530; exp must go to 0 without NaN
    B, T, H = 1, 512, 2
    x, b, c = randn((B, T, H, P), 1), randn((B, T, 1, N), 2), randn((B, T, 1, N), 3)
    a = torch.full((B, T, H), -16.0 * 0.13)
    y_ref = orc.ssd_scan_chunked(x, a, b.expand(B, T, H, N), c.expand(B, T, H, N), 256)
    scan = pm.SsdScan(x.cuda(), a.cuda(), b.cuda(), c.cuda(), 256)
    y = scan.forward()
    assert torch.isfinite(y).all()
    assert_close(y, y_ref, what="y")
    dx, da, db, dc = scan.backward(randn((B, T, H, P), 4).cuda())
    for g in (dx, da, db, dc):
        assert torch.isfinite(g).all()


def test_ssd_initial_state_and_final_state_chain(pm):
    # running two halves with the carried state equals one run over the whole sequence
    B, T, H, P, N, Q = 1, 128, 2, 8, 8, 32
    x, a = randn((B, T, H, P), 1).cuda(), (-rand((B, T, H), 2)).cuda()
    b, c = randn((B, T, 1, N), 3, 0.5).cuda(), randn((B, T, 1, N), 4, 0.5).cuda()
    y_full, fs_full = pm.SsdScan(x, a, b, c, Q).forward(want_final_state=True)
    h = T // 2
    s1 = pm.SsdScan(x[:, :h].contiguous(), a[:, :h].contiguous(), b[:, :h].contiguous(), c[:, :h].contiguous(), Q)
    y1, fs1 = s1.forward(want_final_state=True)
    s2 = pm.SsdScan(x[:, h:].contiguous(), a[:, h:].contiguous(), b[:, h:].contiguous(), c[:, h:].contiguous(), Q)
    y2, fs2 = s2.forward(init_state=fs1, want_final_state=True)
    assert_close(torch.cat([y1, y2], 1), y_full, tol=1e-5, what="y chained")
    assert_close(fs2, fs_full, tol=1e-5, what="final state")


@pytest.mark.parametrize("B,T,H,P,N,G,Q", [(2, 128, 8, 32, 16, 1, 64), (2, 256, 8, 64, 64, 1, 128)])
def test_kernels_are_deterministic(pm, B, T, H, P, N, G, Q):
    x, a = randn((B, T, H, P), 1).cuda(), (-rand((B, T, H), 2)).cuda()
    b, c, dy = randn((B, T, G, N), 3).cuda(), randn((B, T, G, N), 4).cuda(), randn((B, T, H, P), 5).cuda()
    outs = []
    for _ in range(2):
        s = pm.SsdScan(x, a, b, c, Q)
        y = s.forward()
        outs.append((y.clone(),) + tuple(t.clone() for t in s.backward(dy)))
    for u, v in zip(*outs):
        assert torch.equal(u, v)


def test_bad_arguments_raise(pm):
    x = randn((1, 100, 2, 8), 1).cuda()
    a = randn((1, 100, 2), 2).cuda()
    b = randn((1, 100, 2, 4), 3).cuda()
    with pytest.raises(pm.PmbError):
        pm.SsdScan(x, a, b[:, :, :1].contiguous().expand(1, 100, 3, 4).contiguous(), b, 50)  # G=3 with H=2
    with pytest.raises(pm.PmbError):
        pm.matmul(x.reshape(100, 16), a.reshape(100, 2))  # inner dimensions differ
    with pytest.raises(pm.PmbError):
        pm.matmul(x.reshape(100, 16).double(), x.reshape(16, 100))  # unsupported dtype is an error, never a fallback


def test_adamw_with_global_norm_clipping(pm):
    # three steps over a flat buffer against the oracle restatement of optim.rs / clip.rs
    n = 100_003
    p0 = randn((n,), 1)
    p_ref, m_ref, v_ref = [p0.clone()], [torch.zeros(n)], [torch.zeros(n)]
    p_dev = p0.clone().cuda()
    opt = pm.AdamW(p_dev, lr=3e-3, weight_decay=0.1)
    for step in range(1, 4):
        g = randn((n,), 10 + step, 2.0 if step == 2 else 0.001)     # step 2 exceeds the clip threshold, the others do not
        sumsq = opt.step(g.clone().cuda(), max_norm=1.0)
        g_ref = [g.clone()]
        norm = orc.clip_grad_norm(g_ref, 1.0)
        orc.adamw_step(p_ref, g_ref, m_ref, v_ref, step, lr=3e-3, wd=0.1)
        assert abs(float(sumsq.item()) ** 0.5 - norm) < 1e-4 * norm
        assert_close(p_dev, p_ref[0], tol=1e-5, what=f"params after step {step}")
    assert_close(opt.m, m_ref[0], what="m")       # the clip factor is formed in fp32 on the device, in fp64 by the oracle
    assert_close(opt.v, v_ref[0], what="v")
