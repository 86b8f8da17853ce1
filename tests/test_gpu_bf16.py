"""bf16-storage configurations: bf16 GEMM and the bf16 block against the oracle (bound 2e-2, as stated for
bf16 storage; the reference's own bf16 tests hold 1e-2 forward / 5e-2 gradients,
crates/pm-candle/tests/bf16_mixed_precision_cuda.rs:58,72)."""
import pytest
import torch

from oracle import mamba2_oracle as orc
from util import assert_close, assert_close_bf16, block_params, cuda_params, randn, rel_err, to_pm_cfg

pytestmark = pytest.mark.gpu
BF16_TOL = 2e-2


@pytest.fixture(scope="module")
def pm():
    import __graft_entry__ as ge
    ge.build()
    import pm_b200
    assert torch.cuda.is_available()
    return pm_b200


# the last shape has 17 x 18 = 306 tiles of 256x256: the launcher takes the CTA-pair kernel (cta_group::2) for it
@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (304, 200, 104), (128, 552, 128), (64, 40, 72), (8, 8, 8), (2048, 768, 1536),
                                   (4344, 4600, 136)])
@pytest.mark.parametrize("ta,tb", [(0, 1), (0, 0), (1, 0), (1, 1)])
def test_gemm_bf16(pm, M, N, K, ta, tb):
    a = randn((K, M) if ta else (M, K), 1).bfloat16()
    b = randn((N, K) if tb else (K, N), 2).bfloat16()
    ref = (a.T if ta else a).double() @ (b.T if tb else b).double()
    out = pm.matmul_bf16(a.cuda(), b.cuda(), trans_a=bool(ta), trans_b=bool(tb))
    assert rel_err(out, ref) < 1e-5          # products of bf16 values are exact in fp32; only the summation order differs
    r = randn((M, N), 3).bfloat16()
    out16 = pm.matmul_bf16(a.cuda(), b.cuda(), trans_a=bool(ta), trans_b=bool(tb), residual=r.cuda(), out_dtype=torch.bfloat16)
    assert rel_err(out16.float(), ref + r.double()) < 6e-3   # one bf16 rounding of the result
    assert pm.device_status() == 0


def test_cast_matches_torch(pm):
    x = randn((1000, 37), 5)
    assert torch.equal(pm.to_bf16(x.cuda()).cpu(), x.bfloat16())


def _oracle_block_grads(cfg, p, x, cot):
    pr = {k: v.clone().requires_grad_(True) for k, v in p.items()}
    xr = x.clone().requires_grad_(True)
    out = orc.block_forward(pr, cfg, xr)
    (out.float() * cot.float()).sum().backward()
    return out.detach().float(), xr.grad.float(), {k: v.grad for k, v in pr.items()}


# the last case has 4096 tokens (long K for the two weight-gradient products)
@pytest.mark.parametrize("D,N,P,H,Q,B,T", [(128, 16, 32, 8, 64, 2, 128), (768, 64, 64, 24, 256, 1, 512), (128, 16, 32, 8, 64, 4, 1024)])
def test_block_bf16_storage_vs_oracle(pm, D, N, P, H, Q, B, T):
    cfg = orc.Mamba2Config(d_model=D, d_state=N, d_head=P, n_heads=H, block_len=Q)
    p = block_params(cfg, seed=3)
    x, cot = randn((B, T, D), 21).bfloat16(), randn((B, T, D), 22).bfloat16()
    # reference 1: the oracle run in the bf16 compute dtype (bf16 matmuls and roundings, fp32 islands)
    out16, dx16, g16 = _oracle_block_grads(cfg, p, x, cot)
    # reference 2: the fp32 oracle on the same (bf16-representable) inputs
    out32, dx32, g32 = _oracle_block_grads(cfg, p, x.float(), cot.float())
    blk = pm.Mamba2Block(to_pm_cfg(cfg), cuda_params(p), compute_dtype=torch.bfloat16)
    out = blk.forward(x.cuda())
    dx, grads = blk.backward(x.cuda(), cot.cuda())
    assert out.dtype == torch.bfloat16 and dx.dtype == torch.bfloat16
    for ref_out, ref_dx, ref_g, what in ((out16, dx16, g16, "bf16 oracle"), (out32, dx32, g32, "fp32 oracle")):
        assert_close(out.float(), ref_out, tol=BF16_TOL, what=f"out vs {what}")
        assert_close(dx.float(), ref_dx, tol=BF16_TOL, what=f"dx vs {what}")
        for k in p:
            assert_close(grads[k], ref_g[k], tol=BF16_TOL, what=f"d_{k} vs {what}")
    assert pm.device_status() == 0
    # residual and accumulation forms
    out_r = blk.forward(x.cuda(), residual=x.cuda())
    assert_close(out_r.float(), (out.float() + x.cuda().float()), tol=1e-2, what="residual")


def test_lm_step_bf16_storage(pm):
    # flat LM with bf16 activations / GEMM operands: loss and every gradient against the fp32 oracle
    cfg = orc.Mamba2Config(d_model=64, d_state=8, d_head=8, n_heads=8, block_len=32)   # in_proj_dim 152: a multiple of 8
    L, B, T, V = 2, 2, 64, 301
    layers = [block_params(cfg, seed=20 + i) for i in range(L)]
    embed = randn((V, 64), 9, 0.5)
    ids, tg, _ = orc.lcg_batch(7, B, T, V)
    er = embed.clone().requires_grad_(True)
    ls = [{k: v.clone().requires_grad_(True) for k, v in p.items()} for p in layers]
    loss_ref = orc.lm_loss(er, ls, cfg, ids, tg)
    loss_ref.backward()
    # the same model evaluated by the oracle with bf16 storage: how far two correct bf16 evaluations are apart
    e16 = embed.clone().requires_grad_(True)
    l16 = [{k: v.clone().requires_grad_(True) for k, v in p.items()} for p in layers]
    orc.lm_loss(e16, l16, cfg, ids, tg, cdt=torch.bfloat16).backward()
    lm = pm.FlatMamba(to_pm_cfg(cfg), L, V, B, T, compute_dtype=torch.bfloat16)
    lm.load(embed.cuda(), [cuda_params(p) for p in layers])
    loss = lm.step_host(ids.pin_memory(), tg.pin_memory())
    assert abs(loss - float(loss_ref)) < BF16_TOL * abs(float(loss_ref))
    g_embed, g_layers = lm.grads()
    assert_close(g_embed, er.grad, tol=BF16_TOL, what="d_embed")
    for l in range(L):
        for k in layers[l]:
            assert_close_bf16(g_layers[l][k], ls[l][k].grad, l16[l][k].grad, what=f"layer {l} d_{k}", tol=BF16_TOL)
    assert pm.device_status() == 0
    lm.close()


# the first four shapes take the native bf16 scan (plain bf16 tensor-core operands: d_head 64, d_state 64 / 128, block_len
# a multiple of 128, grouped or per-head B / C), the last one the widen -> fp32 scan -> cast route
@pytest.mark.parametrize("B,T,H,P,N,G,Q", [(1, 512, 4, 64, 128, 1, 256), (2, 512, 8, 64, 64, 1, 128), (1, 768, 4, 64, 128, 4, 256),
                                           (3, 384, 2, 64, 64, 1, 384), (2, 128, 4, 16, 8, 4, 32)])
def test_ssd_scan_bf16_inputs_fp32_state(pm, B, T, H, P, N, G, Q):
    # the scan microbenchmark's dims at reduced batch/heads: bf16 x, B, C; dt = softplus(N(-2, 0.5)); A = -exp(U[log 1, log 16])
    x = randn((B, T, H, P), 1).bfloat16(); b = randn((B, T, G, N), 2).bfloat16(); c = randn((B, T, G, N), 3).bfloat16()
    dt = torch.nn.functional.softplus(randn((B, T, H), 4, 0.5) - 2.0)
    A = -torch.exp(torch.rand(H, generator=torch.Generator().manual_seed(5)) * 2.7726)
    a = (dt * A).contiguous()
    xr, ar = x.float().requires_grad_(True), a.clone().requires_grad_(True)
    br, cr = b.float().requires_grad_(True), c.float().requires_grad_(True)
    be, ce = (br.expand(B, T, H, N), cr.expand(B, T, H, N)) if G == 1 else (br, cr)
    y_ref = orc.ssd_scan_ops_default(xr, ar, be, ce, Q)
    dy = randn((B, T, H, P), 6).bfloat16()
    (y_ref * dy.float()).sum().backward()
    scan = pm.SsdScanBf16(x.cuda(), a.cuda(), b.cuda(), c.cuda(), Q)
    y, fs = scan.forward(want_final_state=True)
    assert y.dtype == torch.bfloat16 and fs.dtype == torch.float32
    assert_close(y.float(), y_ref, tol=BF16_TOL, what="y")
    dx, da, db, dc = scan.backward(dy.cuda())
    assert_close(dx.float(), xr.grad, tol=BF16_TOL, what="dx")
    assert_close(da, ar.grad, tol=BF16_TOL, what="da")
    assert_close(db.float(), br.grad, tol=BF16_TOL, what="db")
    assert_close(dc.float(), cr.grad, tol=BF16_TOL, what="dc")
    # final state, and a second segment that starts from it: against the fp32 scan on the same (bf16-rounded) values
    ref = pm.SsdScan(x.float().cuda(), a.cuda(), b.float().cuda(), c.float().cuda(), Q)
    _, fs_ref = ref.forward(want_final_state=True)
    assert_close(fs, fs_ref, tol=BF16_TOL, what="final state")
    y2_ref, fs2_ref = ref.forward(init_state=fs_ref, want_final_state=True)
    y2, fs2 = scan.forward(init_state=fs_ref, want_final_state=True)
    assert_close(y2.float(), y2_ref, tol=BF16_TOL, what="y from a carried state")
    assert_close(fs2, fs2_ref, tol=BF16_TOL, what="final state from a carried state")
    assert pm.device_status() == 0
