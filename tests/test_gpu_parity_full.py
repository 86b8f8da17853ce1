"""GPU parity at the sizes and on the branches the benchmark runs: the headline LM configuration end to end, the
LM head across several row tiles, the decode step at the scan-microbenchmark dims, the strong-decay backward,
two models with different vocabularies in one process, and the bounded-wait status path."""
import os

import pytest
import torch

from oracle import mamba2_oracle as orc
from util import DEPTH24_TOL, FP32_TOL, assert_close, block_params, cuda_params, rand, randn, rel_err, report, to_pm_cfg, tol_for

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pm():
    import __graft_entry__ as ge
    ge.build()
    import pm_b200
    assert torch.cuda.is_available()
    return pm_b200


def _oracle_lm(cfg, embed, layers, ids, tg, dtype=torch.float32):
    er = embed.to(dtype).clone().requires_grad_(True)
    ls = [{k: v.to(dtype).clone().requires_grad_(True) for k, v in p.items()} for p in layers]
    loss = orc.lm_loss(er, ls, cfg, ids, tg)
    loss.backward()
    return float(loss), er.grad, [{k: v.grad for k, v in p.items()} for p in ls]


def test_headline_config_lm_step_vs_oracle(pm):
    """24 layers, d_model 768, 24 heads x 64, d_state 64, chunk 256, vocab 50257 (tied), batch 4 x 512, fp32: loss and
    every gradient of one step against the oracle (crates/pm-candle/tests/checkpoint_grad_parity.rs:99-178 is the
    reference's test of the same property at small dims)."""
    L, D, P, H, N, Q, V, B, T = 24, 768, 64, 24, 64, 256, 50257, 4, 512
    cfg = orc.Mamba2Config(d_model=D, d_state=N, d_head=P, n_heads=H, block_len=Q)
    layers = [orc.init_block_params(cfg, seed=100 + i) for i in range(L)]
    g = torch.Generator(); g.manual_seed(5)
    embed = torch.randn(V, D, generator=g) * 0.02
    ids = torch.randint(0, V, (B, T), generator=g, dtype=torch.int64)
    tg = torch.roll(ids, -1, dims=1).contiguous()
    torch.set_num_threads(os.cpu_count() or 1)
    loss_ref, ge_ref, gl_ref = _oracle_lm(cfg, embed, layers, ids, tg)
    lm = pm.FlatMamba(to_pm_cfg(cfg), L, V, B, T)
    lm.load(embed.cuda(), [cuda_params(p) for p in layers])
    loss = lm.step_host(ids.pin_memory(), tg.pin_memory())
    assert abs(loss - loss_ref) < 1e-4 * abs(loss_ref), (loss, loss_ref)
    ge, gl = lm.grads()
    failures = []

    def check(what, ours, ref, tol):
        try:
            return report("headline_lm", what, ours, ref, tol=tol, elem_tol=1e3 * tol)[0]   # element-wise floor is 1e-3 of the max
        except AssertionError as e:          # collect everything before failing: the report should hold every tensor
            failures.append(str(e))
            return rel_err(ours, ref)

    worst = {"embed": check("d_embed", ge, ge_ref, DEPTH24_TOL)}
    for l in range(L):
        for k in layers[l]:
            worst[k] = max(worst.get(k, 0.0), check(f"layer{l:02d}.d_{k}", gl[l][k], gl_ref[l][k], DEPTH24_TOL))
            assert torch.isfinite(gl[l][k]).all() and gl[l][k].abs().max() > 0, (l, k)
    print("headline LM: worst max-norm error per parameter kind", {k: f"{v:.2e}" for k, v in worst.items()})
    assert pm.device_status() == 0 and lm.bad_tokens() == 0
    lm.close()
    assert not failures, failures


@pytest.mark.parametrize("dtype,tol", [(torch.float32, None), (torch.bfloat16, 2e-2)])
def test_lm_head_across_row_tiles_with_remainder(pm, dtype, tol):
    """4608 tokens = four full row tiles of 1024 and a remainder of 512: the logits tile loop, the accumulation of the
    embedding-table gradient across tiles and the per-tile d(hidden) (crates/pm-core/src/loss.rs:73-209 tiles the
    same way)."""
    cfg = orc.Mamba2Config(d_model=64, d_state=8, d_head=8, n_heads=8, block_len=32)    # in_proj_dim 152: a multiple of 8 (bf16 rule)
    L, B, T, V = 2, 9, 512, 301
    layers = [block_params(cfg, seed=60 + i) for i in range(L)]
    embed = randn((V, 64), 13, 0.5)
    ids, tg, _ = orc.lcg_batch(17, B, T, V)
    loss_ref, ge_ref, gl_ref = _oracle_lm(cfg, embed, layers, ids, tg)
    lm = pm.FlatMamba(to_pm_cfg(cfg), L, V, B, T, compute_dtype=dtype)
    lm.load(embed.cuda(), [cuda_params(p) for p in layers])
    loss = float(lm.step_device(ids.cuda(), tg.cuda()).item())
    rel = tol or 1e-4
    assert abs(loss - loss_ref) < rel * abs(loss_ref)
    ge, gl = lm.grads()
    assert_close(ge, ge_ref, tol=rel, what="d_embed")
    for l in range(L):
        for k in layers[l]:
            assert_close(gl[l][k], gl_ref[l][k], tol=tol or tol_for(k), what=f"layer {l} d_{k}")
    lm.close()


def test_lm_head_small_tiles_equal_one_tile(pm, monkeypatch):
    """The same model with the row tile forced down to 128 rows (many tiles) gives the loss and gradients of the
    single-tile run."""
    cfg = orc.Mamba2Config(d_model=64, d_state=8, d_head=16, n_heads=4, block_len=32)
    L, B, T, V = 2, 4, 96, 301
    layers = [block_params(cfg, seed=70 + i) for i in range(L)]
    embed = randn((V, 64), 14, 0.5)
    ids, tg, _ = orc.lcg_batch(19, B, T, V)
    outs = []
    for rows in (None, "128"):
        if rows:
            monkeypatch.setenv("PMB_LM_TILE_ROWS", rows)
        lm = pm.FlatMamba(to_pm_cfg(cfg), L, V, B, T)
        lm.load(embed.cuda(), [cuda_params(p) for p in layers])
        loss = float(lm.step_device(ids.cuda(), tg.cuda()).item())
        outs.append((loss, lm.flat_grads.clone()))
        lm.close()
    assert abs(outs[0][0] - outs[1][0]) < 1e-6 * abs(outs[0][0])
    assert_close(outs[1][1], outs[0][1], tol=1e-5, what="flat gradients, 128-row tiles vs one tile")


def test_decode_step_at_scan_microbench_dims(pm):
    """One-token recurrence at 32 heads x 64, d_state 128, d_model 2048 (the dims the decode benchmark times) against
    the oracle's step, three tokens in a row (crates/pm-candle/tests/decode_state.rs:106-143)."""
    cfg = orc.Mamba2Config(d_model=2048, d_state=128, d_head=64, n_heads=32, block_len=256)
    p = block_params(cfg, seed=9)
    B = 3
    blk = pm.Mamba2Block(to_pm_cfg(cfg), cuda_params(p))
    st, st_ref = blk.zero_state(B), orc.zero_state(cfg, B)
    st["ssm_state"].copy_(randn(tuple(st["ssm_state"].shape), 2)); st_ref["ssm_state"] = st["ssm_state"].cpu().clone()
    for t in range(3):
        xt = randn((B, 1, 2048), 30 + t)
        y, st = blk.step(xt.cuda(), st)
        y_ref, st_ref = orc.block_step(p, cfg, xt, st_ref)
        report("decode_c5_dims", f"y[{t}]", y, y_ref)
    report("decode_c5_dims", "ssm_state", st["ssm_state"], st_ref["ssm_state"])
    report("decode_c5_dims", "conv_window", st["conv_window"], st_ref["conv_window"])
    assert pm.device_status() == 0


@pytest.mark.parametrize("P,N", [(16, 16), (64, 32), (64, 64)])   # FMA engine / tensor-core engines (3xTF32, fused pairs)
def test_ssd_strong_decay_backward_vs_oracle(pm, P, N):
    """A = -16, dt ~ 0.13, chunk 256 (in-chunk sums near -530): the backward is compared with the oracle's autograd,
    not only checked for finiteness."""
    B, T, H = 1, 512, 2
    x = randn((B, T, H, P), 1).requires_grad_(True)
    b = randn((B, T, 1, N), 2).requires_grad_(True)
    c = randn((B, T, 1, N), 3).requires_grad_(True)
    a = torch.full((B, T, H), -16.0 * 0.13).requires_grad_(True)
    y_ref = orc.ssd_scan_chunked(x, a, b.expand(B, T, H, N), c.expand(B, T, H, N), 256)
    dy = randn((B, T, H, P), 4)
    (y_ref * dy).sum().backward()
    scan = pm.SsdScan(x.detach().cuda(), a.detach().cuda(), b.detach().cuda(), c.detach().cuda(), 256)
    y = scan.forward()
    assert_close(y, y_ref, what="y")
    dx, da, db, dc = scan.backward(dy.cuda())
    for got, ref, name in ((dx, x.grad, "dx"), (da, a.grad, "da"), (db, b.grad, "db"), (dc, c.grad, "dc")):
        assert torch.isfinite(got).all(), name
        report(f"ssd_strong_decay_P{P}", name, got, ref)


def test_two_models_with_different_vocabularies(pm):
    """A second handle with a smaller vocabulary must not disturb the first one's next step (the cross-entropy
    kernel's shared-memory limit is a property of the kernel, not of a handle)."""
    cfg = orc.Mamba2Config(d_model=64, d_state=8, d_head=16, n_heads=4, block_len=32)
    L, B, T = 1, 2, 64
    layers = [block_params(cfg, seed=80)]
    big, small = 4001, 257
    lm_big = pm.FlatMamba(to_pm_cfg(cfg), L, big, B, T)
    lm_big.load(randn((big, 64), 15, 0.5).cuda(), [cuda_params(p) for p in layers])
    ids, tg, _ = orc.lcg_batch(23, B, T, big)
    l0 = float(lm_big.step_device(ids.cuda(), tg.cuda()).item())
    lm_small = pm.FlatMamba(to_pm_cfg(cfg), L, small, B, T)
    lm_small.load(randn((small, 64), 16, 0.5).cuda(), [cuda_params(p) for p in layers])
    ids_s, tg_s, _ = orc.lcg_batch(29, B, T, small)
    assert torch.isfinite(lm_small.step_device(ids_s.cuda(), tg_s.cuda())).all()
    l1 = float(lm_big.step_device(ids.cuda(), tg.cuda()).item())
    torch.cuda.synchronize()
    assert l1 == l0
    lm_big.close(); lm_small.close()


def test_out_of_range_target_is_flagged(pm):
    cfg = orc.Mamba2Config(d_model=64, d_state=8, d_head=16, n_heads=4, block_len=32)
    L, B, T, V = 1, 2, 64, 301
    lm = pm.FlatMamba(to_pm_cfg(cfg), L, V, B, T)
    lm.load(randn((V, 64), 15, 0.5).cuda(), [cuda_params(block_params(cfg, seed=81))])
    ids, tg, _ = orc.lcg_batch(31, B, T, V)
    lm.step_device(ids.cuda(), tg.cuda())
    assert lm.bad_tokens() == 0
    bad_t = tg.clone(); bad_t[1, 3] = V
    lm.step_device(ids.cuda(), bad_t.cuda())
    assert lm.bad_tokens() == 2 and lm.bad_tokens() == 0        # read-and-clear
    bad_i = ids.clone(); bad_i[0, 0] = -1
    lm.step_device(bad_i.cuda(), bad_t.cuda())
    assert lm.bad_tokens() == 3
    with pytest.raises(pm.PmbError, match="target"):
        lm.step_host(ids.pin_memory(), bad_t.pin_memory())
    lm.close()


def test_bounded_wait_gives_up_and_reports(pm):
    """A wait on a barrier that nothing arms runs out after its poll limit: the kernel returns, the status word says
    so, and the next library call on the same context is clean.  (Nothing here faults, traps or waits unboundedly.)"""
    assert pm.device_status() == 0
    pm.selftest_bounded_wait(2048)
    torch.cuda.synchronize()
    assert pm.device_status() == 0x8000          # bit 7 of the scan kernels' byte of the status word
    assert pm.device_status() == 0               # read-and-clear
    a, b = randn((128, 64), 1).cuda(), randn((64, 128), 2).cuda()
    out = pm.matmul(a, b)
    assert rel_err(out, a.cpu().double() @ b.cpu().double()) < 3e-5 and pm.device_status() == 0
