"""GPU parity tests of the block, the checkpointed stack, the decode step and the LM step."""
import numpy as np
import pytest
import torch

from oracle import mamba2_oracle as orc
from util import GOLD, FP32_TOL, assert_close, assert_close_bf16, tol_for, block_params, cuda_params, randn, rel_err, to_pm_cfg

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pm():
    import __graft_entry__ as ge
    ge.build()
    import pm_b200
    assert torch.cuda.is_available()
    return pm_b200


def _oracle_block_grads(cfg, p, x, cot):
    pr = {k: v.clone().requires_grad_(True) for k, v in p.items()}
    xr = x.clone().requires_grad_(True)
    out = orc.block_forward(pr, cfg, xr)
    (out * cot).sum().backward()
    return out.detach(), xr.grad, {k: v.grad for k, v in pr.items()}


def test_block_single_config_matches_committed_golden(pm):
    # the reference's CPU-runnable single-block case: B=2, T=128, D=128, I=256, H=8, P=32, N=16, G=1, Q=64, K=4, fp32
    cfg = orc.Mamba2Config(d_model=128, d_state=16, d_head=32, n_heads=8, block_len=64)
    p = orc.init_block_params(cfg, seed=1)
    x, cot = randn((2, 128, 128), 11), randn((2, 128, 128), 12)
    blk = pm.Mamba2Block(to_pm_cfg(cfg), cuda_params(p))
    out = blk.forward(x.cuda())
    dx, grads = blk.backward(x.cuda(), cot.cuda())
    g = np.load(GOLD / "block_c1.npz")
    assert_close(out, g["out"], what="out")
    assert_close(dx, g["dx"], what="dx")
    for k in p:
        assert torch.isfinite(grads[k]).all() and grads[k].abs().max() > 0, k   # every parameter gets a gradient
        assert_close(grads[k].reshape(g["d_" + k].shape), g["d_" + k], tol=tol_for(k), what="d_" + k)
    assert pm.device_status() == 0


BLOCK_CASES = [  # D, N, P, H, G, K, Q, B, T
    (128, 16, 32, 8, 1, 4, 64, 2, 128),
    (64, 8, 16, 4, 4, 4, 32, 2, 64),      # per-head B/C
    (96, 12, 20, 4, 1, 3, 48, 1, 96),     # ragged dims; J=4*... keeps 16-byte rows
    (64, 8, 8, 4, 1, 4, 50, 1, 120),      # block_len does not divide T -> dense route
    (768, 64, 64, 24, 1, 4, 256, 1, 512), # production layer dims, one sequence
]


@pytest.mark.parametrize("D,N,P,H,G,K,Q,B,T", BLOCK_CASES)
def test_block_fwd_bwd_vs_oracle(pm, D, N, P, H, G, K, Q, B, T):
    cfg = orc.Mamba2Config(d_model=D, d_state=N, d_head=P, n_heads=H, n_groups=G, d_conv=K, block_len=Q)
    p = block_params(cfg, seed=3)
    x, cot = randn((B, T, D), 21), randn((B, T, D), 22)
    out_ref, dx_ref, g_ref = _oracle_block_grads(cfg, p, x, cot)
    blk = pm.Mamba2Block(to_pm_cfg(cfg), cuda_params(p))
    out = blk.forward(x.cuda())
    assert_close(out, out_ref, what="out")
    dx, grads = blk.backward(x.cuda(), cot.cuda())
    assert_close(dx, dx_ref, what="dx")
    fused = (Q % 128 == 0 and N == 64 and P == 64)       # the fused tensor-core scan takes this shape
    for k in p:
        assert_close(grads[k], g_ref[k], tol=tol_for(k, fused), what="d_" + k)
    assert pm.device_status() == 0


def test_block_residual_and_dx_accumulate(pm):
    cfg = orc.Mamba2Config(d_model=64, d_state=8, d_head=16, n_heads=4, block_len=32)
    p = block_params(cfg, seed=5)
    x, cot, acc = randn((2, 64, 64), 1), randn((2, 64, 64), 2), randn((2, 64, 64), 3)
    blk = pm.Mamba2Block(to_pm_cfg(cfg), cuda_params(p))
    xc = x.cuda()
    out = blk.forward(xc)
    out_res = blk.forward(xc, residual=xc)
    assert_close(out_res, (out + xc), tol=1e-6, what="residual")
    dx, _ = blk.backward(xc, cot.cuda())
    dx2, _ = blk.backward(xc, cot.cuda(), dx_accum=acc.cuda())
    assert_close(dx2, dx + acc.cuda(), tol=1e-6, what="dx accumulate")


def test_step_times_T_equals_forward(pm):
    # crates/pm-candle/tests/decode_state.rs:106-143 (1e-4)
    cfg = orc.Mamba2Config(d_model=64, d_state=16, d_head=16, n_heads=4, block_len=16)
    p = block_params(cfg, seed=7)
    B, T = 3, 32
    x = randn((B, T, 64), 1)
    blk = pm.Mamba2Block(to_pm_cfg(cfg), cuda_params(p))
    full = blk.forward(x.cuda())
    st = blk.zero_state(B)
    st_ref = orc.zero_state(cfg, B)
    outs = []
    for t in range(T):
        xt = x[:, t:t + 1].contiguous()
        y, st = blk.step(xt.cuda(), st)
        y_ref, st_ref = orc.block_step(p, cfg, xt, st_ref)
        outs.append(y)
        if t in (0, 5, T - 1):
            assert_close(y, y_ref, what=f"step {t}")
    assert_close(torch.cat(outs, 1), full, what="step x T vs forward")
    assert_close(st["ssm_state"], st_ref["ssm_state"], what="ssm_state")
    assert_close(st["conv_window"], st_ref["conv_window"], what="conv_window")


def _oracle_stack(cfg, layers, x, cot):
    ls = [{k: v.clone().requires_grad_(True) for k, v in p.items()} for p in layers]
    xr = x.clone().requires_grad_(True)
    h = orc.stack_forward(ls, cfg, xr)
    (h * cot).sum().backward()
    return h.detach(), xr.grad, [{k: v.grad for k, v in p.items()} for p in ls]


def test_checkpointed_stack_equals_plain_oracle_gradients(pm):
    # the re-planned policy (block inputs only) must reproduce the un-checkpointed gradients
    # (crates/pm-candle/tests/checkpoint_grad_parity.rs:99-178)
    cfg = orc.Mamba2Config(d_model=64, d_state=8, d_head=16, n_heads=4, block_len=32)
    L, B, T = 3, 2, 64
    layers = [block_params(cfg, seed=10 + i) for i in range(L)]
    x, cot = randn((B, T, 64), 1), randn((B, T, 64), 2)
    h_ref, dx_ref, g_ref = _oracle_stack(cfg, layers, x, cot)
    enc = pm.ContextEncoder(to_pm_cfg(cfg), [cuda_params(p) for p in layers])
    h, saved = enc.forward_checkpointed(x.cuda())
    assert_close(h, h_ref, what="hidden")
    seen = []
    dx, grads = enc.checkpoint_backward(saved, cot.cuda(), on_layer_done=lambda l, u: seen.append(l))
    assert seen == [2, 1, 0]
    assert_close(dx, dx_ref, what="dx")
    for l in range(L):
        for k in layers[l]:
            assert_close(grads[l][k], g_ref[l][k], tol=tol_for(k), what=f"layer {l} d_{k}")


def test_lm_step_loss_and_gradients(pm):
    cfg = orc.Mamba2Config(d_model=64, d_state=8, d_head=16, n_heads=4, block_len=32)
    L, B, T, V = 2, 2, 64, 301
    layers = [block_params(cfg, seed=20 + i) for i in range(L)]
    embed = randn((V, 64), 9, 0.5)
    ids, tg, _ = orc.lcg_batch(7, B, T, V)
    er = embed.clone().requires_grad_(True)
    ls = [{k: v.clone().requires_grad_(True) for k, v in p.items()} for p in layers]
    loss_ref = orc.lm_loss(er, ls, cfg, ids, tg)
    loss_ref.backward()
    lm = pm.FlatMamba(to_pm_cfg(cfg), L, V, B, T)
    lm.load(embed.cuda(), [cuda_params(p) for p in layers])
    loss_dev = lm.step_device(ids.cuda(), tg.cuda())
    assert abs(float(loss_dev.item()) - float(loss_ref)) < 1e-4 * abs(float(loss_ref))
    g_embed, g_layers = lm.grads()
    assert_close(g_embed, er.grad, what="d_embed")
    for l in range(L):
        for k in layers[l]:
            assert_close(g_layers[l][k], ls[l][k].grad, tol=tol_for(k), what=f"layer {l} d_{k}")
    # the host-buffer entry point gives the same loss, twice in a row
    ih, th = ids.pin_memory(), tg.pin_memory()
    l1 = lm.step_host(ih, th)
    l2 = lm.step_host(ih, th)
    assert l1 == l2 and abs(l1 - float(loss_ref)) < 1e-4 * abs(float(loss_ref))
    bad = ids.clone(); bad[0, 0] = V + 5
    with pytest.raises(pm.PmbError):
        lm.step_host(bad.pin_memory(), th)
    lm.close()


def test_lm_step_captured_in_a_cuda_graph_equals_eager(pm):
    cfg = orc.Mamba2Config(d_model=64, d_state=8, d_head=16, n_heads=4, block_len=32)
    L, B, T, V = 3, 2, 64, 301
    layers = [block_params(cfg, seed=50 + i) for i in range(L)]
    lm = pm.FlatMamba(to_pm_cfg(cfg), L, V, B, T)
    lm.load(randn((V, 64), 12, 0.5).cuda(), [cuda_params(p) for p in layers])
    seen = []
    step = lm.capture_step(on_layer_done=lambda l, u: seen.append(l))
    assert seen[-(L + 1):] == [2, 1, 0, -1] and step.launches_per_step > 0
    for seed in (5, 6):
        ids, tg, _ = orc.lcg_batch(seed, B, T, V)
        loss_e = float(lm.step_device(ids.cuda(), tg.cuda()).item())
        ge, gl = lm.grads()
        ge, gl = ge.clone(), [{k: v.clone() for k, v in g.items()} for g in gl]
        loss_g = float(step(ids.pin_memory(), tg.pin_memory()).item())      # host tensors: copied into the static buffers
        assert loss_g == loss_e
        ge2, gl2 = lm.grads()
        assert_close(ge2, ge, tol=1e-6, what="d_embed")     # the embedding scatter adds with atomics: order, not value, may differ
        for a, b in zip(gl, gl2):
            for k in a:
                assert torch.equal(a[k], b[k]), k
    assert pm.device_status() == 0
    lm.close()


def test_lm_checkpoint_round_trip_in_reference_format(pm, tmp_path):
    """save -> the safetensors package reads p_0000.. with the append_params shapes; a second model loads the file
    and computes the same loss; a model of another shape refuses it (pm-train/src/checkpoint.rs:25-97)."""
    sf = pytest.importorskip("safetensors.numpy")
    cfg = orc.Mamba2Config(d_model=64, d_state=8, d_head=16, n_heads=4, block_len=32)
    L, B, T, V = 2, 2, 64, 301
    layers = [block_params(cfg, seed=40 + i) for i in range(L)]
    embed = randn((V, 64), 11, 0.5)
    ids, tg, _ = orc.lcg_batch(3, B, T, V)
    lm = pm.FlatMamba(to_pm_cfg(cfg), L, V, B, T)
    lm.load(embed.cuda(), [cuda_params(p) for p in layers])
    loss0 = float(lm.step_device(ids.cuda(), tg.cuda()).item())
    path = tmp_path / "model.safetensors"
    lm.save_checkpoint(path)
    got = sf.load_file(str(path))
    order = ["in_proj_weight", "conv1d_weight", "conv1d_bias", "a_log", "d_skip", "dt_bias", "norm_weight", "out_proj_weight"]
    assert len(got) == 1 + 8 * L
    assert np.array_equal(got["p_0000"], embed.numpy())
    for l in range(L):
        for j, k in enumerate(order):
            t = got[f"p_{1 + 8 * l + j:04d}"]
            ref = layers[l][k].numpy()
            assert t.shape == (ref.shape if k != "conv1d_weight" else (cfg.xbc_dim, 1, cfg.d_conv))
            assert np.array_equal(t.reshape(ref.shape), ref), k
    lm2 = pm.FlatMamba(to_pm_cfg(cfg), L, V, B, T)
    lm2.load_checkpoint(path)
    assert float(lm2.step_device(ids.cuda(), tg.cuda()).item()) == loss0
    lm3 = pm.FlatMamba(to_pm_cfg(cfg), L + 1, V, B, T)
    with pytest.raises(pm.PmbError, match="tensors, model has"):
        lm3.load_checkpoint(path)
    for m in (lm, lm2, lm3):
        m.close()


@pytest.mark.parametrize("dtype,tol", [(torch.float32, None), (torch.bfloat16, 2e-2)])
def test_two_level_lm_config3_wiring(pm, dtype, tol):
    # the two-level benchmark model's wiring at small dims: 2 + 2 layers, pool 4, one-group causal shift
    cfg = orc.Mamba2Config(d_model=64, d_state=8, d_head=8, n_heads=8, block_len=16)
    L0, L1, B, T, V, g = 2, 2, 2, 64, 301, 4
    layers = [block_params(cfg, seed=30 + i) for i in range(L0 + L1)]
    embed, wproj = randn((V, 64), 9, 0.5), randn((64, 64), 10, 0.125)
    ids, tg, _ = orc.lcg_batch(11, B, T, V)
    er, wr = embed.clone().requires_grad_(True), wproj.clone().requires_grad_(True)
    ls = [{k: v.clone().requires_grad_(True) for k, v in p.items()} for p in layers]
    loss_ref = orc.hier_lm_loss(er, wr, ls[:L0], ls[L0:], cfg, ids, tg, group=g)
    loss_ref.backward()
    l16 = None
    if tol:      # the oracle with bf16 storage: how far two correct bf16 evaluations of this model are apart
        e16, w16 = embed.clone().requires_grad_(True), wproj.clone().requires_grad_(True)
        l16 = [{k: v.clone().requires_grad_(True) for k, v in p.items()} for p in layers]
        orc.hier_lm_loss(e16, w16, l16[:L0], l16[L0:], cfg, ids, tg, group=g, cdt=torch.bfloat16).backward()
    lm = pm.FlatMamba(to_pm_cfg(cfg), L0, V, B, T, compute_dtype=dtype, level1_layers=L1, group=g)
    lm.load(embed.cuda(), [cuda_params(p) for p in layers], wproj=wproj.cuda())
    seen = []
    loss = lm.step_host(ids.pin_memory(), tg.pin_memory(), on_layer_done=lambda l, u: seen.append(l))
    assert seen == [3, 2, 1, 0, -1]          # level 1 first (last to first), then level 0, then the embedding
    rel = tol or 1e-4
    assert abs(loss - float(loss_ref)) < rel * abs(float(loss_ref))
    g_embed, g_layers = lm.grads()
    assert_close(g_embed, er.grad, tol=rel, what="d_embed")
    assert_close(lm.view(lm.flat_grads, -2), wr.grad, tol=rel, what="d_wproj")
    for l in range(L0 + L1):
        for k in layers[l]:
            # bf16 storage: 2e-2 on every gradient, or twice the distance between the oracle's own bf16 and fp32 runs
            # where that is larger at these tiny widths (the reference's own bf16 gradient tolerance is 5e-2,
            # crates/pm-candle/tests/bf16_mixed_precision_cuda.rs:72)
            if tol: assert_close_bf16(g_layers[l][k], ls[l][k].grad, l16[l][k].grad, what=f"layer {l} d_{k}", tol=tol)
            else: assert_close(g_layers[l][k], ls[l][k].grad, tol=tol_for(k), what=f"layer {l} d_{k}")
    lm.close()
