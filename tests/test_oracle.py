"""Pins the CPU oracle: reference golden fixture, known answers, structural invariants."""
import pathlib

import numpy as np
import pytest
import torch

from oracle import mamba2_oracle as orc

GOLD = pathlib.Path(__file__).resolve().parent / "golden"


def _rand(shape, seed, scale=1.0, dtype=torch.float32):
    g = torch.Generator(); g.manual_seed(seed)
    return torch.randn(shape, generator=g, dtype=dtype) * scale


def test_fixture_ssd_q64_all_three_algorithms():
    # reference/fixtures/ssd_q64 (crates/pm-core/tests/ssd_fixture.rs:29-77 holds 5e-3; we hold 5e-5 at max|Y|=5.9)
    f = np.load(GOLD / "ssd_q64.npz")
    X, A, B, C = (torch.from_numpy(f[k]) for k in "XABC")
    Y = f["Y"]
    y_dense = orc.ssd_scan_dense(X, A, B, C).numpy()
    y_chunk, fs = orc.ssd_scan_chunked(X, A, B, C, 64, return_final_state=True)
    y_scalar = orc.ssd_scan_naive_scalar(f["X"], f["A"], f["B"], f["C"])
    assert np.abs(y_dense - Y).max() < 5e-5
    assert np.abs(y_chunk.numpy() - Y).max() < 5e-5
    assert np.abs(y_scalar - Y).max() < 5e-5
    # the reference's Python state is (b,h,p,n); the Rust/Candle layout is (B,H,N,P)
    assert np.abs(fs.numpy().transpose(0, 1, 3, 2) - f["final_state"]).max() < 1e-5


def test_zero_a_collapses_to_running_sum():
    # crates/pm-core/src/mamba2/ssd.rs:105-120, crates/pm-candle/src/ops_impl.rs:574-593
    b, t, h, p, n = 1, 4, 1, 2, 2
    x = torch.ones(b, t, h, p)
    a = torch.zeros(b, t, h)
    bb = (torch.arange(b * t * h * n, dtype=torch.float32) * 0.1).reshape(b, t, h, n)
    y = orc.ssd_scan_ops_default(x, a, bb, bb.clone(), 4)
    v = y.reshape(-1)
    assert abs(float(v[0] - v[1])) < 1e-6 and float(v[6]) > float(v[0])
    expect = torch.tril(bb[0, :, 0] @ bb[0, :, 0].T).sum(-1)
    assert torch.allclose(y[0, :, 0, 0], expect, atol=1e-6)


def test_elementwise_known_answers():
    # crates/pm-candle/src/ops_impl.rs:491-547
    assert torch.allclose(orc.silu(torch.tensor([0.0, 1.0, -1.0, 2.0])),
                          torch.tensor([0.0, 0.7310586, -0.2689414, 1.7615942]), atol=1e-5)
    assert torch.allclose(orc.softplus(torch.tensor([0.0, 1.0, -1.0, 10.0])),
                          torch.tensor([0.6931472, 1.3132617, 0.3132617, 10.000046]), atol=1e-4)
    x = torch.tensor([[1.0, 2.0, 3.0, 4.0]])
    assert torch.allclose(orc.rmsnorm(x, torch.ones(4), 1e-6), x / 7.5 ** 0.5, atol=1e-5)


def test_config_shapes_consistent():
    # crates/pm-candle/tests/mamba2_block.rs:70-87
    cfg = orc.Mamba2Config(d_model=768, d_state=128, d_head=64, n_heads=12)
    assert cfg.d_inner == 768 and cfg.xbc_dim == 1024 and cfg.in_proj_dim == 1804


@pytest.mark.parametrize("G", [1, 4])
def test_dense_chunked_scalar_agree(G):
    Bn, T, H, P, N = 2, 64, 4, 8, 8
    x = _rand((Bn, T, H, P), 1); a = -torch.rand(Bn, T, H, generator=torch.Generator().manual_seed(2))
    b = _rand((Bn, T, G, N), 3, 0.5).expand(Bn, T, H, N) if G == 1 else _rand((Bn, T, H, N), 3, 0.5)
    c = _rand((Bn, T, H, N), 4, 0.5)
    yd = orc.ssd_scan_dense(x, a, b, c)
    yc = orc.ssd_scan_chunked(x, a, b, c, 16)
    ys = torch.from_numpy(orc.ssd_scan_naive_scalar(x.numpy(), a.numpy(), b.contiguous().numpy(), c.numpy()))
    assert (yd - yc).abs().max() < 2e-5 and (yd - ys).abs().max() < 2e-5


def _c1():
    cfg = orc.Mamba2Config(d_model=128, d_state=16, d_head=32, n_heads=8, block_len=64)
    p = orc.init_block_params(cfg, seed=1)
    return cfg, p


def test_block_c1_matches_committed_golden_and_all_params_get_grad():
    # every parameter must receive a finite non-zero gradient
    # (crates/pm-candle/tests/rmsnorm_backward.rs:86-127)
    cfg, p = _c1()
    for v in p.values():
        v.requires_grad_(True)
    x = _rand((2, 128, 128), 11).requires_grad_(True)
    cot = _rand((2, 128, 128), 12)
    out = orc.block_forward(p, cfg, x)
    (out * cot).sum().backward()
    g = np.load(GOLD / "block_c1.npz")
    assert np.abs(out.detach().numpy() - g["out"]).max() < 1e-5
    assert np.abs(x.grad.numpy() - g["dx"]).max() < 1e-4
    for k, v in p.items():
        assert torch.isfinite(v.grad).all() and v.grad.abs().max() > 0, k
        ref = g["d_" + k]
        assert np.abs(v.grad.numpy() - ref).max() <= 1e-4 * max(1.0, np.abs(ref).max()), k


def test_fp32_oracle_error_bounded_by_fp64_run():
    cfg, p = _c1()
    x = _rand((2, 128, 128), 11)
    o32 = orc.block_forward(p, cfg, x)
    p64 = {k: v.double() for k, v in p.items()}
    o64 = orc.block_forward(p64, cfg, x.double())
    assert (o32.double() - o64).abs().max() / o64.abs().max() < 2e-6


def test_step_times_T_equals_forward():
    # crates/pm-candle/tests/decode_state.rs:106-143 (1e-4)
    cfg = orc.Mamba2Config(d_model=32, d_state=8, d_head=8, n_heads=4, block_len=8)
    p = orc.init_block_params(cfg, seed=3)
    x = _rand((2, 16, 32), 5)
    full = orc.block_forward(p, cfg, x)
    st = orc.zero_state(cfg, 2)
    outs = []
    for t in range(16):
        y, st = orc.block_step(p, cfg, x[:, t : t + 1], st)
        outs.append(y)
    assert (torch.cat(outs, 1) - full).abs().max() < 1e-4


def test_checkpointed_grads_equal_plain_grads():
    # crates/pm-candle/tests/checkpoint_grad_parity.rs:99-178 (1e-5)
    cfg = orc.Mamba2Config(d_model=32, d_state=8, d_head=8, n_heads=4, block_len=8)
    V, L = 50, 3
    ids, tg, _ = orc.lcg_batch(7, 2, 16, V)

    def run(ckpt):
        emb = (_rand((V, 32), 1, 0.02)).requires_grad_(True)
        layers = [orc.init_block_params(cfg, seed=10 + i) for i in range(L)]
        for lp in layers:
            for v in lp.values():
                v.requires_grad_(True)
        loss = orc.lm_loss(emb, layers, cfg, ids, tg, checkpointed=ckpt)
        if not ckpt:
            loss.backward()
        return float(loss), [emb.grad] + [v.grad for lp in layers for v in lp.values()]

    l0, g0 = run(False)
    l1, g1 = run(True)
    assert abs(l0 - l1) < 1e-6
    for a, b in zip(g0, g1):
        assert (a - b).abs().max() < 1e-5


def test_lcg_batch_targets_are_rotated_ids():
    ids, tg, _ = orc.lcg_batch(1, 2, 8, 100)
    assert ids.min() >= 0 and ids.max() < 100
    assert torch.equal(tg[:, :-1], ids[:, 1:]) and torch.equal(tg[:, -1], ids[:, 0])


def test_adamw_restatement_matches_torch_adamw():
    # the reference's AdamW (pm-train/src/optim.rs:104-157) is the textbook decoupled-decay form
    p0 = _rand((1000,), 1)
    p_ref = torch.nn.Parameter(p0.clone())
    opt = torch.optim.AdamW([p_ref], lr=3e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.1)
    p, m, v = [p0.clone()], [torch.zeros(1000)], [torch.zeros(1000)]
    for step in range(1, 4):
        g = _rand((1000,), 10 + step)
        p_ref.grad = g.clone()
        opt.step()
        orc.adamw_step(p, [g.clone()], m, v, step, lr=3e-3, wd=0.1)
    assert (p[0] - p_ref.detach()).abs().max() < 1e-6
    g = [torch.full((4,), 3.0)]
    assert abs(orc.clip_grad_norm(g, 1.0) - 6.0) < 1e-6 and abs(float(g[0].norm()) - 1.0) < 1e-6


def test_elementwise_metric_noise_floor_of_fp32():
    """Under the element-wise metric |d| / max(|ref|, 1e-3 max|ref|) the fp32 oracle is already above 1e-4 from its
    own fp64 run (different rounding of the same graph), while it is below 5e-6 in the max-norm metric: the
    element-wise bar of the GPU tests (util.ELEM_TOL) cannot be 1e-4 for any fp32 implementation."""
    from util import block_params, elem_err, rel_err
    cfg = orc.Mamba2Config(d_model=128, d_state=16, d_head=32, n_heads=8, block_len=64)
    p = block_params(cfg, seed=3)
    g = torch.Generator(); g.manual_seed(21)
    x = torch.randn(2, 128, 128, generator=g); cot = torch.randn(2, 128, 128, generator=g)
    outs = {}
    for dt in (torch.float32, torch.float64):
        pr = {k: v.to(dt).clone().requires_grad_(True) for k, v in p.items()}
        xr = x.to(dt).clone().requires_grad_(True)
        out = orc.block_forward(pr, cfg, xr)
        (out * cot.to(dt)).sum().backward()
        outs[dt] = {"out": out.detach(), "dx": xr.grad, "d_in_proj_weight": pr["in_proj_weight"].grad}
    for k in outs[torch.float32]:
        assert rel_err(outs[torch.float32][k], outs[torch.float64][k]) < 5e-6, k
        assert elem_err(outs[torch.float32][k], outs[torch.float64][k]) > 1e-4, k
