"""CPU oracle for the Mamba2 SSD block path (TEST INFRASTRUCTURE, not product code).

This module restates, op for op, the graph that the reference's Candle backend
executes for the Mamba2 block, its SSD scan, its decode step, the residual
stack with per-block activation checkpointing, and the tied-head LM loss.
Gradients come from torch autograd on the restated graph, the role Candle's
autograd plays in the reference.  Only tests, the smoke check and the CPU
baseline leg of the benchmark may import it; the CUDA library never does.

Parity pins (see tests/test_oracle.py): the reference's golden SSD fixture
(reference/fixtures/ssd_q64, regenerated through reference/mamba2_ref.py by
tests/golden/make_golden.py), the structural known answers of
crates/pm-core/src/mamba2/ssd.rs:105-120 and
crates/pm-candle/src/ops_impl.rs:491-593, dense == chunked == scalar,
step x T == forward, checkpointed == plain gradients.

The reference's primitive arithmetic lives in candle-core / candle-nn 0.11.0
(Cargo.lock:153-193), which is not vendored; its semantics are taken from the
call sites in crates/pm-candle/src/ops_impl.rs (one Candle call per op).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------
# Config and parameters (crates/pm-core/src/mamba2/block.rs:48-88, :440-450)
# --------------------------------------------------------------------------

PARAM_ORDER = (
    "in_proj_weight",   # (D, J)   used as x @ W
    "conv1d_weight",    # (X, 1, K)
    "conv1d_bias",      # (X,)
    "a_log",            # (H,)
    "d_skip",           # (H,)
    "dt_bias",          # (H,)
    "norm_weight",      # (I,)
    "out_proj_weight",  # (I, D)
)


@dataclass
class Mamba2Config:
    """Mirror of `Mamba2Config` (block.rs:48-72)."""

    d_model: int
    d_state: int
    d_head: int
    n_heads: int
    n_groups: int = 1
    d_conv: int = 4
    block_len: int = 64
    rmsnorm_eps: float = 1e-5

    @property
    def d_inner(self) -> int:
        return self.n_heads * self.d_head

    @property
    def xbc_dim(self) -> int:
        return self.d_inner + 2 * self.n_groups * self.d_state

    @property
    def in_proj_dim(self) -> int:
        return self.d_inner + self.xbc_dim + self.n_heads


def softplus_inv(y: torch.Tensor) -> torch.Tensor:
    return y + torch.log(-torch.expm1(-y))


def init_block_params(cfg: Mamba2Config, seed: int, dtype=torch.float32) -> dict:
    """Seeded block parameters: Kaiming-uniform projections/conv (U(+-1/sqrt(fan_in))),
    A = -exp(U[log 1, log 16]) per head, dt_bias = softplus^-1(U[1e-3, 1e-1]), D = 1,
    norm weight 1, conv bias 0.  One generator per tensor, seeded seed+i."""

    def gen(i):
        g = torch.Generator()
        g.manual_seed(seed * 1000 + i)
        return g

    def ku(shape, fan_in, i):
        bound = 1.0 / math.sqrt(fan_in)
        return (torch.rand(shape, generator=gen(i), dtype=torch.float64) * 2 - 1) * bound

    H = cfg.n_heads
    p = {
        "in_proj_weight": ku((cfg.d_model, cfg.in_proj_dim), cfg.d_model, 0),
        "conv1d_weight": ku((cfg.xbc_dim, 1, cfg.d_conv), cfg.d_conv, 1),
        "conv1d_bias": torch.zeros(cfg.xbc_dim, dtype=torch.float64),
        "a_log": torch.rand(H, generator=gen(3), dtype=torch.float64) * math.log(16.0),
        "d_skip": torch.ones(H, dtype=torch.float64),
        "dt_bias": softplus_inv(
            1e-3 + torch.rand(H, generator=gen(5), dtype=torch.float64) * (1e-1 - 1e-3)
        ),
        "norm_weight": torch.ones(cfg.d_inner, dtype=torch.float64),
        "out_proj_weight": ku((cfg.d_inner, cfg.d_model), cfg.d_inner, 7),
    }
    return {k: v.to(dtype) for k, v in p.items()}


# --------------------------------------------------------------------------
# Primitive ops as the Candle backend defines them
# --------------------------------------------------------------------------

def softplus(x: torch.Tensor) -> torch.Tensor:
    """max(x,0) + log(1 + exp(-|x|))  (crates/pm-candle/src/ops_impl.rs:123-133)."""
    return torch.relu(x) + torch.log(torch.exp(-x.abs()) + 1.0)


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x * w / sqrt(mean(x^2, -1) + eps)  (crates/pm-candle/src/ops_impl.rs:93,107-115)."""
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x / torch.sqrt(ms + eps) * w


# --------------------------------------------------------------------------
# SSD scan: scalar, dense, chunked (crates/pm-core/src/mamba2/ssd.rs:33-97,
# crates/pm-core/src/mamba2/ssd_ops.rs:61-284)
# --------------------------------------------------------------------------

def ssd_scan_naive_scalar(x, a, b, c):
    """O(B H T^2 (P+N)) scalar loops (ssd.rs:33-97).  numpy float32 in/out; small cases only."""
    x = np.asarray(x, np.float32); a = np.asarray(a, np.float32)
    b = np.asarray(b, np.float32); c = np.asarray(c, np.float32)
    Bn, T, H, P = x.shape
    y = np.zeros_like(x)
    a_cum = np.zeros_like(a)
    for bi in range(Bn):
        for hi in range(H):
            acc = np.float32(0)
            for ti in range(T):
                acc = np.float32(acc + a[bi, ti, hi])
                a_cum[bi, ti, hi] = acc
    for bi in range(Bn):
        for hi in range(H):
            for ti in range(T):
                bc = (b[bi, : ti + 1, hi, :] * c[bi, ti, hi, :][None, :]).sum(-1, dtype=np.float32)
                decay = np.exp(a_cum[bi, ti, hi] - a_cum[bi, : ti + 1, hi]).astype(np.float32)
                w = (decay * bc).astype(np.float32)
                y[bi, ti, hi, :] = (w[:, None] * x[bi, : ti + 1, hi, :]).sum(0, dtype=np.float32)
    return y


def ssd_scan_dense(x, a, b, c):
    """Dense (B,H,T,T) scan with the additive -1e9 log-mask (ssd_ops.rs:83-138)."""
    Bn, T, H, _P = x.shape
    a_cum = torch.cumsum(a, dim=1).transpose(1, 2)               # (B,H,T)
    a_diff = a_cum.unsqueeze(-1) - a_cum.unsqueeze(-2)          # (B,H,T,T)
    log_mask = torch.triu(torch.full((T, T), -1.0e9, dtype=a.dtype), diagonal=1)
    decay = torch.exp(a_diff + log_mask)
    c_perm = c.transpose(1, 2)                                   # (B,H,T,N)
    b_perm_t = b.transpose(1, 2).transpose(2, 3)                 # (B,H,N,T)
    bc = c_perm @ b_perm_t
    combined = decay * bc
    y = combined @ x.transpose(1, 2)                             # (B,H,T,P)
    return y.transpose(1, 2)


def ssd_scan_chunked(x, a, b, c, block_len, initial_state=None, return_final_state=False):
    """Chunked scan, state layout (B,H,N,P), sequential chunk loop (ssd_ops.rs:167-284).

    `initial_state` / `return_final_state` extend the reference signature so the decode
    tests can seed and read the carried state; with the defaults it is the reference call."""
    Bn, T, H, P = x.shape
    N = b.shape[3]
    Q = block_len
    assert T % Q == 0
    nc = T // Q
    y_intra = ssd_scan_dense(
        x.reshape(Bn * nc, Q, H, P), a.reshape(Bn * nc, Q, H),
        b.reshape(Bn * nc, Q, H, N), c.reshape(Bn * nc, Q, H, N),
    ).reshape(Bn, nc, Q, H, P)
    a_pc = a.reshape(Bn, nc, Q, H)
    a_cum = torch.cumsum(a_pc, dim=2)
    a_end = a_cum[:, :, Q - 1 : Q, :]
    decay_to_end = torch.exp(a_end - a_cum)                      # (B,nc,Q,H)
    x_pc = x.reshape(Bn, nc, Q, H, P)
    b_pc = b.reshape(Bn, nc, Q, H, N)
    weighted_x = decay_to_end.unsqueeze(-1) * x_pc
    b_flat = b_pc.transpose(2, 3).transpose(3, 4).reshape(Bn * nc * H, N, Q)
    wx_flat = weighted_x.transpose(2, 3).reshape(Bn * nc * H, Q, P)
    states = (b_flat @ wx_flat).reshape(Bn, nc, H, N, P)
    decay_full = torch.exp(a_end)                                # (B,nc,1,H)
    decay_from_start = torch.exp(a_cum)                          # (B,nc,Q,H)
    c_pc = c.reshape(Bn, nc, Q, H, N)
    h = torch.zeros(Bn, H, N, P, dtype=x.dtype) if initial_state is None else initial_state
    pieces = []
    for ci in range(nc):
        c_bhqn = c_pc[:, ci].transpose(1, 2)                     # (B,H,Q,N)
        prod = (c_bhqn @ h).transpose(1, 2)                      # (B,Q,H,P)
        pieces.append((prod * decay_from_start[:, ci].unsqueeze(-1)).unsqueeze(1))
        h = h * decay_full[:, ci].reshape(Bn, H, 1, 1) + states[:, ci]
    y = (y_intra + torch.cat(pieces, dim=1)).reshape(Bn, T, H, P)
    if return_final_state:
        return y, h
    return y


def ssd_scan_ops_default(x, a, b, c, block_len):
    """Dispatch rule of ssd_ops.rs:61-80."""
    T = x.shape[1]
    if block_len == 0 or block_len >= T or T % block_len != 0:
        return ssd_scan_dense(x, a, b, c)
    return ssd_scan_chunked(x, a, b, c, block_len)


# --------------------------------------------------------------------------
# Mamba2Block::forward (crates/pm-core/src/mamba2/block.rs:118-226)
# --------------------------------------------------------------------------

def block_forward(p: dict, cfg: Mamba2Config, x: torch.Tensor, return_intermediates: bool = False):
    """`x` (B,T,D) in the ambient compute dtype cdt (fp32 or bf16).  Parameters are fp32
    and cast to cdt at the two projections; conv, softplus, exp, ssd_scan and rmsnorm run
    in fp32 ("islands", block.rs:24-42)."""
    Bn, T, D = x.shape
    assert D == cfg.d_model
    assert cfg.n_groups in (1, cfg.n_heads)
    cdt = x.dtype
    f32 = p["in_proj_weight"].dtype if p["in_proj_weight"].dtype == torch.float64 else torch.float32
    I, X, H, N, G, K = cfg.d_inner, cfg.xbc_dim, cfg.n_heads, cfg.d_state, cfg.n_groups, cfg.d_conv
    gn = G * N

    xzd = x @ p["in_proj_weight"].to(cdt)                        # block.rs:143-144
    z = xzd[..., :I]
    xbc = xzd[..., I : I + X]
    dt_raw = xzd[..., I + X :]

    # conv island: (B,X,T) layout, padding K-1, keep the first T outputs (block.rs:150-163)
    xbc_chw = xbc.transpose(1, 2).to(f32)
    conv = F.conv1d(xbc_chw, p["conv1d_weight"], None, stride=1, padding=K - 1, groups=X)
    conv = conv + p["conv1d_bias"].reshape(-1, 1)
    xbc_act = silu(conv.to(cdt)[..., :T].transpose(1, 2))

    x_ssm = xbc_act[..., :I].reshape(Bn, T, H, cfg.d_head)
    b_4d = xbc_act[..., I : I + gn].reshape(Bn, T, G, N)
    c_4d = xbc_act[..., I + gn : I + 2 * gn].reshape(Bn, T, G, N)
    if G != H:
        b_4d = b_4d.expand(Bn, T, H, N)
        c_4d = c_4d.expand(Bn, T, H, N)

    dt = softplus(dt_raw.to(f32) + p["dt_bias"].reshape(1, 1, H)).to(cdt)   # block.rs:184-188
    a_neg = (-torch.exp(p["a_log"])).to(cdt)
    a_bth = a_neg.reshape(1, 1, H) * dt                                       # block.rs:192-196
    x_dt = x_ssm * dt.unsqueeze(-1)                                           # block.rs:198-199

    y = ssd_scan_ops_default(x_dt.to(f32), a_bth.to(f32), b_4d.to(f32), c_4d.to(f32),
                             cfg.block_len).to(cdt)                           # block.rs:203-208
    y = y + p["d_skip"].to(cdt).reshape(1, 1, H, 1) * x_ssm                   # block.rs:210-213
    y = y.reshape(Bn, T, I)
    gated = y * silu(z)                                                       # block.rs:216-217
    normed = rmsnorm(gated.to(f32), p["norm_weight"], cfg.rmsnorm_eps).to(cdt)
    out = normed @ p["out_proj_weight"].to(cdt)                               # block.rs:224-225
    if return_intermediates:
        return out, dict(xzd=xzd, xbc_act=xbc_act, dt=dt, y=y, normed=normed)
    return out


# --------------------------------------------------------------------------
# Mamba2Block::step (block.rs:278-417) with Mamba2State (state.rs:31-51)
# --------------------------------------------------------------------------

def zero_state(cfg: Mamba2Config, batch: int, dtype=torch.float32):
    return dict(
        ssm_state=torch.zeros(batch, cfg.n_heads, cfg.d_state, cfg.d_head, dtype=dtype),
        conv_window=torch.zeros(batch, cfg.xbc_dim, cfg.d_conv - 1, dtype=dtype),
    )


def block_step(p: dict, cfg: Mamba2Config, x_t: torch.Tensor, state: dict):
    """One-token recurrence; returns (y_t (B,1,D), new state).  block.rs:278-417."""
    Bn, T, D = x_t.shape
    assert T == 1 and D == cfg.d_model
    cdt = x_t.dtype
    f32 = state["ssm_state"].dtype
    I, X, H, N, G, K, P = (cfg.d_inner, cfg.xbc_dim, cfg.n_heads, cfg.d_state, cfg.n_groups,
                           cfg.d_conv, cfg.d_head)
    gn = G * N
    xzd = x_t @ p["in_proj_weight"].to(cdt)
    z, xbc, dt_raw = xzd[..., :I], xzd[..., I : I + X], xzd[..., I + X :]
    win = torch.cat([state["conv_window"], xbc.transpose(1, 2).to(f32)], dim=2)   # (B,X,K)
    conv = F.conv1d(win, p["conv1d_weight"], None, stride=1, padding=0, groups=X)
    conv = conv + p["conv1d_bias"].reshape(-1, 1)
    xbc_act = silu(conv.transpose(1, 2).to(cdt))                                  # (B,1,X)
    window_next = win[:, :, 1:]
    x_ssm = xbc_act[..., :I].reshape(Bn, 1, H, P)
    b_4d = xbc_act[..., I : I + gn].reshape(Bn, 1, G, N)
    c_4d = xbc_act[..., I + gn :].reshape(Bn, 1, G, N)
    if G != H:
        b_4d = b_4d.expand(Bn, 1, H, N)
        c_4d = c_4d.expand(Bn, 1, H, N)
    dt = softplus(dt_raw.to(f32) + p["dt_bias"].reshape(1, 1, H))                  # (B,1,H)
    a_dt = (-torch.exp(p["a_log"])).reshape(1, 1, H) * dt
    decay = torch.exp(a_dt).reshape(Bn, H, 1, 1)
    bx = b_4d.to(f32).reshape(Bn, H, N, 1) * x_ssm.to(f32).reshape(Bn, H, 1, P)
    h_new = decay * state["ssm_state"] + dt.reshape(Bn, H, 1, 1) * bx
    y = (c_4d.to(f32).reshape(Bn, H, 1, N) @ h_new).reshape(Bn, 1, H, P).to(cdt)
    y = y + p["d_skip"].to(cdt).reshape(1, 1, H, 1) * x_ssm
    gated = y.reshape(Bn, 1, I) * silu(z)
    normed = rmsnorm(gated.to(f32), p["norm_weight"], cfg.rmsnorm_eps).to(cdt)
    y_t = normed @ p["out_proj_weight"].to(cdt)
    return y_t, dict(ssm_state=h_new.detach(), conv_window=window_next.detach())


# --------------------------------------------------------------------------
# Residual stack and checkpointing (photon/encoder.rs:52-87, checkpoint.rs:68-135)
# --------------------------------------------------------------------------

def stack_forward(layers: list, cfg: Mamba2Config, x: torch.Tensor) -> torch.Tensor:
    """h_l = h_{l-1} + Block_l(h_{l-1}); no norms (encoder.rs:52-62)."""
    h = x
    for p in layers:
        h = h + block_forward(p, cfg, h)
    return h


def stack_forward_checkpointed(layers: list, cfg: Mamba2Config, x: torch.Tensor):
    """Each block's raw output is replaced by a fresh leaf (`boundary`, checkpoint.rs:82)
    so the block's tape is dropped; returns (hidden, segments)."""
    segments = []
    h = x
    for i, p in enumerate(layers):
        with torch.no_grad():
            raw = block_forward(p, cfg, h)
        boundary = raw.detach().clone().requires_grad_(True)
        segments.append(dict(saved_input=h, boundary=boundary, block_id=i))
        h = h + boundary
    return h, segments


def checkpoint_backward(layers: list, cfg: Mamba2Config, segments: list, leaves: list):
    """Reverse walk over segments (checkpoint.rs:110-135): recompute the block from its
    saved input, backprop sum(recompute * dy).  `saved_input` is still attached to the main
    graph, so each inner backward also deposits into earlier boundaries and `leaves`."""
    for seg in reversed(segments):
        dy = seg["boundary"].grad
        if dy is None:
            continue
        recomp = block_forward(layers[seg["block_id"]], cfg, seg["saved_input"])
        phantom = (recomp * dy).sum()
        phantom.backward(retain_graph=True)   # the residual adds of the main tape are walked once per segment


# --------------------------------------------------------------------------
# Flat LM: tied embedding -> stack -> tied head -> mean CE
# (flat.rs:89-138, photon/embedding.rs:54-66, pm-train/src/loss.rs:39-69)
# --------------------------------------------------------------------------

def lm_loss(embed: torch.Tensor, layers: list, cfg: Mamba2Config, ids: torch.Tensor,
            targets: torch.Tensor, cdt=torch.float32, checkpointed: bool = False):
    """Returns the scalar loss; when `checkpointed`, runs the two-phase backward itself and
    returns the detached loss (all leaf .grad fields are then populated)."""
    x = embed[ids].to(cdt)
    if not checkpointed:
        hidden = stack_forward(layers, cfg, x)
        segs = None
    else:
        hidden, segs = stack_forward_checkpointed(layers, cfg, x)
    logits = hidden @ embed.to(cdt).transpose(0, 1)
    logp = torch.log_softmax(logits.to(torch.float32 if embed.dtype != torch.float64 else torch.float64), dim=-1)
    loss = -logp.gather(-1, targets.unsqueeze(-1)).mean()
    if checkpointed:
        loss.backward(retain_graph=True)
        checkpoint_backward(layers, cfg, segs, [])
        return loss.detach()
    return loss


def hier_lm_loss(embed, wproj, layers0, layers1, cfg, ids, targets, group=4, cdt=torch.float32):
    """Two-level benchmark LM (defined by the benchmark's configuration list, not by the reference's PHOTON glue):
    level 0 = Mamba2 stack at token rate; groups of `group` hidden states are mean-pooled and linearly projected
    into level 1, a Mamba2 stack at 1/group rate; its outputs are repeated `group` times, shifted by one group
    (causal), and added to the level-0 output before the tied LM head.  Blocks and stacks are the reference's
    (block.rs:118-226, encoder.rs:52-62); the loss is the mean CE of pm-train/src/loss.rs:39-69."""
    x = embed[ids].to(cdt)
    h0 = stack_forward(layers0, cfg, x)
    Bn, T, D = h0.shape
    pooled = h0.float().reshape(Bn, T // group, group, D).mean(2).to(cdt)
    u = pooled @ wproj.to(cdt)
    h1 = stack_forward(layers1, cfg, u)
    up = torch.repeat_interleave(h1, group, dim=1)
    up = torch.cat([torch.zeros(Bn, group, D, dtype=up.dtype), up[:, : T - group]], dim=1)
    hidden = (h0.float() + up.float()).to(cdt)
    logits = hidden @ embed.to(cdt).transpose(0, 1)
    logp = torch.log_softmax(logits.float(), dim=-1)
    return -logp.gather(-1, targets.unsqueeze(-1)).mean()


def lcg_batch(state: int, b: int, t: int, vocab: int):
    """Seeded uniform token batch, targets = ids rotated left by one within each row
    (crates/pm-cli/src/train_cmd.rs:523-539).  Returns (ids, targets, new_state)."""
    mask = (1 << 64) - 1
    ids = np.zeros(b * t, np.int64)
    for i in range(b * t):
        state = (state * 6364136223846793005 + 1442695040888963407) & mask
        ids[i] = (state >> 33) % vocab
    ids = ids.reshape(b, t)
    targets = np.roll(ids, -1, axis=1)
    return torch.from_numpy(ids), torch.from_numpy(targets.copy()), state


# --------------------------------------------------------------------------
# Optimizer (crates/pm-train/src/clip.rs:13-53, crates/pm-train/src/optim.rs:104-157)
# --------------------------------------------------------------------------

def clip_grad_norm(grads: list, max_norm: float) -> float:
    """Global L2 norm over all tensors; scales them in place by max_norm / norm when the norm exceeds max_norm.
    Returns the unclipped norm."""
    total = sum(float((g.double() ** 2).sum()) for g in grads)
    norm = total ** 0.5
    if norm > max_norm and norm > 0:
        for g in grads:
            g.mul_(max_norm / norm)
    return norm


def adamw_step(params: list, grads: list, m: list, v: list, step: int, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.0):
    """One AdamW step in the reference's operation order; all tensors updated in place; `step` is 1-based."""
    bc1, bc2 = 1.0 - beta1 ** step, 1.0 - beta2 ** step
    for p, g, mi, vi in zip(params, grads, m, v):
        if wd > 0.0:
            p.mul_(1.0 - lr * wd)
        mi.mul_(beta1).add_(g * (1.0 - beta1))
        vi.mul_(beta2).add_(g * g * (1.0 - beta2))
        update = (mi * (1.0 / bc1)) / (torch.sqrt(vi * (1.0 / bc2)) + eps)
        p.sub_(update * lr)
