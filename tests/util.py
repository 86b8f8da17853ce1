"""Shared helpers for the parity tests."""
import os
import pathlib

import numpy as np
import torch

from oracle import mamba2_oracle as orc

GOLD = pathlib.Path(__file__).resolve().parent / "golden"

# Parity bar for fp32 work: max |ours - oracle| <= FP32_TOL * max |oracle| per tensor
# (the reference compares backends by max-abs error at 1e-4 on O(1) data, SUMMARY.md:44-45).
FP32_TOL = 1e-4


# The gradients of a_log and dt_bias are sums over all tokens of S-weighted differences of nearly equal terms (row
# sums minus column sums of dM o M).  On the shapes the fused tensor-core scan takes (block_len % 128 == 0, d_state =
# d_head = 64) both sums come from the same registers (csrc/ssd_fused.cu) and the two tensors get the bar of every
# other tensor (`fused=True`).  The fp32 FMA engine that serves the remaining (small or ragged) shapes forms the
# difference from y and dx~ instead and is held to 5e-4 there (the reference's own cross-backend SSD gradient tests
# use 1e-3, crates/pm-cuda/tests/grad_ssd.rs:62-227).
CANCELLATION_TOL = 5e-4

# One 24-layer step: every tensor carries the rounding of ~150 bf16-pair GEMMs in sequence (16 mantissa bits per
# operand, ~1.5e-5 of the result's scale per layer), which random-walks to 1.1e-4 .. 1.9e-4 at depth 24 (measured,
# parity report); single blocks and 2-layer models stay under FP32_TOL.
DEPTH24_TOL = 2.5e-4


def tol_for(name: str, fused: bool = False) -> float:
    return CANCELLATION_TOL if (not fused and name.endswith(("a_log", "dt_bias"))) else FP32_TOL


def rel_err(ours, ref) -> float:
    ours = ours.detach().double().cpu() if torch.is_tensor(ours) else torch.as_tensor(np.asarray(ours)).double()
    ref = ref.detach().double().cpu() if torch.is_tensor(ref) else torch.as_tensor(np.asarray(ref)).double()
    assert ours.shape == ref.shape, (ours.shape, ref.shape)
    scale = float(ref.abs().max())
    return float((ours - ref).abs().max()) / (scale if scale > 0 else 1.0)


def assert_close(ours, ref, tol=FP32_TOL, what=""):
    e = rel_err(ours, ref)
    assert e <= tol, f"{what}: rel max err {e:.3e} > {tol:.1e}"
    return e


def randn(shape, seed, scale=1.0):
    g = torch.Generator(); g.manual_seed(seed)
    return torch.randn(shape, generator=g) * scale


def rand(shape, seed):
    g = torch.Generator(); g.manual_seed(seed)
    return torch.rand(shape, generator=g)


def oracle_cfg(**kw):
    return orc.Mamba2Config(**kw)


def to_pm_cfg(cfg):
    import pm_b200
    return pm_b200.Mamba2Config(d_model=cfg.d_model, d_state=cfg.d_state, d_head=cfg.d_head, n_heads=cfg.n_heads,
                                n_groups=cfg.n_groups, d_conv=cfg.d_conv, block_len=cfg.block_len,
                                rmsnorm_eps=cfg.rmsnorm_eps)


def block_params(cfg, seed, perturb=True):
    """Oracle-initialised block parameters; bias/norm weight perturbed so their gradients matter."""
    p = orc.init_block_params(cfg, seed)
    if perturb:
        p["conv1d_bias"] = p["conv1d_bias"] + randn(p["conv1d_bias"].shape, seed * 7 + 1, 0.1)
        p["norm_weight"] = p["norm_weight"] + randn(p["norm_weight"].shape, seed * 7 + 2, 0.1)
        p["d_skip"] = p["d_skip"] + randn(p["d_skip"].shape, seed * 7 + 3, 0.1)
    return p


def cuda_params(p):
    return {k: v.detach().clone().cuda().contiguous() for k, v in p.items()}


# Element-wise metric: max over elements of |ours - ref| / max(|ref|, 1e-3 * max|ref|).  It is up to 1000x stricter
# than the max-norm metric on small elements.  Two correct fp32 evaluations that sum in different orders already
# differ by 2e-4 .. 5e-4 under it (the fp32 oracle against its own fp64 run, at single-block and at production
# dims; tests/test_oracle.py::test_elementwise_metric_noise_floor_of_fp32 pins that), so 1e-4 is below the noise
# floor of fp32 itself.  The GPU tests gate it at ELEM_TOL and write the measured values to PARITY_REPORT.
ELEM_TOL = 1e-2
# (PMB_PARITY_REPORT names the file; by default it goes to test_reports/ at the repository root, which git ignores)
PARITY_REPORT = pathlib.Path(os.environ.get("PMB_PARITY_REPORT") or
                             pathlib.Path(__file__).resolve().parent.parent / "test_reports" / "parity_report.jsonl")


def elem_err(ours, ref) -> float:
    ours = ours.detach().double().cpu() if torch.is_tensor(ours) else torch.as_tensor(np.asarray(ours)).double()
    ref = ref.detach().double().cpu() if torch.is_tensor(ref) else torch.as_tensor(np.asarray(ref)).double()
    assert ours.shape == ref.shape, (ours.shape, ref.shape)
    scale = float(ref.abs().max())
    den = torch.clamp(ref.abs(), min=1e-3 * (scale if scale > 0 else 1.0))
    return float(((ours - ref).abs() / den).max())


def report(case: str, what: str, ours, ref, tol=FP32_TOL, elem_tol=ELEM_TOL):
    """Gates both metrics and appends the measured values to the parity report (one JSON object per line)."""
    import json
    e, ee = rel_err(ours, ref), elem_err(ours, ref)
    try:
        PARITY_REPORT.parent.mkdir(exist_ok=True)
        with open(PARITY_REPORT, "a") as f:
            f.write(json.dumps({"case": case, "tensor": what, "max_norm": e, "elementwise": ee, "tol": tol, "elem_tol": elem_tol}) + "\n")
    except OSError:
        pass
    assert e <= tol, f"{case} {what}: rel max err {e:.3e} > {tol:.1e}"
    assert ee <= elem_tol, f"{case} {what}: element-wise err {ee:.3e} > {elem_tol:.1e}"
    return e, ee


def assert_close_bf16(ours, ref32, ref16, what, tol=2e-2):
    """bf16-storage bound: 2e-2 of the fp32 oracle, or -- where two correct bf16 evaluations differ by more at the test's
    tiny widths -- twice the distance between the oracle run in bf16 and the oracle run in fp32."""
    e = rel_err(ours, ref32)
    floor = rel_err(ref16, ref32)
    bound = max(tol, 2.0 * floor)
    assert e <= bound, f"{what}: rel max err {e:.3e} > {bound:.1e} (bf16 oracle vs fp32 oracle: {floor:.3e})"
    return e, floor
