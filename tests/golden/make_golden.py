"""Regenerates the golden vectors under tests/golden/ (needs a checkout of the reference repository).

1. ssd_q64.npz: the reference's own SSD fixture (reference/fixtures/ssd_q64: B=1, T=128,
   H=2, P=8, N=16, Q=64, seed 42).  The inputs are re-drawn exactly as
   reference/gen_fixtures.py:35-46 draws them, pushed through reference/mamba2_ref.py::ssd
   imported from the read-only reference checkout, and compared with the stored .npy files
   before being written here.
2. block_c1.npz: the oracle's output and gradients for the single-block fp32 case
   (B=2, T=128, D=128, H=8, P=32, N=16, Q=64) so a drift of the oracle itself is caught.

Usage: python tests/golden/make_golden.py --reference /path/to/reference-checkout
"""
import argparse
import pathlib
import sys

import numpy as np
import torch

HERE = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of the reference repository")
    args = ap.parse_args()
    ref = pathlib.Path(args.reference)
    sys.path.insert(0, str(ref / "reference"))
    from mamba2_ref import ssd  # noqa: E402  (the reference's Listing-1 script)

    torch.manual_seed(42)
    B, T, H, P, N, Q = 1, 128, 2, 8, 16, 64
    X = torch.randn(B, T, H, P)
    A = -torch.rand(B, T, H)
    Bp = torch.randn(B, T, H, N) * 0.5
    Cp = torch.randn(B, T, H, N) * 0.5
    Y, fs = ssd(X, A, Bp, Cp, Q)
    fx = ref / "reference" / "fixtures" / "ssd_q64"
    for name, val in (("X", X), ("A", A), ("B", Bp), ("C", Cp)):
        stored = np.load(fx / f"{name}.npy")
        assert np.array_equal(stored, val.numpy()), f"{name}: re-drawn inputs differ from the stored fixture"
    dy = np.abs(np.load(fx / "Y.npy") - Y.numpy()).max()
    ds = np.abs(np.load(fx / "final_state.npy") - fs.numpy()).max()
    print(f"ssd_q64: re-run vs stored fixture  max|dY|={dy:.3e}  max|dstate|={ds:.3e}")
    assert dy < 1e-5 and ds < 1e-5
    np.savez_compressed(HERE / "ssd_q64.npz", X=X.numpy(), A=A.numpy(), B=Bp.numpy(), C=Cp.numpy(),
                        Y=np.load(fx / "Y.npy"), final_state=np.load(fx / "final_state.npy"))

    from oracle import mamba2_oracle as orc
    cfg = orc.Mamba2Config(d_model=128, d_state=16, d_head=32, n_heads=8, n_groups=1, d_conv=4, block_len=64)
    p = orc.init_block_params(cfg, seed=1)
    for v in p.values():
        v.requires_grad_(True)
    g = torch.Generator(); g.manual_seed(11)
    x = torch.randn(2, 128, 128, generator=g).requires_grad_(True)
    g2 = torch.Generator(); g2.manual_seed(12)
    cot = torch.randn(2, 128, 128, generator=g2)
    out = orc.block_forward(p, cfg, x)
    (out * cot).sum().backward()
    blob = {"out": out.detach().numpy(), "dx": x.grad.numpy()}
    for k, v in p.items():
        blob["d_" + k] = v.grad.numpy()
    np.savez_compressed(HERE / "block_c1.npz", **blob)
    print("block_c1: |out|max", float(out.abs().max()), " wrote", sorted(blob))


if __name__ == "__main__":
    main()
