"""Helpers shared by the parity tests."""
import numpy as np
import torch


def to_np(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy() if t.is_floating_point() else t.detach().cpu().numpy()


def err_stats(got: np.ndarray, ref: np.ndarray):
    d = got.astype(np.float64) - ref.astype(np.float64)
    return float(np.abs(d).max()), float(np.linalg.norm(d) / max(np.linalg.norm(ref), 1e-30))


def assert_close_bf16(got, ref, what=""):
    """Tolerance of the build target for bf16 runs against the fp32 checker:
    max-abs <= 2e-2 (scaled by max(1, |ref|_inf): bf16 cannot resolve 2e-2 on values above ~4)
    and relative L2 <= 1e-2."""
    mx, rl = err_stats(got, ref)
    scale = max(1.0, float(np.abs(ref).max()))
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    assert mx <= 2e-2 * scale, f"{what}: max-abs {mx:.3e} (ref scale {scale:.2f})"
    assert rl <= 1e-2, f"{what}: rel-L2 {rl:.3e}"
    return mx, rl
