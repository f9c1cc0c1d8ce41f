"""GPU parity of the ordering kernels (through the C ABI) against the CPU checker: bit-exact."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle
from tests.util import to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lb():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import lampa_b200
    return lampa_b200


def _dev(x):
    return x.to("cuda:0")


@pytest.mark.parametrize("N", [1, 37, 1024, 5000, 60000])
def test_bucket_ids_bit_exact(lb, N):
    from lampa_b200 import synth
    x = synth.detector_hits(20253, N)
    alpha, beta = synth.lsh_params(20253)
    out = lb.lsh_hash(_dev(x), _dev(alpha), _dev(beta), 1.0, want_keys=True, want_packed=True)
    ids_ref, keys_ref = oracle.lsh_ids(x.numpy(), alpha.numpy(), beta.numpy(), 1.0, want_keys=True)
    np.testing.assert_array_equal(to_np(out["ids"]), ids_ref)
    np.testing.assert_array_equal(to_np(out["keys"]), keys_ref)
    packed_ref = (ids_ref.astype(np.int64) << np.arange(8)[None, :, None]).sum(1).astype(np.int32)
    np.testing.assert_array_equal(to_np(out["packed"]), packed_ref)


def test_bucket_ids_other_widths_and_generic_dims(lb):
    rng = np.random.default_rng(5)
    x = torch.from_numpy(rng.standard_normal((3000, 11)).astype(np.float32) * 50)
    alpha = torch.from_numpy(rng.standard_normal((5, 9, 4)).astype(np.float32))
    beta = torch.from_numpy(rng.uniform(0, 2.5, 4).astype(np.float32))
    out = lb.lsh_hash(_dev(x), _dev(alpha), _dev(beta), 2.5, dim=9)
    np.testing.assert_array_equal(to_np(out["ids"]), oracle.lsh_ids(x.numpy(), alpha.numpy(), beta.numpy(), 2.5))


@pytest.mark.parametrize("N", [1, 2, 1000, 8191, 8192, 8193, 60000])
def test_stable_sort_rows_bit_exact(lb, N):
    from lampa_b200 import synth
    x = synth.detector_hits(20253, N)
    alpha, beta = synth.lsh_params(20253)
    ids, perm = lb.lsh_bucket_sort(_dev(x), _dev(alpha), _dev(beta), 1.0)
    ids_np = to_np(ids)
    perm_np = to_np(perm)
    assert perm_np.dtype == np.int64
    for r in range(3):
        for h in range(8):
            ref = oracle.segsort(np.ascontiguousarray(ids_np[r, h]))
            np.testing.assert_array_equal(perm_np[r, h], ref)


def test_sort_edge_cases(lb):
    dev = "cuda:0"
    # all-equal keys: identity (stable); empty input; negative and extreme keys; ragged segments
    k = torch.full((5000,), 7, dtype=torch.int32, device=dev)
    np.testing.assert_array_equal(to_np(lb.segmented_sort(k)), np.arange(5000))
    assert lb.segmented_sort(torch.empty(0, dtype=torch.int32, device=dev)).numel() == 0
    rng = np.random.default_rng(1)
    k = rng.integers(-2**31, 2**31 - 1, 70000, dtype=np.int64).astype(np.int32)
    k[:10] = [-2**31, 2**31 - 1, 0, -1, 1, -2**31, 2**31 - 1, 0, -1, 1]
    np.testing.assert_array_equal(to_np(lb.segmented_sort(torch.from_numpy(k).to(dev))), np.argsort(k, kind="stable"))
    seg = np.array([0, 0, 1, 1000, 1000, 20000, 70000], np.int64)
    got = to_np(lb.segmented_sort(torch.from_numpy(k).to(dev), seg_offsets=torch.from_numpy(seg)))
    np.testing.assert_array_equal(got, oracle.segsort(k, seg))
    # few distinct keys (many ties) and float keys incl. negatives and signed zeros
    k2 = rng.integers(-3, 4, 50000).astype(np.int32)
    np.testing.assert_array_equal(to_np(lb.segmented_sort(torch.from_numpy(k2).to(dev))), np.argsort(k2, kind="stable"))
    f = rng.standard_normal(30000).astype(np.float32) * 1e3
    f[:6] = [0.0, -0.0, 0.0, -0.0, np.float32(1e-40), -np.float32(1e-40)]
    got = to_np(lb.segmented_sort(torch.from_numpy(f).to(dev)))
    np.testing.assert_array_equal(got, oracle.segsort(f))
    # composed with a starting order
    init = rng.permutation(30000).astype(np.int64)
    got = to_np(lb.segmented_sort(torch.from_numpy(f).to(dev), init=torch.from_numpy(init).to(dev)))
    np.testing.assert_array_equal(got, oracle.segsort(f, init=init))


def test_permute_invert_roundtrip(lb):
    dev = "cuda:0"
    rng = np.random.default_rng(2)
    for rows, width, dt in [(60000, 128, torch.bfloat16), (1000, 24, torch.float32), (777, 3, torch.float32), (0, 8, torch.float32)]:
        x = torch.randn(rows, width).to(dt)
        perm = torch.from_numpy(rng.permutation(rows).astype(np.int64)) if rows else torch.empty(0, dtype=torch.int64)
        y = lb.permute_rows(x.to(dev), perm.to(dev))
        assert torch.equal(y.cpu(), x[perm])
        inv = lb.invert_permutation(perm.to(dev)) if rows else perm.to(dev)
        if rows:
            np.testing.assert_array_equal(to_np(inv), oracle.invert_perm(perm.numpy()))
            assert torch.equal(lb.permute_rows(y, inv).cpu(), x)
            assert torch.equal(lb.permute_rows(y, perm.to(dev), scatter=True).cpu(), x)


def test_reference_named_ops_against_golden(lb, golden_dir):
    """LSHOrdering / E2LSH / sort_to_buckets / unsort_from_buckets / invert_permutation on the
    fixture produced by the reference's own code (float keys: tolerance on keys, order checked
    under the reference's key)."""
    z = np.load(os.path.join(golden_dir, "lsh_ordering_B2_L1500.npz"))
    dev = "cuda:0"
    coords = torch.from_numpy(z["coords"]).to(dev)
    points = torch.from_numpy(z["points"]).to(dev)
    B, Ln, C = coords.shape
    ordering = lb.LSHOrdering(C, num_hashes=3).to(dev)
    ordering.e2lsh.alpha.data.copy_(torch.from_numpy(z["alpha"]))
    ordering.e2lsh.beta.data.copy_(torch.from_numpy(z["beta"]))
    proj = ordering.e2lsh(coords.reshape(1, B * Ln, C))                     # [3, 1, N]
    np.testing.assert_allclose(to_np(proj)[:, 0], z["proj"][:, :, 0], rtol=1e-5, atol=1e-3)
    ordered, idx = ordering(points, coords)
    idx_np = to_np(idx)
    assert (idx_np == z["indices"]).mean() > 0.99
    assert torch.equal(ordered.cpu(), torch.from_numpy(z["points"])[torch.arange(B)[:, None], idx.cpu()])
    for b in range(B):
        np.testing.assert_array_equal(idx_np[b], oracle.lsh_ordering(z["coords"][b], z["alpha"]))
    ref_idx = torch.from_numpy(z["indices"]).to(dev)
    inv = lb.invert_permutation(ref_idx)
    np.testing.assert_array_equal(to_np(inv), z["inverse"])
    buckets = lb.sort_to_buckets(points, ref_idx[None], 100)
    np.testing.assert_array_equal(to_np(buckets), z["buckets"])
    back = lb.unsort_from_buckets(buckets, inv[None])
    np.testing.assert_array_equal(to_np(back), z["unsorted"])
    qh, kh, shift = lb.lsh_mapping(ordering.e2lsh, coords.reshape(1, B * Ln, C), coords.reshape(1, B * Ln, C))
    assert shift.shape == (3, 1, 1) and torch.equal(qh, kh)
