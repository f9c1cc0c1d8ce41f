"""GPU parity of the region (geo) shift path through the C ABI: bit-exact against the numpy
checker and the reference-generated fixture for ranks, regions, ranges, shifts and keys;
positions agree wherever keys do not tie."""
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
    os.environ["LAMPA_B200_CHECK"] = "1"
    return lampa_b200


def _c(x, dt=None):
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t if dt is None else t.to(dt)


def test_fixture_from_reference(lb, golden_dir):
    z = np.load(os.path.join(golden_dir, "geo_shift_N1090_R12.npz"))
    raw, block = int(z["raw_size"]), int(z["block_size"])
    regions = _c(z["regions"])
    inp = lb.region_inputs(_c(z["coords"]), regions, block)
    assert inp["raw_size"] == raw and inp["coords"].shape[0] == 1100
    assert not inp["coords"][raw:].any()
    # ranks of the real hits equal the inverse of the reference's argsort
    inv_eta = np.empty(1100, np.int64); inv_eta[z["sorted_eta"]] = np.arange(1100)
    np.testing.assert_array_equal(to_np(inp["ranks"][0])[:raw], inv_eta[:raw])
    np.testing.assert_array_equal(to_np(inp["region_indices"][0])[:, :raw], z["reg_eta"][:, :raw])
    np.testing.assert_array_equal(to_np(inp["region_indices"][1])[:, :raw], z["reg_phi"][:, :raw])
    # quantile_partition on the reference's own argsort: every column
    qp = lb.quantile_partition(_c(z["sorted_phi"]), inp["regions_h"][1][:, None])
    np.testing.assert_array_equal(to_np(qp), z["reg_phi"])
    # range over queries and keys (padded rows project to 0 in the reference at that point)
    qh = z["q_hashed"].copy(); kh = z["k_hashed"].copy()
    qh[..., raw:] = 0; kh[..., raw:] = 0
    hs = lb.row_range(_c(qh), _c(kh))
    np.testing.assert_array_equal(to_np(hs).reshape(-1), z["hash_shift"].reshape(-1))
    # get_geo_shift on the reference's regions
    sh = lb.get_geo_shift(inp["regions_h"], _c(z["hash_shift"]), [_c(z["reg_eta"]), _c(z["reg_phi"])], 3)
    assert tuple(sh.shape) == (2, 3, 4, 1100)
    np.testing.assert_array_equal(to_np(sh[0]), z["q_shift"])
    np.testing.assert_array_equal(to_np(sh[1]), z["k_shift"])


def test_fixture_positions_end_to_end(lb, golden_dir):
    z = np.load(os.path.join(golden_dir, "geo_shift_N1090_R12.npz"))
    raw, block = int(z["raw_size"]), int(z["block_size"])
    inp = lb.region_inputs(_c(z["coords"]), _c(z["regions"]), block)
    e2 = lb.E2LSH(n_hashes=3, n_heads=4, dim=8).cuda()
    e2.alpha.data.copy_(_c(z["alpha"])); e2.beta.data.copy_(_c(z["beta"]))
    qpos, kpos = lb.hept_positions(e2, _c(z["q_hat"]), _c(z["k_hat"]), inp["regions_h"], inp["ranks"], raw)
    assert qpos.dtype == torch.int64 and tuple(qpos.shape) == (3, 4, 1100)
    for got, ref_keys, ref_pos in ((qpos, z["q_keys"], z["q_pos"]), (kpos, z["k_keys"], z["k_pos"])):
        got = to_np(got).reshape(12, -1)
        rk = ref_keys.reshape(12, -1)
        # a permutation, padded hits last, and the reference's keys come out in ascending order up
        # to the difference in summation order of the 8-term projections
        assert (np.sort(got, 1) == np.arange(1100)[None]).all()
        assert (got[:, raw:] >= raw).all()
        srt = np.take_along_axis(rk, got, 1)[:, :raw]
        assert (np.diff(srt, axis=1) >= -1e-4 * np.abs(srt[:, 1:]).clip(1)).all()
        assert (got[:, :raw] == ref_pos.reshape(12, -1)[:, :raw]).mean() > 0.99


@pytest.mark.parametrize("n_raw,block,heads,rounds", [(60000, 100, 8, 3), (6001, 64, 4, 2), (64, 64, 1, 1)])
def test_against_numpy_checker(lb, n_raw, block, heads, rounds):
    gen = torch.Generator().manual_seed(77 + n_raw)
    coords = torch.stack([torch.randn(n_raw, generator=gen) * 1.5,
                          (torch.rand(n_raw, generator=gen) * 2 - 1) * np.pi], -1)
    torch.manual_seed(5)
    regions = lb.get_regions(150, rounds, heads)
    dim = 6
    inp = lb.region_inputs(coords.cuda(), regions.cuda(), block)
    n = inp["coords"].shape[0]
    q = torch.zeros(heads, n, dim); q[:, :n_raw] = torch.randn(heads, n_raw, dim, generator=gen)
    k = torch.zeros(heads, n, dim); k[:, :n_raw] = torch.randn(heads, n_raw, dim, generator=gen)
    e2 = lb.E2LSH(n_hashes=rounds, n_heads=heads, dim=dim).cuda()
    # checker
    padded = np.full((n, 2), np.inf, np.float32); padded[:n_raw] = coords.numpy()
    se, sp = oracle.segsort(padded[:, 0]), oracle.segsort(padded[:, 1])
    regions_h = regions.numpy().transpose(1, 0, 2).reshape(2, -1)
    re, rp = oracle.quantile_regions(se, regions_h[0]), oracle.quantile_regions(sp, regions_h[1])
    np.testing.assert_array_equal(to_np(inp["region_indices"][0]), re)
    np.testing.assert_array_equal(to_np(inp["region_indices"][1]), rp)
    alpha = to_np(e2.alpha)
    qh, kh = oracle.e2lsh_proj(q.numpy(), alpha), oracle.e2lsh_proj(k.numpy(), alpha)
    np.testing.assert_array_equal(to_np(e2(q.cuda())), qh)            # frozen operation order: bit-exact
    hs = oracle.row_range(qh, kh)
    np.testing.assert_array_equal(to_np(lb.row_range(e2(q.cuda()), e2(k.cuda()))).reshape(-1), hs)
    shift = oracle.geo_shift(regions_h[0], hs, re, rp)
    qpos, kpos = lb.hept_positions(e2, q.cuda(), k.cuda(), inp["regions_h"], inp["ranks"], n_raw)
    for got, proj in ((qpos, qh), (kpos, kh)):
        keys = oracle.geo_keys(proj.reshape(-1, n), shift, n_raw)
        ref = np.stack([oracle.segsort(r) for r in keys])
        np.testing.assert_array_equal(to_np(got).reshape(-1, n), ref)
    # buckets never mix regions: the (phi, eta) region pair is non-decreasing along the order
    code = rp * (np.ceil(regions_h[0])[:, None] + 1) + re
    along = np.take_along_axis(code, to_np(qpos).reshape(-1, n), 1)[:, :n_raw]
    assert (np.diff(along, axis=1) >= 0).all()
