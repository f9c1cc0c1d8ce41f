"""The CPU oracle against fixtures produced by the reference's own pure-PyTorch code.

Fixtures: tests/golden/*.npz (made by tests/golden/gen_golden.py from
models/hattention/recurrent.py, models/baselines/hmamba.py, models/attention/hept.py,
models/model_utils/hash_utils.py).
"""
import glob
import os

import numpy as np
import pytest

from oracle import oracle


def _cases(golden_dir):
    return sorted(glob.glob(os.path.join(golden_dir, "hgdn_*.npz")))


@pytest.mark.parametrize("name", ["hgdn_T200_H2_K16_V32_L9", "hgdn_T320_H2_K32_V32_L10",
                                  "hgdn_T256_H1_K64_V64_L9"])
def test_hier_and_plain_match_reference_recurrence(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    o, states, counts = oracle.hgdn(z["q"], z["k"], z["v"], z["g"], z["beta"], z["lam"], use_l2norm=False)
    np.testing.assert_allclose(o, z["o_hier"], rtol=2e-4, atol=2e-5)
    np.testing.assert_allclose(states, z["states_hier"], rtol=2e-4, atol=2e-5)
    assert (counts == z["counts_hier"]).all()
    op, ht = oracle.gdn_plain(z["q"], z["k"], z["v"], z["g"], z["beta"], scale=float(z["scale"]))
    np.testing.assert_allclose(op, z["o_plain"], rtol=2e-4, atol=2e-5)
    np.testing.assert_allclose(ht[0], z["final_plain"], rtol=2e-4, atol=2e-5)


def test_hier_matches_reference_chunkwise_statement(golden_dir):
    """Second pin: the reference's own chunkwise statement (hgdn_minimal, hssd_minimal.py:462-493)
    at T = 4096 -- 64 chunks, two blocks of 32, one cross-block level -- against the token
    recurrence of the checker, both fp32."""
    from tests.util import minimal_fixture_inputs
    z = np.load(os.path.join(golden_dir, "hgdn_minimal_T4096_H2_K32_V32_L13.npz"))
    q, k, v, beta, g, lam = (x.numpy() for x in minimal_fixture_inputs(z))
    o, _, _ = oracle.hgdn(q, k, v, g, beta, lam, use_l2norm=False)
    ref = z["o_hier"]
    err = np.abs(o - ref).max()
    rel = np.linalg.norm(o - ref) / np.linalg.norm(ref)
    assert err <= 5e-5 * max(1.0, np.abs(ref).max()) and rel <= 2e-5, (err, rel)


def test_level_function_is_bit_length_of_xor(golden_dir):
    lv = np.load(os.path.join(golden_dir, "levels_weak_130.npz"))["levels"]
    t = np.arange(130)[:, None]
    s = np.arange(130)[None, :]
    mine = np.where(s < t, np.floor(np.log2(np.maximum(t ^ s, 1))).astype(int) + 1, 0)
    assert (mine == lv).all()


def test_plain_initial_state_and_varlen_consistency():
    rng = np.random.default_rng(0)
    T, H, K, V = 150, 2, 16, 16
    q, k = rng.standard_normal((2, T, H, K)).astype(np.float32)
    v = rng.standard_normal((T, H, V)).astype(np.float32)
    g = -np.abs(rng.standard_normal((T, H))).astype(np.float32) * 0.1
    b = rng.uniform(0, 1, (T, H)).astype(np.float32)
    h0 = rng.standard_normal((1, H, K, V)).astype(np.float32) * 0.1
    o_full, ht_full = oracle.gdn_plain(q, k, v, g, b, h0=h0, use_l2norm=True)
    # running the two halves with state hand-over equals the full run
    o_a, ht_a = oracle.gdn_plain(q[:70], k[:70], v[:70], g[:70], b[:70], h0=h0, use_l2norm=True)
    o_b, ht_b = oracle.gdn_plain(q[70:], k[70:], v[70:], g[70:], b[70:], h0=ht_a, use_l2norm=True)
    np.testing.assert_allclose(np.concatenate([o_a, o_b]), o_full, rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(ht_b, ht_full, rtol=1e-6, atol=1e-6)
    # packed varlen == separate calls
    cu = np.array([0, 70, 150])
    h02 = np.concatenate([h0, h0 * 2])
    o_v, ht_v = oracle.gdn_plain(q, k, v, g, b, h0=h02, cu_seqlens=cu, use_l2norm=True)
    o_c, ht_c = oracle.gdn_plain(q[70:], k[70:], v[70:], g[70:], b[70:], h0=h0 * 2, use_l2norm=True)
    np.testing.assert_array_equal(o_v[:70], o_a)
    np.testing.assert_array_equal(o_v[70:], o_c)
    np.testing.assert_array_equal(ht_v[1], ht_c[0])


def test_lsh_ordering_matches_reference(golden_dir):
    z = np.load(os.path.join(golden_dir, "lsh_ordering_B2_L1500.npz"))
    coords, points, alpha = z["coords"], z["points"], z["alpha"]
    Bn, Ln, _ = coords.shape
    # E2LSH float projection (hmamba.py:275-285): [n_hashes, N, 1]
    flat = coords.reshape(Bn * Ln, -1)
    _, keys = oracle.lsh_ids(flat, alpha, np.zeros(3, np.float32), want_keys=True)
    ref_proj = z["proj"][:, :, 0]                      # [3, N]
    np.testing.assert_allclose(keys[:, 0, :], ref_proj, rtol=1e-5, atol=1e-3)
    for b in range(Bn):
        perm = oracle.lsh_ordering(coords[b], alpha)
        ref = z["indices"][b]
        agree = (perm == ref).mean()
        # float re-association near-ties may swap a handful of neighbours
        assert agree > 0.99, agree
        key = oracle.lsh_ordering_keys(coords[b], alpha)
        assert (np.diff(key[perm]) >= 0).all()
        # same multiset, and the reference's permutation is sorted under our key up to rounding
        assert (np.sort(perm) == np.arange(Ln)).all()
        assert (np.diff(key[ref]) >= -1e-3 * np.abs(key).max()).all()
        ordered = oracle.permute_rows(points[b], ref)
        np.testing.assert_array_equal(ordered, z["ordered"][b])
        inv = oracle.invert_perm(ref)
        np.testing.assert_array_equal(inv, z["inverse"][b])
        np.testing.assert_array_equal(oracle.permute_rows(ordered, inv), points[b])
    # sort_to_buckets == row gather reshaped (hept.py:9-14)
    np.testing.assert_array_equal(z["buckets"][0].reshape(Bn, Ln, -1), z["ordered"])


def test_integer_ids_and_stable_sort_properties():
    rng = np.random.default_rng(3)
    N = 5000
    x = rng.standard_normal((N, 24)).astype(np.float32) * 100
    alpha = rng.standard_normal((8, 6, 3)).astype(np.float32)
    beta = rng.uniform(0, 1, 3).astype(np.float32)
    ids = oracle.lsh_ids(x, alpha, beta, w=1.0)
    assert ids.shape == (3, 8, N) and ids.dtype == np.int32
    # numpy restatement with separately rounded multiply/add
    acc = x[:, 0, None, None] * alpha[None, :, 0, :]
    for d in range(1, 6):
        acc = acc + x[:, d, None, None] * alpha[None, :, d, :]
    ref = np.floor((acc + beta[None, None, :]) / np.float32(1.0)).astype(np.int32)   # [N, heads, rounds]
    np.testing.assert_array_equal(ids, ref.transpose(2, 1, 0))
    row = np.ascontiguousarray(ids[1, 3])
    perm = oracle.segsort(row)
    np.testing.assert_array_equal(perm, np.argsort(row, kind="stable"))
    seg = np.array([0, 100, 100, 3000, N])
    perm_s = oracle.segsort(row, seg)
    for a, b in zip(seg[:-1], seg[1:]):
        np.testing.assert_array_equal(perm_s[a:b], np.argsort(row[a:b], kind="stable"))


def test_geo_shift_against_reference_fixture(golden_dir):
    """quantile_partition / get_geo_shift / lsh_mapping of the reference (tests/golden/gen_golden.py)."""
    z = np.load(os.path.join(golden_dir, "geo_shift_N1090_R12.npz"))
    regions = z["regions"]                                     # [c, a, h]
    regions_h = regions.transpose(1, 0, 2).reshape(2, -1)      # "c a h -> a (c h)"
    re = oracle.quantile_regions(z["sorted_eta"], regions_h[0])
    rp = oracle.quantile_regions(z["sorted_phi"], regions_h[1])
    np.testing.assert_array_equal(re, z["reg_eta"])
    np.testing.assert_array_equal(rp, z["reg_phi"])
    raw = int(z["raw_size"])
    qh = z["q_hashed"].copy(); kh = z["k_hashed"].copy()
    qh[..., raw:] = 0.0; kh[..., raw:] = 0.0                   # padded rows project to 0 before the +inf
    np.testing.assert_array_equal(oracle.row_range(qh, kh), z["hash_shift"].reshape(-1))
    shift = oracle.geo_shift(regions_h[0], z["hash_shift"], re, rp)
    np.testing.assert_array_equal(shift, z["q_shift"].reshape(shift.shape))
    np.testing.assert_array_equal(shift, z["k_shift"].reshape(shift.shape))
    keys = oracle.geo_keys(qh, shift, raw)
    np.testing.assert_array_equal(keys, z["q_keys"].reshape(keys.shape))
    # projections: same numbers as the reference's bmm up to summation order
    proj = oracle.e2lsh_proj(z["q_hat"], z["alpha"])
    np.testing.assert_allclose(proj[..., :raw], z["q_hashed"][..., :raw], rtol=1e-5, atol=1e-5)
    # stable sort of the reference keys reproduces the reference positions on the real hits
    # (equal keys may come out in either order from the reference's non-stable argsort)
    kq = z["q_keys"].reshape(-1, keys.shape[-1])
    pos = np.stack([oracle.segsort(r) for r in kq])
    ref_pos = z["q_pos"].reshape(pos.shape)
    differ = pos[:, :raw] != ref_pos[:, :raw]
    assert differ.mean() < 1e-3
    np.testing.assert_array_equal(np.take_along_axis(kq, pos, 1)[:, :raw], np.take_along_axis(kq, ref_pos, 1)[:, :raw])


def test_layer_ops_against_reference_fixture(golden_dir):
    """compute_lambda, the g/beta expressions, ShortConvolution and the gated RMS norm of the
    reference (tests/golden/gen_golden.py::gen_layer)."""
    z = np.load(os.path.join(golden_dir, "layer_ops.npz"))
    for mode, key in (("positive", "lam_positive"), ("bounded", "lam_bounded"), (None, "lam_default")):
        g, beta, lam = oracle.gate_inputs(z["a"], z["b"], z["dl"], z["A_log"], z["dt_bias"], z["L"], mode)
        np.testing.assert_allclose(lam, z[key], rtol=2e-6, atol=1e-6)
    np.testing.assert_allclose(g, z["g"], rtol=2e-6, atol=1e-6)
    np.testing.assert_allclose(beta, z["beta"], rtol=2e-6, atol=1e-6)
    w = z["conv_w"][:, 0]
    np.testing.assert_allclose(oracle.short_conv(z["x"], w, z["conv_b"], z["res"]), z["y"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(oracle.short_conv(z["x"][:1], w, z["conv_b"], cu=z["cu"]), z["y_packed"], rtol=1e-5, atol=1e-5)
    np.testing.assert_array_equal(oracle.short_conv_state(z["x"], 4), z["cache"])
    ys, cs = oracle.short_conv_step(z["x_step"][:, 0], z["cache"], w, z["conv_b"])
    np.testing.assert_allclose(ys, z["y_step"][:, 0], rtol=1e-5, atol=1e-5)
    np.testing.assert_array_equal(cs, z["cache_step"])
    np.testing.assert_allclose(oracle.rmsnorm_gate(z["norm_x"], z["norm_g"], z["norm_w"], 1e-5), z["norm_y"],
                               rtol=1e-5, atol=1e-5)


def test_bucket_attention_against_reference_fixture(golden_dir):
    """The float64 restatement of the HEPT bucket attention against the reference's fp32 run."""
    z = np.load(os.path.join(golden_dir, "hept_bucket_attn.npz"))
    raw, block = int(z["raw_size"]), int(z["block_size"])
    q_hat, k_hat = oracle.hept_prep_qk(z["query"], z["key"], z["w"], z["coords"], raw)
    np.testing.assert_allclose(q_hat, z["q_hat"], rtol=2e-6, atol=1e-7)
    np.testing.assert_allclose(k_hat, z["k_hat"], rtol=2e-6, atol=1e-7)
    C, H, N = z["q_pos"].shape
    sq = np.stack([np.stack([z["q_hat"][h][z["q_pos"][c, h]] for h in range(H)]) for c in range(C)])
    sk = np.stack([np.stack([z["k_hat"][h][z["k_pos"][c, h]] for h in range(H)]) for c in range(C)])
    sv = np.stack([np.stack([z["v"][h][z["k_pos"][c, h]] for h in range(H)]) for c in range(C)])
    shape = (C, H, N // block, block, -1)
    den, so = oracle.qkv_res(sq.reshape(shape), sk.reshape(shape), sv.reshape(shape))
    np.testing.assert_allclose(den, z["denom"], rtol=2e-5)
    np.testing.assert_allclose(so, z["so"], rtol=2e-5, atol=2e-5)
    out, o, lg = oracle.hept_bucket_attention(z["q_hat"], z["k_hat"], z["v"], z["q_pos"], z["k_pos"], block)
    np.testing.assert_allclose(o, z["o"], rtol=2e-5, atol=2e-5)
    np.testing.assert_allclose(lg, z["logits"], rtol=2e-5)
    np.testing.assert_allclose(out, z["out"], rtol=5e-5, atol=2e-5)
