"""GPU parity of the HEPT bucket attention through the C ABI, against the float64 checker and the
reference-generated fixture.

Tolerance (fp32 kernel, float64 checker): |got - ref| <= 2e-5 * max(1, |ref|_inf) elementwise for
the weighted sums, relative 2e-5 for the denominators, 5e-5 for the quotient.  The exponent
q.k - |q|^2/2 - |k|^2/2 is a difference of terms of size |q|^2 ~ 10 in these inputs, so its fp32
rounding error (a few 1e-6 absolute) is the relative error of every weight.
The input preparation (one fp32 product per element) is compared exactly.
"""
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


def _c(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def _close(got, ref, rel, what):
    ref = np.asarray(ref, np.float64)
    err = np.abs(np.asarray(got, np.float64) - ref)
    bound = rel * np.maximum(1.0, np.abs(ref).max())
    assert np.isfinite(got).all(), f"{what}: non-finite"
    assert err.max() <= bound, f"{what}: max error {err.max():.3e} > {bound:.3e}"


def _close_rel(got, ref, rel, what):
    ref = np.asarray(ref, np.float64)
    err = np.abs(np.asarray(got, np.float64) - ref) / np.abs(ref)
    assert err.max() <= rel, f"{what}: max relative error {err.max():.3e}"


def test_fixture_from_reference(lb, golden_dir):
    z = np.load(os.path.join(golden_dir, "hept_bucket_attn.npz"))
    raw, block = int(z["raw_size"]), int(z["block_size"])
    q_hat, k_hat, v = lb.prep_qk(_c(z["query"]), _c(z["key"]), _c(z["w"]), _c(z["coords"]), value=_c(z["value"]),
                                 raw_size=raw, head_major=True)
    oq, ok = oracle.hept_prep_qk(z["query"], z["key"], z["w"], z["coords"], raw)
    np.testing.assert_allclose(to_np(q_hat), z["q_hat"], rtol=2e-6, atol=1e-7)   # torch's exp / sqrt on the scale
    np.testing.assert_allclose(to_np(k_hat), z["k_hat"], rtol=2e-6, atol=1e-7)
    np.testing.assert_allclose(to_np(q_hat), oq, rtol=2e-6, atol=1e-7)
    np.testing.assert_array_equal(to_np(v), z["v"])
    assert not to_np(q_hat)[:, raw:].any() and not to_np(v)[:, raw:].any()
    # reference layout of prep_qk
    q2, k2 = lb.prep_qk(_c(z["query"]), _c(z["key"]), _c(z["w"]), _c(z["coords"]))
    assert tuple(q2.shape) == (z["query"].shape[0], z["query"].shape[1], z["q_hat"].shape[-1])
    np.testing.assert_allclose(to_np(q2)[:raw], z["q_hat"].transpose(1, 0, 2)[:raw], rtol=2e-6, atol=1e-7)

    # qkv_res on the reference's sorted buckets
    C, H, N = z["q_pos"].shape
    sq = np.stack([np.stack([z["q_hat"][h][z["q_pos"][c, h]] for h in range(H)]) for c in range(C)])
    sk = np.stack([np.stack([z["k_hat"][h][z["k_pos"][c, h]] for h in range(H)]) for c in range(C)])
    sv = np.stack([np.stack([z["v"][h][z["k_pos"][c, h]] for h in range(H)]) for c in range(C)])
    shape = (C, H, N // block, block, -1)
    den, so = lb.qkv_res(_c(sq.reshape(shape)), _c(sk.reshape(shape)), _c(sv.reshape(shape)))
    assert tuple(den.shape) == z["denom"].shape and tuple(so.shape) == z["so"].shape
    _close_rel(to_np(den), z["denom"], 2e-5, "denom vs reference")
    _close(to_np(so), z["so"], 2e-5, "so vs reference")

    # fused gather + attention + scatter + combination
    out, o, lg = lb.hept_bucket_attention(_c(z["q_hat"]), _c(z["k_hat"]), _c(z["v"]), _c(z["q_pos"]), _c(z["k_pos"]),
                                          block, return_parts=True)
    _close(to_np(o), z["o"], 2e-5, "o vs reference")
    _close_rel(to_np(lg), z["logits"], 2e-5, "logits vs reference")
    _close(to_np(out), z["out"], 5e-5, "out vs reference")
    # the same from the padded rows that prep_qk returns (16-byte gather path): identical arithmetic
    assert q_hat.stride(1) % 4 == 0 and q_hat.stride(1) >= q_hat.shape[-1]
    out_p = lb.hept_bucket_attention(q_hat, k_hat, v, _c(z["q_pos"]), _c(z["k_pos"]), block)
    _close(to_np(out_p), z["out"], 5e-5, "out from padded rows vs reference")
    ref_out, ref_o, ref_lg = oracle.hept_bucket_attention(z["q_hat"], z["k_hat"], z["v"], z["q_pos"], z["k_pos"], block)
    _close(to_np(o), ref_o, 2e-5, "o vs checker")
    _close_rel(to_np(lg), ref_lg, 2e-5, "logits vs checker")
    _close(to_np(out), ref_out, 5e-5, "out vs checker")


CASES = [
    # N, block, heads, rounds, dq, dv
    (128, 128, 1, 1, 4, 4),
    (300, 100, 2, 3, 30, 24),       # the transformer config: h_dim 24 + 6 coordinates
    (400, 100, 2, 2, 102, 96),      # h_dim 96 + 6 coordinates
    (96, 32, 3, 2, 7, 5),           # odd dims: scalar stores, padded feature groups
    (64, 1, 1, 2, 9, 3),            # buckets of one hit
    (130, 65, 2, 1, 33, 128),       # widest value row
    (77 * 3, 77, 1, 3, 16, 17),
]


@pytest.mark.parametrize("N,block,H,C,dq,dv", CASES)
def test_random_cases_against_checker(lb, N, block, H, C, dq, dv):
    rng = np.random.default_rng(N * 7 + dq)
    q = (rng.standard_normal((H, N, dq)) * (2.0 / np.sqrt(dq))).astype(np.float32)
    k = (q + rng.standard_normal((H, N, dq)) * (1.0 / np.sqrt(dq))).astype(np.float32)
    v = rng.standard_normal((H, N, dv)).astype(np.float32)
    qp = np.stack([np.stack([rng.permutation(N) for _ in range(H)]) for _ in range(C)]).astype(np.int64)
    kp = np.stack([np.stack([rng.permutation(N) for _ in range(H)]) for _ in range(C)]).astype(np.int64)
    out, o, lg = lb.hept_bucket_attention(_c(q), _c(k), _c(v), _c(qp), _c(kp), block, return_parts=True)
    ref_out, ref_o, ref_lg = oracle.hept_bucket_attention(q, k, v, qp, kp, block)
    _close(to_np(o), ref_o, 2e-5, "o")
    _close_rel(to_np(lg), ref_lg, 2e-5, "logits")
    _close(to_np(out), ref_out, 5e-5, "out")
    # sorted-layout entry on the same data equals the scattered one
    sq = np.stack([np.stack([q[h][qp[c, h]] for h in range(H)]) for c in range(C)]).reshape(C, H, N // block, block, dq)
    sk = np.stack([np.stack([k[h][kp[c, h]] for h in range(H)]) for c in range(C)]).reshape(C, H, N // block, block, dq)
    sv = np.stack([np.stack([v[h][kp[c, h]] for h in range(H)]) for c in range(C)]).reshape(C, H, N // block, block, dv)
    den, so = lb.qkv_res(_c(sq), _c(sk), _c(sv))
    so_np, o_np = to_np(so).reshape(C, H, N, dv), to_np(o)
    for c in range(C):
        for h in range(H):
            np.testing.assert_array_equal(o_np[c, h][qp[c, h]], so_np[c, h])
            np.testing.assert_array_equal(to_np(lg)[c, h][qp[c, h]], to_np(den).reshape(C, H, N, 1)[c, h])


def test_slices_of_wider_storage_are_not_read_past_their_width(lb):
    """q_hat / k_hat given as [..., :30] slices of 32-wide rows whose last two columns hold other
    data: the result must be that of the 30 columns alone (the 16-byte row fetch would fold the
    extra columns into q.k and the norms if such a view were read in place)."""
    rng = np.random.default_rng(5)
    H, N, dq, dv, block, C = 2, 400, 30, 24, 100, 2
    wide_q = (rng.standard_normal((H, N, 32)) * 0.4).astype(np.float32)
    wide_k = (wide_q + rng.standard_normal((H, N, 32)) * 0.2).astype(np.float32)
    v = rng.standard_normal((H, N, dv)).astype(np.float32)
    qp = np.stack([np.stack([rng.permutation(N) for _ in range(H)]) for _ in range(C)]).astype(np.int64)
    kp = np.stack([np.stack([rng.permutation(N) for _ in range(H)]) for _ in range(C)]).astype(np.int64)
    out = lb.hept_bucket_attention(_c(wide_q)[..., :dq], _c(wide_k)[..., :dq], _c(v), _c(qp), _c(kp), block)
    ref_out, _, _ = oracle.hept_bucket_attention(np.ascontiguousarray(wide_q[..., :dq]),
                                                 np.ascontiguousarray(wide_k[..., :dq]), v, qp, kp, block)
    _close(to_np(out), ref_out, 5e-5, "out (sliced rows)")


def test_identical_points_and_far_points(lb):
    """All hits of a bucket equal: every weight is 1 (clamp at 0), so = bucket * v, denom = bucket.
    Hits far apart: off-diagonal weights underflow to 0 and each hit sees only itself."""
    N, block, dq, dv = 200, 100, 8, 4
    q = np.tile(np.linspace(-1, 1, dq, dtype=np.float32), (1, N, 1))
    v = np.ones((1, N, dv), np.float32)
    pos = np.arange(N, dtype=np.int64).reshape(1, 1, N)
    out, o, lg = lb.hept_bucket_attention(_c(q), _c(q), _c(v), _c(pos), _c(pos), block, return_parts=True)
    np.testing.assert_allclose(to_np(lg), block, rtol=1e-6)
    np.testing.assert_allclose(to_np(o), block, rtol=1e-6)
    np.testing.assert_allclose(to_np(out), 1.0, rtol=1e-6)
    far = (np.arange(N, dtype=np.float32)[None, :, None] * 10.0) * np.ones((1, 1, dq), np.float32)
    vv = np.arange(N * dv, dtype=np.float32).reshape(1, N, dv)
    out = lb.hept_bucket_attention(_c(far), _c(far), _c(vv), _c(pos), _c(pos), block)
    got = to_np(out)
    assert np.isfinite(got).all()
    # rounding of the exponent can leave the self-weight below 1 at |q|^2 ~ 3e7; the quotient does not see it
    np.testing.assert_allclose(got, vv, rtol=1e-6)


def test_attention_core_end_to_end(lb):
    """The layer's forward between the projections and the output projection: input preparation, region
    shift, bucket orders and attention in one call, against the checker run on the positions the call
    itself produced (the positions have their own parity tests)."""
    raw, block, heads, rounds, d, cd, nw = 1130, 100, 4, 3, 24, 6, 5
    gen = torch.Generator().manual_seed(99)
    coords_raw = torch.randn(raw, cd, generator=gen)
    coords_raw[:, 1] = (torch.rand(raw, generator=gen) * 2 - 1) * 3.14159
    w = torch.randn(heads, d, cd - 1, nw, generator=gen) * 0.3 - 0.8
    torch.manual_seed(5)
    regions = lb.get_regions(40, rounds, heads)
    e2lsh = lb.E2LSH(n_hashes=rounds, n_heads=heads, dim=d + cd).cuda()
    inp = lb.region_inputs(coords_raw.cuda(), regions, block)
    n = inp["coords"].shape[0]
    assert n == 1200
    query = lb.pad_to_multiple(torch.randn(raw, heads, d, generator=gen) * 0.6, block, dims=0).cuda()
    key = lb.pad_to_multiple(torch.randn(raw, heads, d, generator=gen) * 0.6, block, dims=0).cuda()
    value = lb.pad_to_multiple(torch.randn(raw, heads, d, generator=gen), block, dims=0).cuda()
    out = lb.hept_attention_core(e2lsh, query, key, value, w.cuda(), inp["coords"], inp["regions_h"], inp["ranks"],
                                 raw, block)
    assert tuple(out.shape) == (heads, n, d)
    q_hat, k_hat, v = lb.prep_qk(query, key, w.cuda(), inp["coords"], value=value, raw_size=raw, head_major=True)
    oq, ok = oracle.hept_prep_qk(to_np(query), to_np(key), w.numpy(), to_np(inp["coords"]), raw)
    np.testing.assert_allclose(to_np(q_hat), oq, rtol=2e-6, atol=1e-7)
    np.testing.assert_allclose(to_np(k_hat), ok, rtol=2e-6, atol=1e-7)
    q_pos, k_pos = lb.hept_positions(e2lsh, q_hat, k_hat, inp["regions_h"], inp["ranks"], raw)
    # projections read in place from the padded rows equal those of a dense copy
    q_pos_c, _ = lb.hept_positions(e2lsh, q_hat.contiguous(), k_hat.contiguous(), inp["regions_h"], inp["ranks"], raw)
    np.testing.assert_array_equal(to_np(q_pos), to_np(q_pos_c))
    for p in (q_pos, k_pos):
        assert (np.sort(to_np(p), axis=-1) == np.arange(n)).all()
    ref_out, _, _ = oracle.hept_bucket_attention(to_np(q_hat), to_np(k_hat), to_np(v), to_np(q_pos), to_np(k_pos), block)
    _close(to_np(out)[:, :raw], ref_out[:, :raw], 5e-5, "attention core")


def test_argument_errors(lb):
    q = torch.zeros(1, 100, 8, device="cuda")
    v = torch.zeros(1, 100, 4, device="cuda")
    pos = torch.arange(100, device="cuda").view(1, 1, 100)
    with pytest.raises(ValueError):
        lb.hept_bucket_attention(q, q, v, pos, pos, 30)            # N not a multiple of the bucket
    with pytest.raises(ValueError):
        lb.hept_bucket_attention(q, q, v, pos[:, :, :50], pos, 50)
    with pytest.raises(TypeError):
        lb.hept_bucket_attention(q.half(), q.half(), v, pos, pos, 50)
    big = torch.zeros(1, 1, 256, 8, device="cuda")
    with pytest.raises(lb.LampaError):
        lb.qkv_res(big, big, big)                                  # bucket of 256 > 128
