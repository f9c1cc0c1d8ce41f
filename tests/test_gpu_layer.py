"""GPU parity of the layer's producers / consumers (short convolution, gate inputs, gated RMS
norm) through the C ABI, against the numpy checker and the reference-generated fixture.

Tolerance: fp32 storage 1e-5 (relative + absolute; the kernels use the fast exp); bf16 storage:
one bf16 ulp of the fp32 result (2^-8 relative) plus 1e-3 absolute.
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
    return lampa_b200


def _c(x, dt=None):
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t if dt is None else t.to(dt)


def _close(got, ref, bf16=False, what=""):
    got = np.asarray(got, np.float32)
    if bf16:
        np.testing.assert_allclose(got, ref, rtol=2 ** -7, atol=2e-3, err_msg=what)
    else:
        np.testing.assert_allclose(got, ref, rtol=1e-5, atol=1e-5, err_msg=what)


def _conv(lb, z, dtype=torch.float32, bias=True):
    from lampa_b200.layer import ShortConvolution
    D, _, W = z["conv_w"].shape
    conv = ShortConvolution(D, W, bias=bias, activation="silu").cuda()
    conv.weight.data.copy_(_c(z["conv_w"]))
    if bias:
        conv.bias.data.copy_(_c(z["conv_b"]))
    return conv.to(dtype)


def test_fixture_from_reference(lb, golden_dir):
    from lampa_b200.layer import FusedRMSNormGated, compute_lambda, gate_inputs
    z = np.load(os.path.join(golden_dir, "layer_ops.npz"))
    g, beta, lam = gate_inputs(_c(z["a"]), _c(z["b"]), _c(z["dl"]), _c(z["A_log"]), _c(z["dt_bias"]), _c(z["L"]), "positive")
    assert g.dtype == torch.float32
    _close(to_np(g), z["g"], what="g"); _close(to_np(beta), z["beta"], what="beta"); _close(to_np(lam), z["lam_positive"], what="lambda")
    for mode, key in (("bounded", "lam_bounded"), (None, "lam_default")):
        _close(to_np(compute_lambda(_c(z["L"])[None, None], _c(z["dl"]), mode)), z[key], what=key)
    conv = _conv(lb, z)
    y, cache = conv(_c(z["x"]), residual=_c(z["res"]), output_final_state=True)
    _close(to_np(y), z["y"], what="conv"); np.testing.assert_array_equal(to_np(cache), z["cache"])
    yp, cp = conv(_c(z["x"][:1]), cu_seqlens=_c(z["cu"]), output_final_state=True)
    _close(to_np(yp), z["y_packed"], what="conv packed")
    np.testing.assert_array_equal(to_np(cp), oracle.short_conv_state(z["x"][:1], 4, z["cu"]))
    ys, cs = conv(_c(z["x_step"]), cache=cache)                      # one token per row: the decode step
    assert cs is cache
    _close(to_np(ys), z["y_step"], what="conv step"); np.testing.assert_array_equal(to_np(cache), z["cache_step"])
    norm = FusedRMSNormGated(z["norm_w"].shape[0], eps=1e-5).cuda()
    norm.weight.data.copy_(_c(z["norm_w"]))
    _close(to_np(norm(_c(z["norm_x"]), _c(z["norm_g"]))), z["norm_y"], what="norm")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_conv_sizes_and_types(lb, dtype):
    from lampa_b200.layer import ShortConvolution
    gen = torch.Generator().manual_seed(5)
    for (B, T, D, W, bias) in [(1, 1000, 512, 4, False), (3, 17, 64, 2, True), (2, 300, 1024, 8, True), (1, 5, 8, 4, False)]:
        conv = ShortConvolution(D, W, bias=bias).cuda().to(dtype)
        x = torch.randn(B, T, D, generator=gen).to(dtype)
        res = torch.randn(B, T, D, generator=gen).to(dtype)
        w = to_np(conv.weight.float().reshape(D, W)); b = None if not bias else to_np(conv.bias.float())
        y, st = conv(x.cuda(), residual=res.cuda(), output_final_state=True)
        assert y.dtype == dtype and tuple(st.shape) == (B, D, W)
        _close(to_np(y.float()), oracle.short_conv(to_np(x.float()), w, b, to_np(res.float())), dtype != torch.float32, f"{B},{T},{D},{W}")
        np.testing.assert_array_equal(to_np(st.float()), oracle.short_conv_state(to_np(x.float()), W))
    # packed with empty and one-token sequences; state of short sequences is zero-filled
    lens = [40, 0, 1, 3, 700, 16, 17]
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    conv = ShortConvolution(256, 4).cuda().to(dtype)
    x = torch.randn(1, int(cu[-1]), 256, generator=gen).to(dtype)
    y, st = conv(x.cuda(), cu_seqlens=torch.from_numpy(cu).cuda(), output_final_state=True)
    w = to_np(conv.weight.float().reshape(256, 4))
    _close(to_np(y.float()), oracle.short_conv(to_np(x.float()), w, cu=cu), dtype != torch.float32, "packed")
    np.testing.assert_array_equal(to_np(st.float()), oracle.short_conv_state(to_np(x.float()), 4, cu))


def test_conv_prefill_then_steps_equals_one_pass(lb):
    from lampa_b200.layer import ShortConvolution
    gen = torch.Generator().manual_seed(6)
    B, T, D, W = 2, 50, 128, 4
    conv = ShortConvolution(D, W, bias=True).cuda()
    x = torch.randn(B, T + 5, D, generator=gen).cuda()
    full, _ = conv(x)
    y0, cache = conv(x[:, :T].contiguous(), output_final_state=True)
    outs = [y0]
    for t in range(T, T + 5):
        yt, cache = conv(x[:, t:t + 1].contiguous(), cache=cache)
        outs.append(yt)
    _close(to_np(torch.cat(outs, 1)), to_np(full), what="prefill + decode")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_gates_and_norm_sizes(lb, dtype):
    from lampa_b200.layer import gate_inputs, rms_norm_gated
    gen = torch.Generator().manual_seed(8)
    B, T, H, Lv, Dv = 2, 333, 8, 17, 128
    a, b = torch.randn(B, T, H, generator=gen).to(dtype), torch.randn(B, T, H, generator=gen).to(dtype)
    dl = (3 * torch.randn(B, T, H * Lv, generator=gen)).to(dtype)
    A_log, dtb, Lp = torch.randn(H, generator=gen), torch.randn(H, generator=gen), 1 + torch.randn(H, Lv, generator=gen)
    mask = (torch.rand(B, T, generator=gen) > 0.2).float()
    g, beta, lam = gate_inputs(a.cuda(), b.cuda(), dl.cuda(), A_log.cuda(), dtb.cuda(), Lp.cuda(), "positive", attention_mask=mask.cuda())
    rg, rb, rl = oracle.gate_inputs(to_np(a.float()), to_np(b.float()), to_np(dl.float()).reshape(B, T, H, Lv), to_np(A_log), to_np(dtb), to_np(Lp))
    m = to_np(mask)
    _close(to_np(g), rg * m[..., None], what="g")
    _close(to_np(beta.float()), rb * m[..., None], dtype != torch.float32, "beta")
    _close(to_np(lam.float()), rl * m[..., None, None], dtype != torch.float32, "lambda")
    assert beta.dtype == dtype and lam.dtype == dtype and tuple(lam.shape) == (B, T, H, Lv)
    for D in (64, 128, 512):
        x, gg = (2 * torch.randn(B, T, H, D, generator=gen)).to(dtype), torch.randn(B, T, H, D, generator=gen).to(dtype)
        w = (1 + 0.1 * torch.randn(D, generator=gen))
        for act in ("swish", "sigmoid"):
            y = rms_norm_gated(x.cuda(), gg.cuda(), w.cuda(), None, act, eps=1e-5)
            ref = oracle.rmsnorm_gate(to_np(x.float()), to_np(gg.float()), to_np(w), 1e-5, act == "sigmoid")
            _close(to_np(y.float()), ref, dtype != torch.float32, f"norm {D} {act}")


def test_layer_chain_feeds_the_mixer(lb):
    """conv -> gates -> hierarchical op -> gated norm, as HGatedDeltaNet.forward chains them."""
    from lampa_b200 import synth
    from lampa_b200.layer import FusedRMSNormGated, ShortConvolution, gate_inputs
    gen = torch.Generator().manual_seed(9)
    B, T, H, K, V = 1, 256, 2, 64, 64
    Lv = lb.num_levels_required(T)
    dt = torch.bfloat16
    convs = [ShortConvolution(H * K, 4).cuda().to(dt) for _ in range(3)]
    proj = [torch.randn(B, T, H * K, generator=gen).to(dt).cuda() for _ in range(3)]
    q, k, v = (c(p)[0].view(B, T, H, K) for c, p in zip(convs, proj))
    a, b = torch.randn(B, T, H, generator=gen).to(dt).cuda(), torch.randn(B, T, H, generator=gen).to(dt).cuda()
    dl = torch.randn(B, T, H * Lv, generator=gen).to(dt).cuda()
    A_log, dtb, Lp = torch.zeros(H).cuda(), torch.zeros(H).cuda(), torch.ones(H, Lv).cuda()
    g, beta, lam = gate_inputs(a, b, dl, A_log, dtb, Lp, "positive")
    o, _ = lb.chunk_h_gated_delta_rule(q, k, v, g, lam, beta, use_qk_l2norm_in_kernel=True)
    gate = torch.randn(B, T, H, V, generator=gen).to(dt).cuda()
    y = FusedRMSNormGated(V).cuda().to(dt)(o, gate)
    oref = oracle.hgdn(to_np(q[0].float()), to_np(k[0].float()), to_np(v[0].float()), to_np(g[0]), to_np(beta[0].float()),
                       to_np(lam[0].float()), use_l2norm=True)[0]
    yref = oracle.rmsnorm_gate(oref, to_np(gate[0].float()), None, 1e-5)
    err = np.linalg.norm(to_np(y[0].float()) - yref) / np.linalg.norm(yref)
    assert err < 2e-2, err


@pytest.mark.parametrize("D,dt", [(128, torch.bfloat16), (96, torch.float16), (256, torch.float32), (520, torch.bfloat16)])
def test_add_rms_norm_with_and_without_permutation(lb, D, dt):
    """Fused residual add + RMS norm + row permutation against the plain statements
    (rms_norm_ref of models/hattention/fused_norm.py:1313-1330 with residual, prenorm=True)."""
    gen = torch.Generator().manual_seed(D)
    lens = [37, 0, 64, 211]
    rows = sum(lens)
    cu = torch.tensor([0] + lens).cumsum(0)
    res = torch.randn(rows, D, generator=gen)
    delta = torch.randn(rows, D, generator=gen).to(dt)
    w = torch.rand(D, generator=gen) + 0.5
    perm = torch.cat([torch.randperm(n, generator=gen) for n in lens])           # local to each segment
    glob = torch.cat([perm[cu[i]:cu[i + 1]] + cu[i] for i in range(len(lens))])   # r for every j

    def norm(v):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-6) * w

    tol = 1e-5 if dt == torch.float32 else 8e-3
    # norm only, gathered: y[j] = norm(res[r])
    r0 = res.clone().cuda()
    y = lb.add_rms_norm(r0, None, w.cuda(), 1e-6, perm=perm.cuda(), seg_offsets=cu, out_dtype=dt)
    assert torch.equal(r0.cpu(), res)
    torch.testing.assert_close(y.float().cpu(), norm(res[glob]).to(dt).float(), rtol=tol, atol=tol)
    # delta in the other order, result in row order: res[r] += delta[j]; y[r] = norm(res[r])
    r1 = res.clone().cuda()
    y = lb.add_rms_norm(r1, delta.cuda(), w.cuda(), 1e-6, perm=perm.cuda(), seg_offsets=cu, y_at_r=True, out_dtype=dt)
    want = res.clone()
    want[glob] += delta.float()
    torch.testing.assert_close(r1.cpu(), want, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(y.float().cpu(), norm(want).to(dt).float(), rtol=tol, atol=tol)
    # delta in row order, result gathered: res[r] += delta[r]; y[j] = norm(res[r])
    r2 = res.clone().cuda()
    y = lb.add_rms_norm(r2, delta.cuda(), w.cuda(), 1e-6, perm=perm.cuda(), seg_offsets=cu, delta_at_r=True, out_dtype=dt)
    want = res + delta.float()
    torch.testing.assert_close(r2.cpu(), want, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(y.float().cpu(), norm(want)[glob].to(dt).float(), rtol=tol, atol=tol)
    # add only, no permutation
    r3 = res.clone().cuda()
    assert lb.add_rms_norm(r3, delta.cuda(), None, out_dtype=None) is None
    torch.testing.assert_close(r3.cpu(), want, rtol=1e-6, atol=1e-6)
