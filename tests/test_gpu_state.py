"""GPU parity of the hierarchical rule's Fenwick state (prefill final state and decode step),
through the C ABI, against the CPU checker's token recurrence.

Outputs: the bf16 tolerance of the forward tests (tests/util.assert_close_bf16).
States: the whole tensor [H, K, V, L] within max-abs 2e-2 of its largest value and relative L2
1e-2, and every level on its own within the same two figures after rescaling by
max(level's largest value, 1e-3 of the tensor's largest value).  The floor is there because a level
that has been carried across many chunks is attenuated far below the others (each chunk applies 64
rank-one contractions in a 64-dimensional space; after 32 chunks nothing measurable is left in
these inputs): below a thousandth of the tensor's scale its own relative accuracy says nothing
about the state, and what is compared there is its absolute contribution.
Counts are compared exactly.
"""
import os

import numpy as np
import pytest
import torch

from oracle import oracle
from tests.util import assert_close_bf16, err_stats, to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lb():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import lampa_b200
    os.environ["LAMPA_B200_CHECK"] = "1"
    return lampa_b200


def _cuda(d):
    return {k: v.to("cuda:0") for k, v in d.items()}


def _close_level(got, ref, what, floor):
    """One level against the checker, rescaled first (strongly decayed levels sit near 1e-30,
    where squaring for the L2 norm would underflow)."""
    m = max(float(np.abs(ref).max()), floor)
    if m < 1e-35:
        assert float(np.abs(got).max()) < 1e-33, what
        return
    g, r = got.astype(np.float64) / m, ref.astype(np.float64) / m
    d = g - r
    mx = float(np.abs(d).max())
    rl = float(np.linalg.norm(d) / max(np.linalg.norm(r), np.sqrt(r.size) * 1e-3))   # floor-sized levels: against the floor
    assert np.isfinite(got).all(), f"{what}: non-finite state"
    assert mx <= 2e-2, f"{what}: max-abs {mx:.3e} of the level's scale"
    assert rl <= 1e-2, f"{what}: rel-L2 {rl:.3e}"


def _close_states(got, ref, what):
    top = float(np.abs(ref).max())
    mx, rl = err_stats(got, ref)
    print(f"[parity] {what} Fenwick states: max-abs {mx:.3e} of |ref|_inf {top:.3e}, rel-L2 {rl:.3e}")
    assert mx <= 2e-2 * max(top, 1e-30) and rl <= 1e-2, f"{what}: whole state max-abs {mx:.3e} rel-L2 {rl:.3e}"
    for l in range(ref.shape[-1]):
        _close_level(got[..., l], ref[..., l], f"{what} level {l}", 1e-3 * top)


def _ref(inp, T=None):
    sl = slice(None) if T is None else slice(0, T)
    return oracle.hgdn(to_np(inp["q"][0, sl]), to_np(inp["k"][0, sl]), to_np(inp["v"][0, sl]),
                       to_np(inp["g"][0, sl]), to_np(inp["beta"][0, sl]), to_np(inp["lam"][0, sl]),
                       use_l2norm=True)


STATE_CASES = [
    # T, H, K, V, g_shift, extra levels
    (64, 1, 64, 64, -3.0, 0),
    (128, 2, 64, 64, -3.0, 1),
    (192, 2, 64, 64, 2.0, 0),
    (2368, 2, 64, 64, -4.0, 0),     # 37 chunks: last chunk index 36 = 100100b, one cross-block level
    (6400, 2, 64, 64, -5.0, 2),     # 100 chunks: index 99 = 1100011b
    (4096, 1, 64, 64, -4.0, 0),     # index 63: every level occupied
    (4160, 1, 64, 64, -4.0, 0),     # index 64: only the top level
    (5056, 2, 32, 32, -4.0, 0),
    (4096 + 320, 3, 16, 32, 2.0, 1),
    (64 * 601, 1, 64, 64, -6.0, 0),  # 601 chunks (index 600 = 1001011000b), decay of ~0.0025 per token
]


@pytest.mark.parametrize("T,H,K,V,gs,extra", STATE_CASES)
def test_prefill_state_matches_token_recurrence(lb, T, H, K, V, gs, extra):
    from lampa_b200 import synth
    Lv = lb.num_levels_required(T) + extra
    inp = synth.gdn_inputs(20260, T, H, K, V, L=Lv, g_shift=gs)
    d = _cuda(inp)
    o, hs = lb.chunk_h_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["lam"], d["beta"],
                                        output_final_state=True, use_qk_l2norm_in_kernel=True)
    oref, sref, cref = _ref(inp)
    assert isinstance(hs, lb.HState) and hs.states.dtype == torch.float32
    assert tuple(hs.states.shape) == (1, H, K, V, Lv) and tuple(hs.counts.shape) == (Lv,)
    assert_close_bf16(to_np(o[0]), oref, "o")
    np.testing.assert_array_equal(to_np(hs.counts), cref)
    got = to_np(hs.states[0])
    for l in range(Lv):
        if cref[l] == 0:
            assert not got[..., l].any(), f"level {l} must be empty"
    _close_states(got, sref, f"T={T} K={K}")
    # the plain final state is the sum over levels when every lambda is 1
    _, ht = lb.chunk_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"], output_final_state=True,
                                      use_qk_l2norm_in_kernel=True)
    assert_close_bf16(got.sum(-1), to_np(ht[0]), "sum of levels vs plain final state")


def test_prefill_batch_rows_are_independent(lb):
    from lampa_b200 import synth
    T, H, K, V = 704, 2, 64, 64
    Lv = lb.num_levels_required(T)
    a = synth.gdn_inputs(1, T, H, K, V, L=Lv, g_shift=-3.0)
    b = synth.gdn_inputs(2, T, H, K, V, L=Lv, g_shift=-3.0)
    d = {k: torch.cat([a[k], b[k]], 0).cuda() for k in a}
    o, hs = lb.chunk_h_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["lam"], d["beta"],
                                        output_final_state=True, use_qk_l2norm_in_kernel=True)
    for i, inp in enumerate((a, b)):
        oref, sref, cref = _ref(inp)
        assert_close_bf16(to_np(o[i]), oref, f"o row {i}")
        _close_states(to_np(hs.states[i]), sref, f"states row {i}")
        np.testing.assert_array_equal(to_np(hs.counts), cref)


@pytest.mark.parametrize("T,K,V", [(200, 64, 64), (70, 32, 32), (40, 16, 32)])
def test_prefill_with_ragged_tail_and_decode(lb, T, K, V):
    """T mod 64 tokens go through the step kernel (T < 64: all of them); then one more decode step
    through the initial_state branch of the API."""
    from lampa_b200 import synth
    H = 2
    Lv = lb.num_levels_required(T + 64) + 1
    inp = synth.gdn_inputs(31, T + 1, H, K, V, L=Lv, g_shift=-3.0)
    d = _cuda(inp)
    cut = {k: x[:, :T] for k, x in d.items()}
    o, hs = lb.chunk_h_gated_delta_rule(cut["q"], cut["k"], cut["v"], cut["g"], cut["lam"], cut["beta"],
                                        output_final_state=True, use_qk_l2norm_in_kernel=True)
    oref, sref, cref = _ref(inp, T)
    assert_close_bf16(to_np(o[0]), oref, "o with tail")
    _close_states(to_np(hs.states[0]), sref, "states with tail")
    np.testing.assert_array_equal(to_np(hs.counts), cref)
    # decode token T
    last = {k: x[:, T:T + 1] for k, x in d.items()}
    o1, hs1 = lb.chunk_h_gated_delta_rule(last["q"], last["k"], last["v"], last["g"], last["lam"], last["beta"],
                                          initial_state=hs, output_final_state=True, use_qk_l2norm_in_kernel=True)
    assert hs1 is hs and tuple(o1.shape) == (1, 1, H, V)
    oref1, sref1, cref1 = _ref(inp)
    assert_close_bf16(to_np(o1[0, 0]), oref1[T], "decode output")
    _close_states(to_np(hs.states[0]), sref1, "decode states")
    np.testing.assert_array_equal(to_np(hs.counts), cref1)


def test_decode_from_empty_state_crosses_chunk_boundaries(lb):
    """130 decode steps from an empty state: every cascade depth up to level 8 occurs."""
    from lampa_b200 import synth
    T, H, K, V, Lv = 130, 2, 64, 64, 10
    inp = synth.gdn_inputs(33, T, H, K, V, L=Lv, g_shift=-3.0)
    d = _cuda(inp)
    hs = lb.HState(2, lb.HType.WEAK, lb.HStruct.GDELTA, (1, H, K, V, Lv), torch.float32, "cuda:0")
    scale = K ** -0.5
    outs = []
    for t in range(T):
        o, hs = lb.hattention_step(hs, d["q"][:, t], d["k"][:, t], d["v"][:, t], d["beta"][:, t], d["g"][:, t],
                                   d["lam"][:, t] / scale, scale, 2, lb.HType.WEAK, lb.HStruct.GDELTA,
                                   use_qk_l2norm_in_kernel=True)
        outs.append(o)
    oref, sref, cref = _ref(inp)
    assert_close_bf16(to_np(torch.cat(outs, 0)), oref, "decode outputs")
    _close_states(to_np(hs.states[0]), sref, "decode states")
    np.testing.assert_array_equal(to_np(hs.counts), cref)


def test_state_golden_fixture_from_reference(lb, golden_dir):
    """states / counts written by the reference's hattention_recurrent (tests/golden)."""
    for name in ("hgdn_T320_H2_K32_V32_L10", "hgdn_T256_H1_K64_V64_L9", "hgdn_T200_H2_K16_V32_L9"):
        z = np.load(os.path.join(golden_dir, name + ".npz"))
        t = {k: torch.from_numpy(z[k])[None].cuda() for k in ("q", "k", "v", "g", "beta", "lam")}
        _, hs = lb.chunk_h_gated_delta_rule(t["q"].bfloat16(), t["k"].bfloat16(), t["v"].bfloat16(), t["g"],
                                            t["lam"], t["beta"], output_final_state=True,
                                            use_qk_l2norm_in_kernel=True)
        np.testing.assert_array_equal(to_np(hs.counts), z["counts_hier"])
        got, ref = to_np(hs.states[0]), z["states_hier"]
        mx = np.abs(got - ref).max()
        assert mx < 5e-2 * max(1.0, np.abs(ref).max()), (name, mx)


def test_step_reports_a_full_hierarchy(lb):
    """A cascade that would leave the last level is reported in the status word, state untouched."""
    H, K, V, Lv = 1, 64, 64, 2
    hs = lb.HState(2, lb.HType.WEAK, lb.HStruct.GDELTA, (1, H, K, V, Lv), torch.float32, "cuda:0")
    g = torch.zeros(1, H, device="cuda:0")
    x = torch.randn(1, H, K, device="cuda:0").bfloat16()
    lam = torch.ones(1, H, Lv, device="cuda:0")
    scale = K ** -0.5
    os.environ["LAMPA_B200_CHECK"] = "0"
    try:
        for _ in range(2):          # two levels: the third token's cascade would leave level 1
            lb.hattention_step(hs, x, x, x, g + 0.5, g, lam, scale, 2, lb.HType.WEAK, lb.HStruct.GDELTA,
                               use_qk_l2norm_in_kernel=True)
        lb.check_status(torch.device("cuda:0"))
        before = hs.states.clone()
        lb.hattention_step(hs, x, x, x, g + 0.5, g, lam, scale, 2, lb.HType.WEAK, lb.HStruct.GDELTA,
                           use_qk_l2norm_in_kernel=True)
        with pytest.raises(lb.LampaError):
            lb.check_status(torch.device("cuda:0"))
        assert torch.equal(before, hs.states)
    finally:
        os.environ["LAMPA_B200_CHECK"] = "1"


def test_final_state_of_packed_sequences_through_the_c_abi(lb):
    """lampa_hgdn_final_state with cu_seqlens: one Fenwick state and one counts row per sequence
    (the Python op does not expose this; the C entry point does)."""
    import ctypes
    from lampa_b200 import _lib as L, synth
    H, K, V = 2, 64, 64
    lens = [2112, 64, 0, 4160, 640]
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    T = int(cu[-1])
    Lv = lb.num_levels_required(max(lens)) + 1
    inp = synth.gdn_inputs(41, T, H, K, V, L=Lv, g_shift=-3.0)
    d = _cuda(inp)
    cud = torch.from_numpy(cu).cuda()
    N = len(lens)
    desc = L.GdnDesc(B=1, T=T, H=H, K=K, V=V, L=Lv, nseq=N, qkv_dtype=L.LAMPA_BF16, gb_dtype=L.LAMPA_F32,
                     lam_dtype=L.LAMPA_F32, use_l2norm=1, scale=1.0)
    nbytes = ctypes.c_size_t(0)
    L.check(L.lib().lampa_gdn_workspace_bytes(ctypes.byref(desc), ctypes.byref(nbytes)), "workspace")
    buf = torch.empty(nbytes.value + 1024, dtype=torch.uint8, device="cuda:0")
    ws = buf[(-buf.data_ptr()) % 1024:][: nbytes.value]
    o = torch.empty(1, T, H, V, dtype=torch.bfloat16, device="cuda:0")
    st = L.status_word(torch.device("cuda:0"))
    stream = L.stream_ptr(torch.device("cuda:0"))
    L.check(L.lib().lampa_hgdn_fwd(ctypes.byref(desc), L.ptr(d["q"]), L.ptr(d["k"]), L.ptr(d["v"]), L.ptr(d["g"]),
                                   L.ptr(d["beta"]), L.ptr(d["lam"]), L.ptr(cud), L.ptr(o), L.ptr(ws), ws.numel(),
                                   L.ptr(st), stream), "lampa_hgdn_fwd")
    states = torch.full((N, H, K, V, Lv), float("nan"), device="cuda:0")
    counts = torch.full((N, Lv), -1, dtype=torch.int32, device="cuda:0")
    L.check(L.lib().lampa_hgdn_final_state(ctypes.byref(desc), L.ptr(d["k"]), L.ptr(d["v"]), L.ptr(d["g"]),
                                           L.ptr(d["beta"]), L.ptr(cud), L.ptr(ws), ws.numel(), L.ptr(states),
                                           L.ptr(counts), L.ptr(st), stream), "lampa_hgdn_final_state")
    L.check_status(torch.device("cuda:0"))
    for n, (s, e) in enumerate(zip(cu[:-1], cu[1:])):
        got_s, got_c = to_np(states[n]), to_np(counts[n])
        if e == s:
            assert not got_s.any() and not got_c.any()
            continue
        sub = {k: x[:, s:e] for k, x in inp.items()}
        _, sref, cref = _ref(sub)
        np.testing.assert_array_equal(got_c, cref)
        _close_states(got_s, sref, f"sequence {n}")


def test_final_state_of_packed_sequences_through_the_python_op(lb):
    """chunk_h_gated_delta_rule(output_final_state=True, cu_seqlens=...) returns one Fenwick state
    and one counts row per sequence."""
    from lampa_b200 import synth
    H, K, V = 2, 32, 32
    lens = [1280, 64, 3200]
    cu = torch.tensor([0] + lens).cumsum(0)
    T = int(cu[-1])
    Lv = lb.num_levels_required(max(lens))
    inp = synth.gdn_inputs(43, T, H, K, V, L=Lv, g_shift=-3.0)
    d = _cuda(inp)
    o, hs = lb.chunk_h_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["lam"], d["beta"], cu_seqlens=cu,
                                        output_final_state=True, use_qk_l2norm_in_kernel=True)
    assert isinstance(hs, lb.HState) and tuple(hs.states.shape) == (3, H, K, V, Lv) and tuple(hs.counts.shape) == (3, Lv)
    for n, (s, e) in enumerate(zip(cu[:-1].tolist(), cu[1:].tolist())):
        sub = {k: x[:, s:e] for k, x in inp.items()}
        oref, sref, cref = _ref(sub)
        assert_close_bf16(to_np(o[0, s:e]), oref, f"o of sequence {n}")
        np.testing.assert_array_equal(to_np(hs.counts[n]), cref)
        _close_states(to_np(hs.states[n]), sref, f"sequence {n}")
