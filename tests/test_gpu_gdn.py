"""GPU parity of the gated-delta forward ops (through the C ABI) against the CPU checker.

Tolerance (bf16 operands, fp32 accumulation, against the fp32 token recurrence):
max-abs <= 2e-2 * max(1, |ref|_inf) and relative L2 <= 1e-2.
"""
import os

import numpy as np
import pytest
import torch

from oracle import oracle
from tests.util import assert_close_bf16, to_np

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


def _plain_ref(inp, scale=None, h0=None, cu=None, l2=True):
    return oracle.gdn_plain(to_np(inp["q"][0]), to_np(inp["k"][0]), to_np(inp["v"][0]), to_np(inp["g"][0]),
                            to_np(inp["beta"][0]), scale=scale, h0=h0, cu_seqlens=cu, use_l2norm=l2)


PLAIN_CASES = [
    # T, H, K, V, g_shift, h0
    (64, 1, 64, 64, -3.0, False),
    (1, 2, 64, 64, -3.0, True),
    (200, 2, 64, 64, 2.0, True),
    (2048, 2, 64, 64, -4.0, False),
    (2112, 3, 64, 64, -4.0, True),
    (6144, 4, 64, 64, 2.0, False),       # benchmark configuration 0's shape
    (5000, 2, 32, 32, -4.0, True),
    (3000, 3, 16, 32, -5.0, True),
]


@pytest.mark.parametrize("T,H,K,V,gs,h0", PLAIN_CASES)
def test_plain_matches_token_recurrence(lb, T, H, K, V, gs, h0):
    from lampa_b200 import synth
    inp = synth.gdn_inputs(20250, T, H, K, V, g_shift=gs, h0=h0)
    d = _cuda(inp)
    o, ht = lb.chunk_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d.get("h0"),
                                      output_final_state=True, use_qk_l2norm_in_kernel=True)
    oref, htref = _plain_ref(inp, h0=None if not h0 else to_np(inp["h0"]))
    assert o.dtype == torch.bfloat16 and ht.dtype == torch.float32
    assert_close_bf16(to_np(o[0]), oref, "o")
    assert_close_bf16(to_np(ht), htref, "final_state")


def test_plain_options_dtypes_scale_and_batch(lb):
    from lampa_b200 import synth
    T, H, K, V = 700, 2, 64, 64
    inp = synth.gdn_inputs(7, T, H, K, V, g_shift=-3.0)
    d = _cuda(inp)
    # no l2norm, custom scale, no final state
    o, ht = lb.chunk_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"], scale=0.3)
    assert ht is None
    oref, _ = _plain_ref(inp, scale=0.3, l2=False)
    assert_close_bf16(to_np(o[0]), oref, "o (no l2norm, scale 0.3)")
    # fp16 inputs (rounded to bf16 operands inside); output in the input dtype
    dt = torch.float16
    o2, _ = lb.chunk_gated_delta_rule(d["q"].to(dt), d["k"].to(dt), d["v"].to(dt), d["g"], d["beta"],
                                      use_qk_l2norm_in_kernel=True)
    assert o2.dtype == dt
    oref2, _ = _plain_ref(inp)
    assert_close_bf16(to_np(o2[0]), oref2, f"o ({dt})")
    # fp32 q / k / v are refused, as by the reference (gated_delta_rule_ori.py:313)
    with pytest.raises(AssertionError):
        lb.chunk_gated_delta_rule(d["q"].float(), d["k"].float(), d["v"].float(), d["g"], d["beta"])
    # bf16 g / beta
    o3, _ = lb.chunk_gated_delta_rule(d["q"], d["k"], d["v"], d["g"].bfloat16(), d["beta"].bfloat16(),
                                      use_qk_l2norm_in_kernel=True)
    inp3 = dict(inp, g=inp["g"].bfloat16().float(), beta=inp["beta"].bfloat16().float())
    assert_close_bf16(to_np(o3[0]), _plain_ref(inp3)[0], "o (bf16 g, beta)")
    # batch of 2 == two separate calls
    q2 = torch.cat([d["q"], d["q"].flip(1)], 0)
    k2 = torch.cat([d["k"], d["k"].flip(1)], 0)
    v2 = torch.cat([d["v"], d["v"].flip(1)], 0)
    g2 = torch.cat([d["g"], d["g"].flip(1)], 0)
    b2 = torch.cat([d["beta"], d["beta"].flip(1)], 0)
    ob, hb = lb.chunk_gated_delta_rule(q2, k2, v2, g2, b2, output_final_state=True, use_qk_l2norm_in_kernel=True)
    oa, ha = lb.chunk_gated_delta_rule(q2[1:], k2[1:], v2[1:], g2[1:], b2[1:], output_final_state=True,
                                       use_qk_l2norm_in_kernel=True)
    assert torch.equal(ob[1:], oa) and torch.equal(hb[1:], ha)


def test_plain_varlen_matches_separate_sequences(lb):
    from lampa_b200 import synth
    H, K, V = 2, 64, 64
    lens = [130, 64, 1, 2500, 0, 777]
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    T = int(cu[-1])
    inp = synth.gdn_inputs(11, T, H, K, V, g_shift=-3.0)
    gen = torch.Generator().manual_seed(3)
    h0 = 0.1 * torch.randn(len(lens), H, K, V, generator=gen)
    d = _cuda(inp)
    o, ht = lb.chunk_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=h0.cuda(),
                                      output_final_state=True, cu_seqlens=torch.from_numpy(cu).cuda(),
                                      use_qk_l2norm_in_kernel=True)
    oref, htref = _plain_ref(inp, h0=h0.numpy(), cu=cu)
    assert_close_bf16(to_np(o[0]), oref, "o varlen")
    assert_close_bf16(to_np(ht), htref, "final_state varlen")
    # bit-identical to running one sequence alone
    s = 3
    sl = slice(int(cu[s]), int(cu[s + 1]))
    o1, h1 = lb.chunk_gated_delta_rule(d["q"][:, sl], d["k"][:, sl], d["v"][:, sl], d["g"][:, sl], d["beta"][:, sl],
                                       initial_state=h0[s:s + 1].cuda(), output_final_state=True,
                                       use_qk_l2norm_in_kernel=True)
    assert torch.equal(o1[0], o[0, sl]) and torch.equal(h1[0], ht[s])


def test_plain_deterministic_and_state_handover(lb):
    from lampa_b200 import synth
    inp = _cuda(synth.gdn_inputs(5, 4096, 2, 64, 64, g_shift=-5.0))
    args = (inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"])
    o1, h1 = lb.chunk_gated_delta_rule(*args, output_final_state=True, use_qk_l2norm_in_kernel=True)
    o2, h2 = lb.chunk_gated_delta_rule(*args, output_final_state=True, use_qk_l2norm_in_kernel=True)
    assert torch.equal(o1, o2) and torch.equal(h1, h2)
    # first half, then second half seeded with the first half's final state
    half = [x[:, :2048] for x in args]
    rest = [x[:, 2048:] for x in args]
    oa, ha = lb.chunk_gated_delta_rule(*half, output_final_state=True, use_qk_l2norm_in_kernel=True)
    ob, hb = lb.chunk_gated_delta_rule(*rest, initial_state=ha, output_final_state=True, use_qk_l2norm_in_kernel=True)
    assert_close_bf16(to_np(torch.cat([oa, ob], 1)), to_np(o1), "hand-over o")
    assert_close_bf16(to_np(hb), to_np(h1), "hand-over state")


def test_plain_full_size_config1(lb):
    """Benchmark configuration 1: T=65536, H=8, K=V=64, bf16, with and without an initial state."""
    from lampa_b200 import synth
    inp = synth.gdn_inputs(20251, 65536, 8, 64, 64, g_shift=2.0, h0=True)
    d = _cuda(inp)
    o, ht = lb.chunk_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"],
                                      output_final_state=True, use_qk_l2norm_in_kernel=True)
    oref, htref = _plain_ref(inp, h0=to_np(inp["h0"]))
    assert_close_bf16(to_np(o[0]), oref, "o config 1")
    assert_close_bf16(to_np(ht), htref, "final state config 1")
    # slow-decay variant exercises the inter-chunk path over all 1024 chunks
    inp = synth.gdn_inputs(20251, 65536, 8, 64, 64, g_shift=-6.0)
    d = _cuda(inp)
    o, ht = lb.chunk_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"], output_final_state=True,
                                      use_qk_l2norm_in_kernel=True)
    oref, htref = _plain_ref(inp)
    assert_close_bf16(to_np(o[0]), oref, "o config 1 slow decay")
    assert_close_bf16(to_np(ht), htref, "final state config 1 slow decay")


HIER_CASES = [
    # T, H, K, V, g_shift
    (64, 1, 64, 64, -3.0),
    (128, 2, 64, 64, -3.0),
    (200, 2, 64, 64, 2.0),
    (2048, 2, 64, 64, -4.0),
    (4096, 2, 64, 64, -4.0),
    (8256, 2, 64, 64, -5.0),
    (5000, 2, 32, 32, -4.0),
    (4096, 3, 16, 32, 2.0),
]


def _hier_ref(inp, cu=None):
    return oracle.hgdn(to_np(inp["q"][0]), to_np(inp["k"][0]), to_np(inp["v"][0]), to_np(inp["g"][0]),
                       to_np(inp["beta"][0]), to_np(inp["lam"][0]), cu_seqlens=cu, use_l2norm=True)[0]


@pytest.mark.parametrize("T,H,K,V,gs", HIER_CASES)
def test_hier_matches_token_recurrence(lb, T, H, K, V, gs):
    from lampa_b200 import synth
    Lv = lb.num_levels_required(T)
    inp = synth.gdn_inputs(20252, T, H, K, V, L=Lv, g_shift=gs)
    d = _cuda(inp)
    o, fs = lb.chunk_h_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["lam"], d["beta"],
                                        use_qk_l2norm_in_kernel=True)
    assert fs is None and o.dtype == torch.bfloat16
    assert_close_bf16(to_np(o[0]), _hier_ref(inp), "o hier")


def test_hier_against_reference_chunkwise_statement(lb, golden_dir):
    """The reference's own chunkwise statement (hgdn_minimal) at T = 4096: cross-block level and
    block composites against numbers the reference itself produced."""
    from tests.util import minimal_fixture_inputs
    z = np.load(os.path.join(golden_dir, "hgdn_minimal_T4096_H2_K32_V32_L13.npz"))
    q, k, v, beta, g, lam = minimal_fixture_inputs(z)
    qb, kb, vb = (x.bfloat16() for x in (q, k, v))
    o, _ = lb.chunk_h_gated_delta_rule(qb[None].cuda(), kb[None].cuda(), vb[None].cuda(), g[None].cuda(), lam[None].cuda(),
                                       beta[None].cuda(), use_qk_l2norm_in_kernel=True)
    # the fixture was computed from the fp32 inputs: the comparison carries the bf16 rounding of q, k, v as well
    assert_close_bf16(to_np(o[0]), z["o_hier"], "o vs hgdn_minimal (reference fixture)")


def test_hier_golden_fixture_from_reference(lb, golden_dir):
    """Inputs and outputs produced by the reference's hattention_recurrent (tests/golden)."""
    for name in ("hgdn_T320_H2_K32_V32_L10", "hgdn_T256_H1_K64_V64_L9", "hgdn_T200_H2_K16_V32_L9"):
        z = np.load(os.path.join(golden_dir, name + ".npz"))
        t = {k: torch.from_numpy(z[k])[None].cuda() for k in ("q", "k", "v", "g", "beta", "lam")}
        o, _ = lb.chunk_h_gated_delta_rule(t["q"].bfloat16(), t["k"].bfloat16(), t["v"].bfloat16(), t["g"], t["lam"],
                                           t["beta"], use_qk_l2norm_in_kernel=True)
        # fixture inputs are fp32; compare against the checker on the bf16-rounded inputs and,
        # more loosely, against the reference's fp32 output itself
        ref_r = oracle.hgdn(to_np(t["q"].bfloat16()[0]), to_np(t["k"].bfloat16()[0]), to_np(t["v"].bfloat16()[0]),
                            z["g"], z["beta"], z["lam"], use_l2norm=True)[0]
        assert_close_bf16(to_np(o[0]), ref_r, name)
        mx = np.abs(to_np(o[0]) - z["o_hier"]).max()
        assert mx < 5e-2 * max(1.0, np.abs(z["o_hier"]).max()), (name, mx)
        op, _ = lb.chunk_gated_delta_rule(t["q"].bfloat16(), t["k"].bfloat16(), t["v"].bfloat16(), t["g"], t["beta"],
                                          scale=float(z["scale"]), use_qk_l2norm_in_kernel=True)
        assert np.abs(to_np(op[0]) - z["o_plain"]).max() < 5e-2 * max(1.0, np.abs(z["o_plain"]).max())


def test_hier_with_unit_weights_equals_plain(lb):
    from lampa_b200 import synth
    T, H, K, V = 4096, 2, 64, 64
    inp = _cuda(synth.gdn_inputs(9, T, H, K, V, L=lb.num_levels_required(T), g_shift=-4.0))
    scale = K ** -0.5
    lam = torch.full_like(inp["lam"], scale)
    oh, _ = lb.chunk_h_gated_delta_rule(inp["q"], inp["k"], inp["v"], inp["g"], lam, inp["beta"],
                                        use_qk_l2norm_in_kernel=True)
    op, _ = lb.chunk_gated_delta_rule(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"],
                                      use_qk_l2norm_in_kernel=True)
    assert_close_bf16(to_np(oh), to_np(op), "hier(lambda=scale) vs plain")
    # hattention_kernel takes l already divided by scale
    ok = lb.hattention_kernel(inp["q"], inp["k"], inp["v"], inp["beta"], inp["g"], inp["lam"] / scale, scale, False, 2,
                              lb.HType.WEAK, lb.HStruct.GDELTA, use_qk_l2norm_in_kernel=True)
    oh2, _ = lb.chunk_h_gated_delta_rule(inp["q"], inp["k"], inp["v"], inp["g"], inp["lam"], inp["beta"],
                                         use_qk_l2norm_in_kernel=True)
    assert_close_bf16(to_np(ok), to_np(oh2), "hattention_kernel vs chunk_h_gated_delta_rule")


def test_hier_varlen_and_padding(lb):
    from lampa_b200 import synth
    H, K, V = 2, 64, 64
    lens = [2100, 64, 130, 0, 4500]
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    T = int(cu[-1])
    Lv = lb.num_levels_required(max(lens))
    inp = synth.gdn_inputs(13, T, H, K, V, L=Lv, g_shift=-4.0)
    d = _cuda(inp)
    o, _ = lb.chunk_h_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["lam"], d["beta"],
                                       cu_seqlens=torch.from_numpy(cu).cuda(), use_qk_l2norm_in_kernel=True)
    assert_close_bf16(to_np(o[0]), _hier_ref(inp, cu=cu), "o hier varlen")
    # padding a sequence with inert tokens (k = v = 0, beta = 0, g = 0, lambda = 0) leaves the real part unchanged
    Tr, Tp = 1000, 1024
    inp = synth.gdn_inputs(14, Tp, H, K, V, L=lb.num_levels_required(Tp), g_shift=-4.0)
    for key in ("k", "v", "beta", "g", "lam", "q"):
        inp[key][:, Tr:] = 0
    d = _cuda(inp)
    o_pad, _ = lb.chunk_h_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["lam"], d["beta"],
                                           use_qk_l2norm_in_kernel=True)
    o_cut, _ = lb.chunk_h_gated_delta_rule(d["q"][:, :Tr], d["k"][:, :Tr], d["v"][:, :Tr], d["g"][:, :Tr],
                                           d["lam"][:, :Tr], d["beta"][:, :Tr], use_qk_l2norm_in_kernel=True)
    assert torch.equal(o_pad[:, :Tr], o_cut)


def test_hier_full_size_config2(lb):
    """Benchmark configuration 2: 60000 real tokens padded to 61440, H=8, K=V=64, L=17, bf16."""
    from lampa_b200 import synth
    T, Tr, H = 61440, 60000, 8
    inp = synth.gdn_inputs(20252, T, H, 64, 64, L=17, g_shift=2.0)
    for key in ("k", "v", "beta", "g", "lam"):
        inp[key][:, Tr:] = 0
    d = _cuda(inp)
    o, _ = lb.chunk_h_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["lam"], d["beta"],
                                       use_qk_l2norm_in_kernel=True)
    ref = _hier_ref({k: v[:, :Tr] for k, v in inp.items()})
    assert_close_bf16(to_np(o[0, :Tr]), ref, "o config 2")
    inp = synth.gdn_inputs(20252, T, H, 64, 64, L=17, g_shift=-6.0)
    d = _cuda(inp)
    o, _ = lb.chunk_h_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["lam"], d["beta"],
                                       use_qk_l2norm_in_kernel=True)
    assert_close_bf16(to_np(o[0]), _hier_ref(inp), "o config 2 slow decay")


def test_error_conventions(lb):
    from lampa_b200 import synth
    d = _cuda(synth.gdn_inputs(1, 128, 2, 64, 64, L=8))
    with pytest.raises(DeprecationWarning):
        lb.chunk_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"], head_first=True)
    with pytest.raises(ValueError):
        lb.chunk_gated_delta_rule(d["q"].repeat(2, 1, 1, 1), d["k"].repeat(2, 1, 1, 1), d["v"].repeat(2, 1, 1, 1),
                                  d["g"].repeat(2, 1, 1), d["beta"].repeat(2, 1, 1),
                                  cu_seqlens=torch.tensor([0, 128]).cuda())
    with pytest.raises(ValueError):
        lb.chunk_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"], cu_seqlens=torch.tensor([0, 64, 128]).cuda(),
                                  initial_state=torch.zeros(3, 2, 64, 64).cuda())
    with pytest.raises(AssertionError):
        lb.chunk_h_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["lam"], d["beta"], use_qk_l2norm_in_kernel=False)
    with pytest.raises(ValueError):   # 128 tokens need 8 levels
        lb.chunk_h_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["lam"][..., :7], d["beta"],
                                    use_qk_l2norm_in_kernel=True)
    with pytest.raises(lb.LampaError):   # CPU tensors: there is no CPU path
        lb.chunk_gated_delta_rule(d["q"].cpu(), d["k"].cpu(), d["v"].cpu(), d["g"].cpu(), d["beta"].cpu())
    # packed sequences with too few levels are reported by the device status word
    with pytest.raises(lb.LampaError):
        lb.chunk_h_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["lam"][..., :7].contiguous(), d["beta"],
                                    cu_seqlens=torch.tensor([0, 128]).cuda(), use_qk_l2norm_in_kernel=True)


def test_packed_events_like_config4(lb):
    """Benchmark configuration 4's mixer shape: many events of ragged length packed with cu_seqlens,
    H = 4, K = V = 32 (a subset of events keeps the CPU check short); each event restarts the hierarchy."""
    from lampa_b200 import synth
    H, K, V = 4, 32, 32
    lens = synth.event_sizes(20254, 64)[:12].tolist()
    lens = [n // 8 for n in lens]                      # 750 .. 7500 hits per event
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    T = int(cu[-1])
    Lv = lb.num_levels_required(max(lens))
    inp = synth.gdn_inputs(20254, T, H, K, V, L=Lv, g_shift=-3.0)
    d = _cuda(inp)
    cu_d = torch.from_numpy(cu).cuda()
    o, _ = lb.chunk_h_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["lam"], d["beta"], cu_seqlens=cu_d,
                                       use_qk_l2norm_in_kernel=True)
    assert_close_bf16(to_np(o[0]), _hier_ref(inp, cu=cu), "o hier, packed events")
    op, ht = lb.chunk_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"], cu_seqlens=cu_d,
                                       output_final_state=True, use_qk_l2norm_in_kernel=True)
    oref, htref = _plain_ref(inp, cu=cu)
    assert_close_bf16(to_np(op[0]), oref, "o plain, packed events")
    assert_close_bf16(to_np(ht), htref, "final states, packed events")
    # K = V = 64 packed events go through the tcgen05 output pass
    inp = synth.gdn_inputs(20255, T, 2, 64, 64, L=Lv, g_shift=-3.0)
    d = _cuda(inp)
    o, _ = lb.chunk_h_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["lam"], d["beta"], cu_seqlens=cu_d,
                                       use_qk_l2norm_in_kernel=True)
    assert_close_bf16(to_np(o[0]), _hier_ref(inp, cu=cu), "o hier, packed events, K=V=64")


def test_tensor_core_paths_agree(lb):
    """The tcgen05 kernels and their mma.sync twins (lampa_debug_force_mma_sync) on the same input: hierarchical
    and plain rule, preparation and output passes, fixed-length and packed input, an odd number of heads."""
    from lampa_b200 import _lib as L, synth
    T, H = 8192 + 640, 3
    inp = _cuda(synth.gdn_inputs(31, T, H, 64, 64, L=lb.num_levels_required(T), g_shift=-4.0))
    h0 = torch.randn(1, H, 64, 64, device="cuda") * 0.1
    cu = torch.tensor([0, 700, 764, 5000, T], dtype=torch.int64)
    h0p = torch.randn(4, H, 64, 64, device="cuda") * 0.1
    hier = lambda: lb.chunk_h_gated_delta_rule(inp["q"], inp["k"], inp["v"], inp["g"], inp["lam"], inp["beta"],
                                               use_qk_l2norm_in_kernel=True)[0]
    plain = lambda: lb.chunk_gated_delta_rule(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], initial_state=h0,
                                              output_final_state=True, use_qk_l2norm_in_kernel=True)
    packed = lambda: lb.chunk_gated_delta_rule(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], initial_state=h0p,
                                               output_final_state=True, cu_seqlens=cu, use_qk_l2norm_in_kernel=True)
    res = {}
    try:
        for mode in (0, 1):                      # 0: the tcgen05 kernels; 1: their mma.sync twins
            assert L.lib().lampa_debug_force_mma_sync(mode) == 0
            res[mode] = (hier(), plain(), packed())
    finally:
        L.lib().lampa_debug_force_mma_sync(0)
    (o_t, (p_t, s_t), (q_t, r_t)), (o_m, (p_m, s_m), (q_m, r_m)) = res[0], res[1]
    assert not torch.equal(o_t, o_m) and not torch.equal(p_t, p_m)          # different kernels did run
    assert_close_bf16(to_np(o_t), to_np(o_m), "hier: tcgen05 vs mma.sync")
    assert_close_bf16(to_np(p_t), to_np(p_m), "plain: tcgen05 vs mma.sync")
    assert_close_bf16(to_np(s_t), to_np(s_m), "plain final state: tcgen05 vs mma.sync")
    assert_close_bf16(to_np(q_t), to_np(q_m), "plain, packed: tcgen05 vs mma.sync")
    assert_close_bf16(to_np(r_t), to_np(r_m), "plain, packed, final states: tcgen05 vs mma.sync")


def test_head_slices_reproduce_the_full_call(lb):
    """Splitting one event by head (what a rank of a head-sharded job computes) gives the same rows as the full call."""
    from lampa_b200 import synth
    T, H = 4096 + 200, 4
    inp = _cuda(synth.gdn_inputs(77, T, H, 64, 64, L=lb.num_levels_required(T), g_shift=-4.0))
    full, _ = lb.chunk_h_gated_delta_rule(inp["q"], inp["k"], inp["v"], inp["g"], inp["lam"], inp["beta"],
                                          use_qk_l2norm_in_kernel=True)
    parts = []
    for h0, h1 in ((0, 1), (1, 4)):           # uneven on purpose: a lone head and an odd group
        sl = {k: inp[k][:, :, h0:h1].contiguous() for k in ("q", "k", "v", "g", "beta", "lam")}
        o, _ = lb.chunk_h_gated_delta_rule(sl["q"], sl["k"], sl["v"], sl["g"], sl["lam"], sl["beta"],
                                           use_qk_l2norm_in_kernel=True)
        parts.append(o)
    assert torch.equal(torch.cat(parts, dim=2), full)


def test_traced_calls_become_one_dispatcher_node(lb):
    """Under torch.compile the two forwards are single opaque nodes (torch.ops.lampa_b200.*): the whole function
    traces without a graph break and gives the eager result."""
    from lampa_b200 import synth
    T, H = 1024 + 100, 2
    inp = _cuda(synth.gdn_inputs(5, T, H, 64, 64, L=lb.num_levels_required(T), g_shift=-4.0))

    def plain(q, k, v, g, b):
        o, s = lb.chunk_gated_delta_rule(q, k, v, g, b, output_final_state=True, use_qk_l2norm_in_kernel=True)
        return o.float() * 2 + 1, s

    def hier(q, k, v, g, lam, b):
        return lb.chunk_h_gated_delta_rule(q, k, v, g, lam, b, use_qk_l2norm_in_kernel=True)[0].float() - 1

    pa = (inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"])
    ha = (inp["q"], inp["k"], inp["v"], inp["g"], inp["lam"], inp["beta"])
    with torch.no_grad():
        want_p, want_h = plain(*pa), hier(*ha)
        got_p = torch.compile(plain, backend="aot_eager", fullgraph=True)(*pa)
        got_h = torch.compile(hier, backend="aot_eager", fullgraph=True)(*ha)
    assert torch.equal(got_p[0], want_p[0]) and torch.equal(got_p[1], want_p[1])
    assert torch.equal(got_h, want_h)


@pytest.mark.parametrize("K,V,force_mma", [(64, 64, False), (64, 64, True), (32, 32, False)])
def test_output_scatter_equals_a_separate_row_scatter(lb, K, V, force_mma, monkeypatch):
    """out_perm folds the un-ordering into the output store: same bits as the plain call followed by a row scatter."""
    from lampa_b200 import _lib as L, synth
    T, n, H = 2048 + 128, 2100, 3                      # the last 76 tokens are padding and stay where they are
    inp = _cuda(synth.gdn_inputs(9, T, H, K, V, L=lb.num_levels_required(T), g_shift=-4.0))
    args = (inp["q"], inp["k"], inp["v"], inp["g"], inp["lam"], inp["beta"])
    perm = torch.randperm(n, generator=torch.Generator().manual_seed(3)).cuda()
    bad = perm.clone()
    bad[5] = T + 7
    L.lib().lampa_debug_force_mma_sync(int(force_mma))
    try:
        plain, _ = lb.chunk_h_gated_delta_rule(*args, use_qk_l2norm_in_kernel=True)
        fused, _ = lb.chunk_h_gated_delta_rule(*args, use_qk_l2norm_in_kernel=True, out_perm=perm)
        monkeypatch.setenv("LAMPA_B200_CHECK", "0")    # the status word is read below, not inside the call
        out, _ = lb.chunk_h_gated_delta_rule(*args, use_qk_l2norm_in_kernel=True, out_perm=bad)
    finally:
        L.lib().lampa_debug_force_mma_sync(0)
    want = plain.clone()
    want[0, :n] = lb.permute_rows(plain[0, :n].reshape(n, H * V), perm, scatter=True).view(n, H, V)
    assert torch.equal(fused, want)
    # an index outside the output is skipped and reported, nothing else is disturbed
    torch.cuda.synchronize()
    with pytest.raises(lb.LampaError):
        lb.check_status(out.device)
    lb.check_status(out.device)                        # reading the status clears it
    keep = torch.ones(n, dtype=torch.bool, device="cuda")
    keep[5] = False
    assert torch.equal(out[0, perm[keep]], want[0, perm[keep]])
