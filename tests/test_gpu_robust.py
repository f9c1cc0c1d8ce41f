"""Device-side error reporting, in forms that fault nothing: a bounded wait made to run out by
lowering its poll budget, indices outside their segment, malformed packed offsets.  Each case
checks the status word, that the call returned, and that the next normal call is correct."""
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
    return lampa_b200


def _status(lb):
    from lampa_b200 import _lib as L
    torch.cuda.synchronize()
    st = L.status_word(torch.device("cuda:0"))
    vals = st.tolist()
    st.zero_()
    return vals


@pytest.mark.parametrize("hier,T", [(True, 64 * 40), (False, 64 * 40), (True, 64 * 3)])
def test_wait_that_runs_out_sets_timeout_and_returns(lb, hier, T):
    from lampa_b200 import _lib as L, synth
    H, K, V = 2, 64, 64
    Lv = lb.num_levels_required(T)
    inp = synth.gdn_inputs(3, T, H, K, V, L=Lv, g_shift=-3.0)
    d = {k: v.to("cuda:0") for k, v in inp.items()}
    old = os.environ.pop("LAMPA_B200_CHECK", None)

    def run():
        if hier:
            return lb.chunk_h_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["lam"], d["beta"],
                                               use_qk_l2norm_in_kernel=True)[0]
        return lb.chunk_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"], use_qk_l2norm_in_kernel=True)[0]

    try:
        _status(lb)
        assert L.lib().lampa_debug_set_poll_budget(0) == 0
        run()
        vals = _status(lb)                     # synchronises: the kernels came back
        assert vals[0] == L.ERR_TIMEOUT, vals
    finally:
        L.lib().lampa_debug_set_poll_budget(1 << 22)
        if old is not None:
            os.environ["LAMPA_B200_CHECK"] = old
    o = run()
    assert _status(lb)[0] == 0
    a = [inp[k][0].float().numpy() for k in ("q", "k", "v", "g", "beta")]
    ref = oracle.hgdn(*a, inp["lam"][0].numpy(), use_l2norm=True)[0] if hier else oracle.gdn_plain(*a, use_l2norm=True)[0]
    assert_close_bf16(to_np(o[0]), ref, "call after a timed-out one")


def test_indices_outside_their_segment_are_skipped_and_reported(lb):
    from lampa_b200 import _lib as L
    _status(lb)
    src = torch.arange(40, dtype=torch.float32, device="cuda:0").view(10, 4)
    perm = torch.tensor([1, 0, 3, 2, 4, 0, 1, 2, 3, 99], dtype=torch.int64, device="cuda:0")   # two segments of 5
    dst = lb.permute_rows(src, perm, nseg=2)
    vals = _status(lb)
    assert vals[0] == L.ERR_BOUNDS and vals[1] == 10 and vals[2] == 9
    assert torch.equal(dst[:9], src[[1, 0, 3, 2, 4, 5, 6, 7, 8]])
    bad = torch.tensor([[0, 1, -1, 3]], dtype=torch.int64, device="cuda:0")
    lb.invert_permutation(bad)
    assert _status(lb)[0] == L.ERR_BOUNDS
    keys = torch.arange(16, dtype=torch.int32, device="cuda:0")
    lb.segmented_sort(keys, seg_offsets=torch.tensor([0, 8, 40]))                    # second segment leaves the array
    assert _status(lb)[0] == L.ERR_BOUNDS
    good = lb.segmented_sort(keys.flip(0), seg_offsets=torch.tensor([0, 8, 16]))
    assert _status(lb)[0] == 0
    assert good.tolist() == list(range(7, -1, -1)) * 2


def test_malformed_packed_offsets(lb):
    from lampa_b200 import _lib as L, synth
    T, H, K, V = 640, 1, 64, 64
    inp = synth.gdn_inputs(4, T, H, K, V, L=12, g_shift=-3.0)
    d = {k: v.to("cuda:0") for k, v in inp.items()}
    # host-resident offsets are checked on the host
    with pytest.raises(ValueError):
        lb.chunk_h_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["lam"], d["beta"],
                                    cu_seqlens=torch.tensor([0, 700]), use_qk_l2norm_in_kernel=True)
    with pytest.raises(ValueError):
        lb.chunk_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"], cu_seqlens=torch.tensor([-64, 0, 640]))
    with pytest.raises(ValueError):   # 640 tokens in one sequence need 7 + 4 levels
        lb.chunk_h_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["lam"][..., :9], d["beta"],
                                    cu_seqlens=torch.tensor([0, 640]), use_qk_l2norm_in_kernel=True)
    # device-resident offsets: the kernels empty the bad sequence and report it
    old = os.environ.pop("LAMPA_B200_CHECK", None)
    try:
        _status(lb)
        lb.chunk_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"],
                                  cu_seqlens=torch.tensor([-64, 0, 640], device="cuda:0"))
        assert _status(lb)[0] == L.ERR_BOUNDS
        lb.chunk_h_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["lam"][..., :9].contiguous(), d["beta"],
                                    cu_seqlens=torch.tensor([0, 640], device="cuda:0"), use_qk_l2norm_in_kernel=True)
        assert _status(lb)[0] == L.ERR_LEVELS
    finally:
        if old is not None:
            os.environ["LAMPA_B200_CHECK"] = old


def test_forward_only_ops_refuse_autograd(lb):
    q = torch.zeros(1, 128, 2, 64, dtype=torch.bfloat16, device="cuda:0", requires_grad=True)
    g = torch.zeros(1, 128, 2, device="cuda:0")
    with pytest.raises(NotImplementedError):
        lb.chunk_gated_delta_rule(q, q, q, g, g)
    with torch.no_grad():
        o, _ = lb.chunk_gated_delta_rule(q, q, q, g, g)
    assert not o.requires_grad
