"""GPU parity of the packed, event-sharded model forward (benchmark configuration 4) against its
CPU statement (tests/model_oracle.py: the same weights, the CPU checker for every library op).

Orderings: bit-exact.  Every block alone, fed with the CPU statement's own input to that block:
the op tolerance (max-abs 2e-2, see tests/util.max_abs_bound, and relative L2 1e-2).  The whole
forward [N, 24] fp32, where the bf16 mixers and MLPs of four blocks compound: relative L2 <= 1e-2
and max-abs within four times the op bound.
"""
import os

import numpy as np
import pytest
import torch

from tests import model_oracle
from tests.util import assert_close_bf16, err_stats, to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lb():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import lampa_b200
    os.environ["LAMPA_B200_CHECK"] = "1"
    return lampa_b200


def _events(lengths, seed):
    from lampa_b200 import synth
    hits = torch.cat([synth.detector_hits(seed + i, int(n)) for i, n in enumerate(lengths)])
    cu = torch.zeros(len(lengths) + 1, dtype=torch.int64)
    cu[1:] = torch.tensor([int(n) for n in lengths]).cumsum(0)
    return hits, cu


def _model(max_hits):
    from lampa_b200.model import LSHGatedDelta
    torch.manual_seed(20254)
    return LSHGatedDelta(max_hits_per_event=max_hits)


def test_small_events_match_cpu_statement(lb):
    """Ragged events, one shorter than a chunk, one empty."""
    lengths = [700, 63, 0, 1500, 64, 2049]
    hits, cu = _events(lengths, 7)
    m = _model(4096)
    ref, perms_ref, parts, streams = model_oracle.forward(m, hits, cu, return_parts=True)
    md = m.to("cuda:0")
    cud = cu.to("cuda:0")
    perms = md.orderings(hits.to("cuda:0"), cud)
    np.testing.assert_array_equal(to_np(perms), perms_ref)
    assert all(p[0] > 0.02 * p[1] for p in parts), "the mixer must contribute to the residual stream"
    for b, blk in enumerate(md.blocks):          # each block on the CPU statement's input to it
        got = blk(streams[b].to("cuda:0"), perms[b % md.rounds], cud)
        assert_close_bf16(to_np(got), streams[b + 1].numpy(), f"block {b} alone")
    out = md(hits.to("cuda:0"), cud)
    lb.check_status()
    assert_close_bf16(to_np(out), ref.numpy(), "model, ragged small events", max_abs_factor=4.0)


def test_events_of_the_benchmark_size_range(lb):
    from lampa_b200 import synth
    lengths = synth.event_sizes(20254, 64)[:8].tolist()        # 6 259 ... 51 410 hits
    hits, cu = _events(lengths, 20254)
    m = _model(60000)
    ref = model_oracle.forward(m, hits, cu)
    md = m.to("cuda:0")
    out = md(hits.to("cuda:0"), cu.to("cuda:0"))
    lb.check_status()
    assert_close_bf16(to_np(out), ref.numpy(), f"model, 8 events ({sum(lengths)} hits)", max_abs_factor=4.0)


def test_event_shards_reproduce_the_packed_forward(lb):
    """What a rank computes on its share of the events equals those events' rows of the whole batch."""
    from lampa_b200 import sharding
    lengths = [3000, 500, 1800, 2500, 64, 1200, 900]
    hits, cu = _events(lengths, 11)
    md = _model(4096).to("cuda:0")
    full = md(hits.to("cuda:0"), cu.to("cuda:0"))
    plan = sharding.lpt_assign(lengths, 3)
    assert sharding.imbalance(lengths, plan) < 1.2
    for owned in plan:
        local, cu_l = sharding.shard_events(hits, lengths, owned)
        out = md(local.to("cuda:0"), cu_l.to("cuda:0"))
        want = torch.cat([full[cu[e]:cu[e + 1]] for e in owned])
        mx, rl = err_stats(to_np(out), to_np(want))
        assert rl <= 1e-3, (owned, mx, rl)
    with pytest.raises(ValueError):
        md.check_event_sizes([70000])
