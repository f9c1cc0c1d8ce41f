"""CPU-side checks: the C-ABI library loads and exports what the header declares, host-side
argument validation, and the multi-rank sharding plan (2 gloo ranks)."""
import os
import re
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from lampa_b200 import _lib, build
    build.build()
    hdr = open(os.path.join(ROOT, "include", "lampa_b200.h")).read()
    declared = sorted(set(re.findall(r"\b(lampa_[a-z0-9_]+)\s*\(", hdr)))
    assert declared, "no declarations found"
    lib = _lib.lib()
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert lib.lampa_version() >= 100
    assert lib.lampa_error_string(-6).decode().startswith("lambda")


def test_host_side_argument_errors_without_a_gpu():
    import ctypes
    from lampa_b200 import _lib
    lib = _lib.lib()
    n = ctypes.c_size_t(0)
    bad = _lib.GdnDesc(B=1, T=128, H=2, K=48, V=64, L=0, nseq=0, qkv_dtype=0, gb_dtype=2, lam_dtype=2, use_l2norm=1, scale=0.1)
    assert lib.lampa_gdn_workspace_bytes(ctypes.byref(bad), ctypes.byref(n)) == -2          # unsupported head dim
    ok = _lib.GdnDesc(B=1, T=61440, H=8, K=64, V=64, L=17, nseq=0, qkv_dtype=0, gb_dtype=2, lam_dtype=0, use_l2norm=1, scale=0.1)
    assert lib.lampa_gdn_workspace_bytes(ctypes.byref(ok), ctypes.byref(n)) == 0
    assert 300e6 < n.value < 600e6
    lay = (ctypes.c_size_t * 12)()
    assert lib.lampa_gdn_workspace_layout(ctypes.byref(ok), lay) == 0
    assert lay[1] % 128 == 0 and lay[7] == 10 and lay[9] == 32
    assert lib.lampa_segsort_workspace_bytes(-1, ctypes.byref(n)) == -1
    assert lib.lampa_lsh_hash(None, 24, 0, None, None, 1.0, 10, 8, 3, 6, None, None, None, None) == -1
    assert lib.lampa_permute_rows(None, None, None, 1, 10, 6, 0, None, None, None) == -1            # row bytes not /4
    assert lib.lampa_bucket_rbf_attn(None, None, None, None, None, 3, 8, 1000, 30, 30, 24, 32, 24, 0, 1, None, None, None) == -1   # n % bucket
    assert lib.lampa_bucket_rbf_attn(None, None, None, None, None, 3, 8, 900, 300, 30, 24, 30, 24, 0, 1, None, None, None) == -1   # null tensors
    assert lib.lampa_bucket_rbf_attn(None, None, None, None, None, 3, 8, 900, 100, 30, 24, 28, 24, 0, 1, None, None, None) == -1   # pitch < width
    assert lib.lampa_bucket_attn_combine(None, None, 0, 10, 4, None, None) == -1
    assert lib.lampa_hept_prep_qk(None, None, None, None, None, 10, 0, 4, 2, 8, 10, None, None, None, None) == -1


def test_python_api_rejects_cpu_tensors_and_bad_shapes():
    import lampa_b200
    q = torch.randn(1, 128, 2, 64).bfloat16()
    with pytest.raises(AssertionError):          # fp32 q / k / v are refused, as by the reference
        lampa_b200.chunk_gated_delta_rule(q.float(), q.float(), q.float(), torch.zeros(1, 128, 2), torch.zeros(1, 128, 2))
    with pytest.raises(NotImplementedError):     # forward only: no silent detach
        qg = q.clone().requires_grad_(True)
        lampa_b200.chunk_gated_delta_rule(qg, qg, qg, torch.zeros(1, 128, 2), torch.zeros(1, 128, 2))
    with pytest.raises(ValueError):              # host-resident cu_seqlens are validated on the host
        lampa_b200.chunk_gated_delta_rule(q, q, q, torch.zeros(1, 128, 2), torch.zeros(1, 128, 2), cu_seqlens=torch.tensor([0, 200]))
    with pytest.raises(lampa_b200.LampaError):
        lampa_b200.chunk_gated_delta_rule(q, q, q, torch.zeros(1, 128, 2), torch.zeros(1, 128, 2))
    with pytest.raises(DeprecationWarning):
        lampa_b200.chunk_gated_delta_rule(q, q, q, torch.zeros(1, 128, 2), torch.zeros(1, 128, 2), head_first=True)
    with pytest.raises(AssertionError):
        lampa_b200.chunk_gated_delta_rule(q, q.half(), q, torch.zeros(1, 128, 2), torch.zeros(1, 128, 2))
    with pytest.raises(lampa_b200.LampaError):
        lampa_b200.segmented_sort(torch.zeros(10, dtype=torch.int32))
    assert lampa_b200.num_levels_required(61440) == 17 and lampa_b200.num_levels_required(64) == 7
    assert lampa_b200.num_levels_required(65536) == 17 and lampa_b200.num_levels_required(65537) == 18


def test_lpt_plan_properties():
    from lampa_b200 import sharding, synth
    lens = synth.event_sizes(20254, 64).tolist()
    for g in (1, 2, 4, 8):
        plan = sharding.lpt_assign(lens, g)
        assert sorted(e for o in plan for e in o) == list(range(64))
        assert sharding.imbalance(lens, plan) < 1.03
    cu, spans = sharding.pack_events(lens, plan[3])
    assert cu[-1].item() == sum(lens[e] for e in plan[3]) and len(spans) == len(plan[3])
    assert sharding.head_slice(8, 3, 4) == (6, 8)
    with pytest.raises(ValueError):
        sharding.head_slice(6, 0, 4)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, lens):
    sys.path.insert(0, ROOT)
    from lampa_b200 import sharding
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # rank 1 starts from different (wrong) lengths: the plan must come from rank 0
        mine = torch.tensor(lens if rank == 0 else [1] * len(lens), dtype=torch.int64)
        plan = sharding.agree_on_plan(mine)
        assert plan == sharding.lpt_assign(lens, world)
        owned = plan[rank]
        # each event's "output" is its global row index: after the gather every rank holds 0..N-1
        starts = [0]
        for n in lens:
            starts.append(starts[-1] + n)
        local = torch.cat([torch.arange(starts[e], starts[e + 1], dtype=torch.float32)[:, None].repeat(1, 3)
                           for e in owned]) if owned else torch.zeros(0, 3)
        full = sharding.gather_event_outputs(local, lens, plan)
        assert torch.equal(full[:, 0], torch.arange(starts[-1], dtype=torch.float32))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_rank_plan_and_gather_over_gloo():
    lens = [700, 60, 1500, 333, 64, 900, 5]
    mp.spawn(_rank_main, args=(2, _free_port(), lens), nprocs=2, join=True)


def _head_rank_main(rank, world, port):
    sys.path.insert(0, ROOT)
    from lampa_b200 import sharding
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, T, H, V = 1, 37, 6, 5
        full = torch.arange(B * T * H * V, dtype=torch.float32).view(B, T, H, V)
        h0, h1 = sharding.head_slice(H, rank, world)
        assert (h0, h1) == (rank * H // world, (rank + 1) * H // world)
        got = sharding.gather_heads(full[:, :, h0:h1])        # a strided view: gather_heads makes it dense
        assert torch.equal(got, full)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_rank_head_split_and_gather_over_gloo():
    mp.spawn(_head_rank_main, args=(2, _free_port()), nprocs=2, join=True)
    from lampa_b200 import sharding
    with pytest.raises(ValueError):
        sharding.head_slice(8, 0, 3)


class _EventMeanModel:
    """Stand-in for the packed model on CPU ranks: every row minus its event's mean (so that a
    wrong event boundary or a wrong gather position shows), three output columns."""

    class _Head:
        out_features = 3

    head = _Head()

    def check_event_sizes(self, lengths):
        pass

    def __call__(self, hits, cu):
        out = torch.empty(hits.shape[0], 3)
        for s, e in zip(cu[:-1].tolist(), cu[1:].tolist()):
            out[s:e] = hits[s:e, :3] - hits[s:e, :3].mean(0, keepdim=True)
        return out


def _sharded_rank_main(rank, world, port, lens):
    sys.path.insert(0, ROOT)
    from lampa_b200.model import forward_sharded
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        gen = torch.Generator().manual_seed(5)
        hits = torch.randn(sum(lens), 4, generator=gen)
        model = _EventMeanModel()
        cu = torch.tensor([0] + lens).cumsum(0)
        want = model(hits, cu)
        got, info = forward_sharded(model, hits, lens)
        assert torch.equal(got, want)
        assert info["imbalance"] >= 1.0 and info["owned"] >= 1
        local, _ = forward_sharded(model, hits, lens, gather=False)
        assert local.shape[0] < hits.shape[0]
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_rank_sharded_forward_over_gloo():
    lens = [700, 60, 1500, 333, 64, 900, 5]
    mp.spawn(_sharded_rank_main, args=(2, _free_port(), lens), nprocs=2, join=True)


def test_get_regions_matches_reference_draws(golden_dir):
    """Seeded region counts equal the reference's get_regions (fixture written by gen_golden.py)."""
    import numpy as np
    import torch
    from lampa_b200.geo import get_regions, pad_to_multiple
    z = np.load(os.path.join(golden_dir, "geo_shift_N1090_R12.npz"))
    torch.manual_seed(11)
    r = get_regions(40, 3, 4)
    assert tuple(r.shape) == (3, 2, 4)
    np.testing.assert_array_equal(r.numpy(), z["regions"])
    x = torch.arange(10.0).view(5, 2)
    p = pad_to_multiple(x, 4, dims=0, value=float("inf"))
    assert tuple(p.shape) == (8, 2) and torch.isinf(p[5:]).all() and torch.equal(p[:5], x)
    assert pad_to_multiple(x, 5, dims=0) is x


def test_dispatcher_entries_have_shape_functions():
    """torch.ops.lampa_b200.{gdn_fwd, hgdn_fwd}: the shape functions answer for meta tensors (what a tracer sees)."""
    from lampa_b200 import torch_ops  # noqa: F401
    B, T, H, K, V, Lv = 1, 300, 3, 64, 64, 10
    m = lambda *s, dt=torch.bfloat16: torch.empty(*s, dtype=dt, device="meta")
    q, k, v = m(B, T, H, K), m(B, T, H, K), m(B, T, H, V)
    g, beta = m(B, T, H, dt=torch.float32), m(B, T, H, dt=torch.float32)
    o, ht = torch.ops.lampa_b200.gdn_fwd(q, k, v, g, beta, 0.125, None, None, True)
    assert o.shape == (B, T, H, V) and o.dtype == torch.bfloat16 and ht.shape == (B, H, K, V) and ht.dtype == torch.float32
    cu = torch.empty(5, dtype=torch.int64, device="meta")
    o, ht = torch.ops.lampa_b200.gdn_fwd(q, k, v, g, beta, 0.125, None, cu, True)
    assert ht.shape == (4, H, K, V)
    o = torch.ops.lampa_b200.hgdn_fwd(q, k, v, g, beta, m(B, T, H, Lv), None, True)
    assert o.shape == (B, T, H, V) and o.dtype == torch.bfloat16
