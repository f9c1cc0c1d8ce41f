"""The allocation-free sort entry point against the workspace-based one.

Some hosts of this library cannot allocate device memory at call time: a reconstruction loop that
reserves everything at start-up and bans cudaMalloc afterwards, or a process whose device memory
is owned by an allocator the library cannot reach.  For them lampa_segsort_stable_static keeps
its ping-pong buffers in a fixed array inside the library.  This file calls it through the C ABI
and requires bit-identical permutations to lampa_segsort_stable, on two calls in a row (the
second smaller, so that it runs over the first call's leftovers), and a clean refusal above the
fixed capacity.  It is named to be collected last.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _sort_both(L, keys, nseg=None, seg=None, init=None, check_free=False):
    dev = keys.device
    lib = L.lib()
    n = keys.numel()
    kt = L.LAMPA_KEY_I32 if keys.dtype == torch.int32 else L.LAMPA_KEY_F32
    st = L.status_word(dev)
    stream = L.stream_ptr(dev)
    nseg = (seg.numel() - 1) if seg is not None else (nseg or 1)
    want = torch.empty(n, dtype=torch.int64, device=dev)
    nb = ctypes.c_size_t(0)
    assert lib.lampa_segsort_workspace_bytes(n, ctypes.byref(nb)) == 0
    ws = torch.empty(nb.value, dtype=torch.uint8, device=dev)
    rc = lib.lampa_segsort_stable(L.ptr(keys), kt, n, L.ptr(seg), nseg, L.ptr(init), L.ptr(want), L.ptr(ws),
                                  ws.numel(), L.ptr(st), stream)
    assert rc == 0
    got = torch.full((n,), -1, dtype=torch.int64, device=dev)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated(dev)
    free_before = torch.cuda.mem_get_info(dev)[0]
    rc = lib.lampa_segsort_stable_static(L.ptr(keys), kt, n, L.ptr(seg), nseg, L.ptr(init), L.ptr(got),
                                         L.ptr(st), stream)
    assert rc == 0, lib.lampa_error_string(rc)
    assert torch.cuda.memory_allocated(dev) == before      # nothing was taken from torch's allocator either
    torch.cuda.synchronize()
    if check_free:
        # the driver's own count of free device memory: it sees a cudaMalloc made inside the library, which
        # torch's counter cannot.  Only meaningful once the library's module image is resident (any call
        # after the first); device allocations come in 2 MiB granules.
        assert free_before - torch.cuda.mem_get_info(dev)[0] < (2 << 20)
    return got, want


def test_static_sort_matches_workspace_sort_on_two_calls_in_a_row():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from lampa_b200 import _lib as L
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(77)
    # call 1: 24 rows of 60000 ids (the benchmark's sort), full-range values in some rows
    k1 = rng.integers(-20000, 20000, size=(24, 60000)).astype(np.int32)
    k1[3] = rng.integers(-2**31, 2**31 - 1, size=60000, dtype=np.int64).astype(np.int32)
    k1 = torch.from_numpy(k1).to(dev)
    got, want = _sort_both(L, k1.view(-1), nseg=24)
    assert torch.equal(got, want)
    ref = np.argsort(k1[3].cpu().numpy(), kind="stable")
    assert np.array_equal(got.view(24, 60000)[3].cpu().numpy(), ref)
    # call 2: smaller, ragged segments, float keys, a starting order: runs over call 1's leftovers
    f = torch.from_numpy(rng.standard_normal(50000).astype(np.float32)).to(dev)
    seg = torch.tensor([0, 1, 1, 4097, 30000, 50000], dtype=torch.int64, device=dev)
    lens = (seg[1:] - seg[:-1]).tolist()
    init = torch.cat([torch.from_numpy(rng.permutation(n).astype(np.int64)) for n in lens]).to(dev)
    got, want = _sort_both(L, f, seg=seg, init=init, check_free=True)
    assert torch.equal(got, want)
    # and once more with the first input: same answer as before
    got2, want2 = _sort_both(L, k1.view(-1), nseg=24, check_free=True)
    assert torch.equal(got2, want2)
    L.check_status(dev)


def test_static_sort_rejects_inputs_beyond_its_capacity():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from lampa_b200 import _lib as L
    dev = torch.device("cuda:0")
    n = L.SEGSORT_STATIC_MAX_KEYS + 1
    keys = torch.zeros(n, dtype=torch.int32, device=dev)
    perm = torch.full((n,), -7, dtype=torch.int64, device=dev)
    rc = L.lib().lampa_segsort_stable_static(L.ptr(keys), L.LAMPA_KEY_I32, n, None, 1, None, L.ptr(perm),
                                             L.ptr(L.status_word(dev)), L.stream_ptr(dev))
    assert rc == L.ERR_TOO_LARGE
    assert "capacity" in L.lib().lampa_error_string(rc).decode()
    torch.cuda.synchronize()
    assert bool((perm == -7).all())          # nothing was launched
    # exactly at the capacity it still works
    n = L.SEGSORT_STATIC_MAX_KEYS
    keys = torch.randint(-1000, 1000, (n,), dtype=torch.int32, device=dev)
    got, want = _sort_both(L, keys, nseg=1)
    assert torch.equal(got, want)
