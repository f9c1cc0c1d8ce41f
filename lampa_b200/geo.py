"""Region (geo) shift of the LSH keys, host side.

Same names and argument meaning as the reference:
  get_regions, quantile_partition    models/model_utils/hash_utils.py:14-43
  get_geo_shift                      models/attention/hept.py:78-88
  pad_to_multiple                    models/model_utils/hash_utils.py:61-80
plus the two call sequences they appear in, as single functions:
  region_inputs      prepare_input, models/hattention/modeling_gated_deltaproduct.py:1200-1223
  hept_positions     HEPTAttention.forward up to the bucket positions, models/attention/hept.py:118-138
All device arithmetic runs in the CUDA library (sorts, inverse permutations, ranges, shifted keys).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from . import _lib as L
from .lsh import E2LSH, invert_permutation, segmented_sort


def get_regions(num_regions: int, num_or_hashes: int, num_heads: int, num_and_hashes: int = 2) -> torch.Tensor:
    """Random fractional region counts [num_or_hashes, num_and_hashes, num_heads] whose product
    over the AND axis is num_regions, rounded to thirds (hash_utils.py:30-43).  Host-side
    parameter initialisation; draws one uniform number at a time, like the reference, so that a
    seeded run gives the same regions."""
    lo = 2.0
    hi = 2.0 * num_regions ** (1.0 / num_and_hashes) - lo
    rows = num_or_hashes * num_heads
    draws = torch.tensor([[torch.rand(1).item() * (hi - lo) + lo for _ in range(num_and_hashes)]
                          for _ in range(rows)])
    draws = (num_regions / draws.prod(dim=1, keepdim=True)) ** (1.0 / num_and_hashes) * draws
    draws = torch.round(draws * 3) / 3
    return draws.view(num_heads, num_or_hashes, num_and_hashes).permute(1, 2, 0)     # "(h c) a -> c a h"


def pad_to_multiple(tensor: torch.Tensor, multiple: int, dims=-1, value: float = 0) -> torch.Tensor:
    """Pad the given dims at their end up to a multiple (hash_utils.py:61-80)."""
    dims = [dims] if isinstance(dims, int) else list(dims)
    pad = [0] * (2 * tensor.ndim)
    for d in dims:
        d = d if d >= 0 else tensor.ndim + d
        rem = tensor.size(d) % multiple
        if rem:
            pad[2 * (tensor.ndim - d - 1) + 1] = multiple - rem
    return tensor if not any(pad) else F.pad(tensor, tuple(pad), value=value)


def _rows(x: torch.Tensor) -> torch.Tensor:
    return x.reshape(-1).to(torch.float32).contiguous()


@torch.no_grad()
def ranks_of(values: torch.Tensor) -> torch.Tensor:
    """Rank of each element of a 1-D fp32 tensor in ascending order (stable): the inverse of argsort."""
    return invert_permutation(segmented_sort(values.to(torch.float32).contiguous(), nseg=1))


@torch.no_grad()
def quantile_partition(sorted_indices: torch.Tensor, num_regions: torch.Tensor) -> torch.Tensor:
    """sorted_indices [N] (an argsort), num_regions [R, 1] -> region numbers fp32 [R, N]."""
    dev = L.require_cuda(sorted_indices, num_regions)
    rank = invert_permutation(sorted_indices.to(torch.int64).contiguous())
    return _regions_from_rank(rank, _rows(num_regions), dev)


def _regions_from_rank(rank: torch.Tensor, num_regions: torch.Tensor, dev) -> torch.Tensor:
    R, n = num_regions.numel(), rank.numel()
    out = torch.empty(R, n, dtype=torch.float32, device=dev)
    L.check(L.lib().lampa_quantile_regions(L.ptr(rank), L.ptr(num_regions), R, n, L.ptr(out), L.stream_ptr(dev)),
            "lampa_quantile_regions")
    return out


@torch.no_grad()
def get_geo_shift(regions_h, hash_shift: torch.Tensor, region_indices: Sequence[torch.Tensor],
                  num_or_hashes: int) -> torch.Tensor:
    """regions_h [2, R]; hash_shift [R, 1]; region_indices (eta [R, N], phi [R, N]) ->
    [2, num_or_hashes, heads, N] (the query and key halves are the same numbers)."""
    reg_eta, reg_phi = (x.to(torch.float32).contiguous() for x in region_indices)
    dev = L.require_cuda(reg_eta, reg_phi, hash_shift)
    R, n = reg_eta.shape
    shift = torch.empty(R, n, dtype=torch.float32, device=dev)
    re = _rows(regions_h[0]).to(dev)
    L.check(L.lib().lampa_geo_keys(None, L.ptr(reg_eta), L.ptr(reg_phi), None, None, L.ptr(re), None,
                                   L.ptr(_rows(hash_shift)), R, n, n, L.ptr(shift), L.stream_ptr(dev)),
            "lampa_geo_keys")
    shift = shift.view(num_or_hashes, R // num_or_hashes, n)
    return torch.stack([shift, shift], 0)


@torch.no_grad()
def row_range(a: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """max - min over the last axis of a (and b): the `hash_shift` of lsh_mapping, shape a.shape[:-1] + (1,)."""
    dev = L.require_cuda(a, b)
    a = a.to(torch.float32).contiguous()
    b = None if b is None else b.to(torch.float32).contiguous()
    n = a.shape[-1]
    rows = a.numel() // n
    out = torch.empty(rows, dtype=torch.float32, device=dev)
    L.check(L.lib().lampa_row_range(L.ptr(a), L.ptr(b), rows, n, None, None, L.ptr(out), L.stream_ptr(dev)),
            "lampa_row_range")
    return out.view(*a.shape[:-1], 1)


@torch.no_grad()
def region_inputs(coords: torch.Tensor, regions: torch.Tensor, block_size: int):
    """coords [N_raw, >=2] (eta, phi first), regions [c, a, h] -> dict with the padded coordinates
    (padding rows zeroed, as the reference leaves them), raw_size, regions_h [a, c*h],
    region_indices [eta, phi] (fp32 [R, N]) and the two rank vectors they were made from."""
    dev = L.require_cuda(coords)
    raw = coords.shape[0]
    padded = pad_to_multiple(coords.to(torch.float32), block_size, dims=0, value=float("inf")).contiguous()
    rank_eta = ranks_of(padded[:, 0])
    rank_phi = ranks_of(padded[:, 1])
    regions_h = regions.to(device=dev, dtype=torch.float32).permute(1, 0, 2).reshape(regions.shape[1], -1).contiguous()
    reg_eta = _regions_from_rank(rank_eta, regions_h[0].contiguous(), dev)
    reg_phi = _regions_from_rank(rank_phi, regions_h[1].contiguous(), dev)
    padded[raw:] = 0.0
    return {"coords": padded, "raw_size": raw, "regions_h": regions_h, "region_indices": [reg_eta, reg_phi],
            "ranks": [rank_eta, rank_phi]}


@torch.no_grad()
def hept_positions(e2lsh: E2LSH, q_hat: torch.Tensor, k_hat: torch.Tensor, regions_h: torch.Tensor,
                   ranks: Sequence[torch.Tensor], raw_size: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Bucket order of queries and keys: project, take the joint key range per (round, head) row,
    add the region shift (padded hits -> +inf), sort each row.  q_hat, k_hat [heads, N, dim] with
    the padded rows zeroed; returns (q_positions, k_positions), int64 [rounds, heads, N]."""
    dev = L.require_cuda(q_hat, k_hat)
    qh, kh = e2lsh(q_hat), e2lsh(k_hat)                       # [rounds, heads, N] fp32
    rounds, heads, n = qh.shape
    R = rounds * heads
    hs = row_range(qh, kh).reshape(-1)
    re, rp = (_rows(regions_h[0]).to(dev), _rows(regions_h[1]).to(dev))
    rank_eta, rank_phi = (r.to(torch.int64).contiguous() for r in ranks)
    out = []
    for proj in (qh, kh):
        keys = torch.empty(R, n, dtype=torch.float32, device=dev)
        L.check(L.lib().lampa_geo_keys(L.ptr(proj), None, None, L.ptr(rank_eta), L.ptr(rank_phi), L.ptr(re),
                                       L.ptr(rp), L.ptr(hs), R, n, int(raw_size), L.ptr(keys), L.stream_ptr(dev)),
                "lampa_geo_keys")
        out.append(segmented_sort(keys.view(-1), nseg=R).view(rounds, heads, n))
    return out[0], out[1]
