"""Drop-in host side of the LSH ordering ops.

Mirrors, by name and argument meaning:
  E2LSH, lsh_mapping                models/model_utils/hash_utils.py:333-371
  LSHOrdering                       models/baselines/hmamba.py:288-353
  invert_permutation                models/model_utils/hash_utils.py:46-57
  batched_index_select              models/model_utils/hash_utils.py:83-93
  sort_to_buckets / unsort_from_buckets   models/attention/hept.py:9-19
and adds the integer bucket ids (floor((a.x + b) / w)) with their stable sort, which the
reference never computes.  All data movement and sorting runs in the CUDA library.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch
import torch.nn as nn

from . import _lib as L


# ---- thin wrappers over the C ABI ------------------------------------------------------------------
@torch.no_grad()
def lsh_hash(x: torch.Tensor, alpha: torch.Tensor, beta: torch.Tensor, w: float = 1.0, *,
             dim: Optional[int] = None, per_head_rows: bool = False, want_ids: bool = True,
             want_keys: bool = False, want_packed: bool = False):
    """Hash rows of x.

    x: fp32 [N, row] (first `dim` floats hashed; shared by all heads) or, with per_head_rows,
    [heads, N, dim].  alpha [heads, dim, rounds], beta [rounds] or [1, rounds].
    Returns a dict with 'ids' int32 [rounds, heads, N], 'keys' fp32 [rounds, heads, N] (a.x),
    'packed' int32 [rounds, N] (sum_h ids << h) for the requested outputs.
    """
    dev = L.require_cuda(x, alpha, beta)
    heads, d, rounds = alpha.shape
    dim = d if dim is None else dim
    if dim != d:
        raise ValueError("alpha's middle dimension must equal dim")
    # head-major rows that sit in padded storage (last stride 1, heads dense over the row pitch) are read in place
    in_place = (per_head_rows and x.dim() == 3 and x.dtype == torch.float32 and x.stride(2) == 1
                and x.stride(1) >= x.shape[2] and x.stride(0) == x.stride(1) * x.shape[1])
    if not in_place:
        x = x.to(torch.float32).contiguous()
    alpha = alpha.detach().to(torch.float32).contiguous()
    beta = beta.detach().to(torch.float32).reshape(-1).contiguous()
    if beta.numel() != rounds:
        raise ValueError("beta must have one offset per round")
    if per_head_rows:
        if x.dim() != 3 or x.shape[0] != heads or x.shape[2] != dim:
            raise ValueError("x must be [heads, N, dim]")
        N, row_stride, head_stride = x.shape[1], x.stride(1), x.stride(0)
    else:
        if x.dim() != 2 or x.shape[1] < dim:
            raise ValueError("x must be [N, row >= dim]")
        N, row_stride, head_stride = x.shape[0], x.shape[1], 0
    out = {}
    ids = torch.empty(rounds, heads, N, dtype=torch.int32, device=dev) if want_ids else None
    keys = torch.empty(rounds, heads, N, dtype=torch.float32, device=dev) if want_keys else None
    packed = torch.empty(rounds, N, dtype=torch.int32, device=dev) if want_packed else None
    rc = L.lib().lampa_lsh_hash(L.ptr(x), row_stride, head_stride, L.ptr(alpha), L.ptr(beta), float(w), N,
                                heads, rounds, dim, L.ptr(ids), L.ptr(keys), L.ptr(packed), L.stream_ptr(dev))
    L.check(rc, "lampa_lsh_hash")
    if want_ids:
        out["ids"] = ids
    if want_keys:
        out["keys"] = keys
    if want_packed:
        out["packed"] = packed
    return out


@torch.no_grad()
def segmented_sort(keys: torch.Tensor, seg_offsets: Optional[torch.Tensor] = None, nseg: Optional[int] = None,
                   init: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Stable ascending sort per segment of a flat int32 / fp32 key array.

    Segments come from `seg_offsets` (int64 [nseg+1]) or are `nseg` equal parts.  Returns int64
    indices local to each segment.  With `init` (a starting order per segment) the result is
    init[stable_sort(keys[init])] — the norm pre-sort followed by the key sort of LSHOrdering.
    """
    dev = L.require_cuda(keys, init)
    if keys.dtype == torch.int32:
        kt = L.LAMPA_KEY_I32
    elif keys.dtype == torch.float32:
        kt = L.LAMPA_KEY_F32
    else:
        raise TypeError("keys must be int32 or float32")
    flat = keys.contiguous().view(-1)
    n = flat.numel()
    if seg_offsets is not None:
        seg_offsets = seg_offsets.to(device=dev, dtype=torch.int64).contiguous()
        nseg = seg_offsets.numel() - 1
    elif nseg is None:
        nseg = 1
    if init is not None:
        init = init.to(torch.int64).contiguous().view(-1)
    perm = torch.empty(n, dtype=torch.int64, device=dev)
    nb = ctypes.c_size_t(0)
    L.check(L.lib().lampa_segsort_workspace_bytes(n, ctypes.byref(nb)), "lampa_segsort_workspace_bytes")
    ws = torch.empty(nb.value, dtype=torch.uint8, device=dev)
    rc = L.lib().lampa_segsort_stable(L.ptr(flat), kt, n, L.ptr(seg_offsets), nseg, L.ptr(init), L.ptr(perm),
                                      L.ptr(ws), ws.numel(), L.ptr(L.status_word(dev)), L.stream_ptr(dev))
    L.check(rc, "lampa_segsort_stable")
    return perm


@torch.no_grad()
def permute_rows(src: torch.Tensor, perm: torch.Tensor, seg_offsets: Optional[torch.Tensor] = None,
                 nseg: int = 1, scatter: bool = False) -> torch.Tensor:
    """dst[s0+i] = src[s0+perm[s0+i]] per segment (or the scatter form); src is [rows, ...]."""
    dev = L.require_cuda(src, perm)
    src = src.contiguous()
    rows = perm.numel()
    if src.shape[0] != rows:
        src = src.view(rows, -1)
    row_bytes = src[0].numel() * src.element_size() if rows else src.element_size()
    if row_bytes % 4:
        raise ValueError("row size must be a multiple of 4 bytes")
    perm = perm.to(torch.int64).contiguous().view(-1)
    if seg_offsets is not None:
        seg_offsets = seg_offsets.to(device=dev, dtype=torch.int64).contiguous()
        nseg = seg_offsets.numel() - 1
    dst = torch.empty_like(src)
    rc = L.lib().lampa_permute_rows(L.ptr(src), L.ptr(perm), L.ptr(seg_offsets), nseg, rows, row_bytes,
                                    int(scatter), L.ptr(dst), L.ptr(L.status_word(dev)), L.stream_ptr(dev))
    L.check(rc, "lampa_permute_rows")
    return dst


# ---- reference-named entry points ----------------------------------------------------------------------
@torch.no_grad()
def invert_permutation(perm: torch.Tensor) -> torch.Tensor:
    """perm: (..., n) -> inverse permutation along the last axis (hash_utils.py:46-57)."""
    dev = L.require_cuda(perm)
    p = perm.to(torch.int64).contiguous()
    n = p.shape[-1]
    inv = torch.empty_like(p)
    nseg = p.numel() // n if n else 1
    rc = L.lib().lampa_invert_perm(L.ptr(p), None, max(nseg, 1), p.numel(), L.ptr(inv), L.ptr(L.status_word(dev)),
                                   L.stream_ptr(dev))
    L.check(rc, "lampa_invert_perm")
    return inv


@torch.no_grad()
def batched_index_select(values: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """values (1 or n_hashes, batch, seqlen, dim), indices (n_hashes, batch, seqlen)
    -> (n_hashes, batch, seqlen, dim) (hash_utils.py:83-93)."""
    h, b, s = indices.shape
    d = values.shape[-1]
    if values.shape[0] == h:
        return permute_rows(values.reshape(h * b * s, d), indices.reshape(-1), nseg=h * b).view(h, b, s, d)
    out = [permute_rows(values[0].reshape(b * s, d), indices[i].reshape(-1), nseg=b) for i in range(h)]
    return torch.stack(out, 0).view(h, b, s, d)


def sort_to_buckets(x: torch.Tensor, perm: torch.Tensor, bucketsz: int) -> torch.Tensor:
    """x (b, s, d), perm (h, b, s) -> (h, b, s/bucketsz, bucketsz, d) (hept.py:9-14)."""
    h, b, s = perm.shape
    g = batched_index_select(x.unsqueeze(0), perm)
    return g.view(h, b, s // bucketsz, bucketsz, x.shape[-1])


def unsort_from_buckets(s_x: torch.Tensor, perm_inverse: torch.Tensor) -> torch.Tensor:
    """s_x (h, b, nbuckets, bucketsz, d), perm_inverse (h, b, s) -> (h, b, s, d) (hept.py:17-19)."""
    h, b, nb, bs, d = s_x.shape
    return batched_index_select(s_x.reshape(h, b, nb * bs, d), perm_inverse)


class E2LSH(nn.Module):
    """Parameters and forward of the reference E2LSH (hash_utils.py:359-371).

    forward(vecs [n_heads, N, dim]) -> float projections [n_hashes, n_heads, N]
    (`bmm(vecs, alpha).permute(2, 0, 1)`).  `bucket_ids` adds the quantised ids.
    """

    def __init__(self, n_hashes: int, n_heads: int, dim: int, r: float = 1.0):
        super().__init__()
        self.alpha = nn.Parameter(torch.normal(0, 1, (n_heads, dim, n_hashes)), requires_grad=False)
        self.beta = nn.Parameter(torch.rand(1, n_hashes) * r, requires_grad=False)
        self.r = float(r)

    def forward(self, vecs: torch.Tensor) -> torch.Tensor:
        return lsh_hash(vecs, self.alpha, self.beta, self.r, per_head_rows=True,
                        want_ids=False, want_keys=True)["keys"]

    def bucket_ids(self, vecs: torch.Tensor, w: Optional[float] = None) -> torch.Tensor:
        return lsh_hash(vecs, self.alpha, self.beta, self.r if w is None else w, per_head_rows=True)["ids"]


@torch.no_grad()
def lsh_mapping(e2lsh: E2LSH, queries: torch.Tensor, keys: torch.Tensor):
    """(queries_hashed, keys_hashed, hash_shift) as hash_utils.py:333-340."""
    qh = e2lsh(queries)
    kh = e2lsh(keys)
    mx = torch.max(qh.max(-1, keepdim=True).values, kh.max(-1, keepdim=True).values)
    mn = torch.min(qh.min(-1, keepdim=True).values, kh.min(-1, keepdim=True).values)
    return qh, kh, mx - mn


class LSHOrdering(nn.Module):
    """Reorders each event's points by an LSH key (hmamba.py:288-353).

    forward(points [B,L,D], coords [B,L,C] or None) -> (ordered_points [B,L,D], indices [B,L]).
    key = sum_i 2^i * (coords . alpha[0,:,i]); rows are pre-sorted by ||coords|| and then stably
    sorted by key.  (With the reference's single head its shift term is identically zero.)
    """

    def __init__(self, input_dim: int, num_hashes: int = 3):
        super().__init__()
        self.num_hashes = num_hashes
        self.e2lsh = E2LSH(self.num_hashes, n_heads=1, dim=input_dim)

    @torch.no_grad()
    def bucket_keys(self, coords: torch.Tensor) -> torch.Tensor:
        B, Ln, C = coords.shape
        flat = coords.reshape(B * Ln, C)
        proj = lsh_hash(flat, self.e2lsh.alpha, self.e2lsh.beta, 1.0, want_ids=False, want_keys=True)["keys"]
        expo = torch.tensor([2.0 ** i for i in range(self.num_hashes)], device=coords.device)
        return (proj[:, 0, :] * expo[:, None]).sum(0).view(B, Ln)

    @torch.no_grad()
    def forward(self, points: torch.Tensor, coords: torch.Tensor = None) -> Tuple[torch.Tensor, torch.Tensor]:
        B, Ln, D = points.shape
        c = points if coords is None else coords
        c = c.to(torch.float32)
        keys = self.bucket_keys(c)
        norm = c.norm(dim=-1)
        norm_idx = segmented_sort(norm, nseg=B)
        idx = segmented_sort(keys, nseg=B, init=norm_idx).view(B, Ln)
        ordered = permute_rows(points.reshape(B * Ln, D), idx.view(-1), nseg=B).view(B, Ln, D)
        return ordered, idx


@torch.no_grad()
def lsh_bucket_sort(x: torch.Tensor, alpha: torch.Tensor, beta: torch.Tensor, w: float = 1.0,
                    seg_offsets: Optional[torch.Tensor] = None):
    """Integer pipeline of one packed batch: ids [rounds, heads, N] and, per (round, head) row and
    per event, the stable ascending permutation [rounds, heads, N] (int64, local to the event)."""
    ids = lsh_hash(x, alpha, beta, w)["ids"]
    rounds, heads, N = ids.shape
    if seg_offsets is None:
        perm = segmented_sort(ids, nseg=rounds * heads)
    else:
        so = seg_offsets.to(device=ids.device, dtype=torch.int64)
        rows = torch.arange(rounds * heads, device=ids.device, dtype=torch.int64)[:, None] * N
        full = torch.cat([(rows + so[None, :-1]).reshape(-1), torch.tensor([rounds * heads * N], device=ids.device)])
        perm = segmented_sort(ids, seg_offsets=full)
    return ids, perm.view(rounds, heads, N)
