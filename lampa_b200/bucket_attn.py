"""Bucketed RBF-kernel attention of the HEPT layer, host side.

Same names and argument meaning as the reference:
  qkv_res(s_query, s_key, s_value) -> (denom, so)          models/attention/hept.py:22-33
  prep_qk(query, key, w, coords) -> (q_hat, k_hat)         models/attention/hept.py:55-63
plus `hept_bucket_attention`, the statements of HEPTAttention.forward from `sort_to_buckets` to
`o.sum(0) / logits.sum(0)` (hept.py:141-151) as one call that gathers by position inside the
kernel instead of materialising the sorted copies, and `hept_attention_core`, the whole forward
between the q/k/v projections and the output projection (hept.py:108-151).  fp32, forward only;
everything runs in the CUDA library on the current stream.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch

from . import _lib as L
from .geo import hept_positions


def _f32(t: torch.Tensor) -> torch.Tensor:
    if t.dtype != torch.float32:
        raise TypeError("bucket attention runs in fp32")
    return t.contiguous()


_ZERO_PADDED = "_lampa_zero_padded_rows"


def assume_zero_padded(t: torch.Tensor) -> torch.Tensor:
    """Declare that the storage columns between this view's width and its row pitch hold zeros, so
    that `hept_bucket_attention` may read the rows in place with 16-byte fetches."""
    setattr(t, _ZERO_PADDED, True)
    return t


def _rows(t: torch.Tensor):
    """(tensor, row pitch) of a [..., rows, width] fp32 tensor: a dense view of padded storage
    (last stride 1, every leading axis dense over the row pitch) is passed as it is, anything
    else is made contiguous.  The kernel's 16-byte row fetch reads a row up to its width rounded
    up to 4 floats and needs those extra columns to be zero, so a view narrower than its pitch
    is only taken in place when its width is a multiple of 4 or when `prep_qk` produced it (it
    writes the padding as zeros and marks the tensor); a slice of wider storage that holds other
    data is copied."""
    if t.dtype != torch.float32:
        raise TypeError("bucket attention runs in fp32")
    ld = t.stride(-2) if t.dim() >= 2 else t.shape[-1]
    ok = t.stride(-1) == 1 and ld >= t.shape[-1]
    ok = ok and (ld == t.shape[-1] or t.shape[-1] % 4 == 0 or getattr(t, _ZERO_PADDED, False))
    pitch = ld
    for ax in range(t.dim() - 2, -1, -1):
        ok = ok and (t.stride(ax) == pitch or t.shape[ax] == 1)
        pitch *= t.shape[ax]
    if ok:
        return t, ld
    t = t.contiguous()
    return t, t.shape[-1]


@torch.no_grad()
def qkv_res(s_query: torch.Tensor, s_key: torch.Tensor, s_value: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """s_query, s_key [..., buckets, bucketsz, dq], s_value [..., buckets, bucketsz, dv], rows already
    in bucket order -> (denom [..., buckets, bucketsz, 1], so [..., buckets, bucketsz, dv])."""
    dev = L.require_cuda(s_query, s_key, s_value)
    q, k, v = _f32(s_query), _f32(s_key), _f32(s_value)
    if q.shape != k.shape or q.shape[:-1] != v.shape[:-1] or q.dim() < 2:
        raise ValueError("qkv_res: s_query / s_key / s_value shapes do not match")
    bucket, dq, dv = q.shape[-2], q.shape[-1], v.shape[-1]
    n = q.numel() // dq                       # every bucket is independent: one (round, head) row of n hits
    so = torch.empty(v.shape, dtype=torch.float32, device=dev)
    denom = torch.empty(v.shape[:-1] + (1,), dtype=torch.float32, device=dev)
    rc = L.lib().lampa_bucket_rbf_attn(L.ptr(q), L.ptr(k), L.ptr(v), None, None, 1, 1, n, bucket, dq, dv, dq, dv, 1, 0,
                                       L.ptr(so), L.ptr(denom), L.stream_ptr(dev))
    L.check(rc, "lampa_bucket_rbf_attn")
    return denom, so


@torch.no_grad()
def hept_bucket_attention(q_hat: torch.Tensor, k_hat: torch.Tensor, value: torch.Tensor, q_positions: torch.Tensor,
                          k_positions: torch.Tensor, block_size: int, return_parts: bool = False):
    """q_hat, k_hat [heads, N, dq], value [heads, N, dv], q_positions / k_positions int64
    [rounds, heads, N] (the argsorts of the shifted keys) -> out [heads, N, dv]: per round the
    hits are bucketed in position order, attended inside buckets, written back to hit order;
    rounds are summed and so / denom returned.  return_parts: also (o [rounds, heads, N, dv],
    logits [rounds, heads, N, 1]), the tensors the reference sums."""
    dev = L.require_cuda(q_hat, k_hat, value, q_positions, k_positions)
    (q, ldq), (k, ldk), (v, ldv) = _rows(q_hat), _rows(k_hat), _rows(value)
    if ldk != ldq:
        q, k, ldq = q.contiguous(), k.contiguous(), q.shape[-1]
    heads, n, dq = q.shape
    dv = v.shape[-1]
    if k.shape != q.shape or v.shape[:2] != q.shape[:2]:
        raise ValueError("hept_bucket_attention: q_hat / k_hat / value shapes do not match")
    rounds = q_positions.shape[0]
    if tuple(q_positions.shape) != (rounds, heads, n) or tuple(k_positions.shape) != (rounds, heads, n):
        raise ValueError("positions must be [rounds, heads, N]")
    if n % block_size != 0:
        raise ValueError("N must be a multiple of block_size (pad_to_multiple)")
    qp = q_positions.to(torch.int64).contiguous()
    kp = k_positions.to(torch.int64).contiguous()
    so = torch.empty(rounds, heads, n, dv, dtype=torch.float32, device=dev)
    denom = torch.empty(rounds, heads, n, 1, dtype=torch.float32, device=dev)
    s = L.stream_ptr(dev)
    rc = L.lib().lampa_bucket_rbf_attn(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(qp), L.ptr(kp), rounds, heads, n,
                                       int(block_size), dq, dv, ldq, ldv, 0, 1, L.ptr(so), L.ptr(denom), s)
    L.check(rc, "lampa_bucket_rbf_attn")
    out = torch.empty(heads, n, dv, dtype=torch.float32, device=dev)
    L.check(L.lib().lampa_bucket_attn_combine(L.ptr(so), L.ptr(denom), rounds, heads * n, dv, L.ptr(out), s),
            "lampa_bucket_attn_combine")
    return (out, so, denom) if return_parts else out


def _coord_scale(w: torch.Tensor) -> torch.Tensor:
    """sqrt(2 * [qw_0, qw_0, qw_1, ...]) with qw = exp(min(sum_d w, 50)) summed over the k
    weights per distance: [heads, r + 1] from the relative-position weights w [heads, d, r, k]
    (parameter-sized; hept.py:56-59)."""
    qw = w.sum(dim=1).clamp(max=50).exp().sum(dim=-1)
    return torch.sqrt(2 * torch.cat([qw[:, :1], qw], dim=-1)).to(torch.float32).contiguous()


@torch.no_grad()
def prep_qk(query: torch.Tensor, key: torch.Tensor, w: torch.Tensor, coords: torch.Tensor,
            value: Optional[torch.Tensor] = None, raw_size: Optional[int] = None, head_major: bool = False):
    """query, key [N, heads, d], coords [N, r + 1] -> (q_hat, k_hat) [N, heads, d + r + 1] as the
    reference; head_major=True returns them as [heads, N, d + r + 1] (what the attention consumes)
    with rows >= raw_size zeroed, and the value rearranged alongside when given."""
    dev = L.require_cuda(query, key, coords, w, value)
    q, k, c = _f32(query), _f32(key), _f32(coords)
    n, heads, d = q.shape
    cd = c.shape[-1]
    scale = _coord_scale(w.detach())
    if tuple(scale.shape) != (heads, cd):
        raise ValueError("w must be [heads, d, coords_dim - 1, k]")
    v = None if value is None else _f32(value)
    ldq = (d + cd + 3) // 4 * 4                 # rows padded with zeros to whole 16-byte pieces
    qh = torch.empty(heads, n, ldq, dtype=torch.float32, device=dev)
    kh = torch.empty_like(qh)
    vo = None if v is None else torch.empty(heads, n, v.shape[-1], dtype=torch.float32, device=dev)
    if v is not None and v.shape[-1] != d:
        raise ValueError("value must have the head dim of query")
    rc = L.lib().lampa_hept_prep_qk(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(scale), L.ptr(c), n, heads, d, cd, ldq,
                                    n if raw_size is None else int(raw_size), L.ptr(qh), L.ptr(kh), L.ptr(vo),
                                    L.stream_ptr(dev))
    L.check(rc, "lampa_hept_prep_qk")
    qh, kh = qh[..., :d + cd], kh[..., :d + cd]      # views of the padded rows
    assume_zero_padded(qh)                           # columns d + cd .. ldq - 1 are zero: _rows may pass them in place
    assume_zero_padded(kh)
    if head_major:
        return (qh, kh) if v is None else (qh, kh, vo)
    return qh.transpose(0, 1), kh.transpose(0, 1)


@torch.no_grad()
def hept_attention_core(e2lsh, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, w: torch.Tensor,
                        coords: torch.Tensor, regions_h: torch.Tensor, ranks: Sequence[torch.Tensor],
                        raw_size: int, block_size: int) -> torch.Tensor:
    """HEPTAttention.forward between the projections and `out_linear`: query, key, value
    [N, heads, d] (N padded to block_size), coords [N, r + 1] with the padded rows zeroed, `ranks`
    the (eta, phi) ranks of the hits (geo.region_inputs) -> [heads, N, d]."""
    q_hat, k_hat, v = prep_qk(query, key, w, coords, value=value, raw_size=raw_size, head_major=True)
    q_pos, k_pos = hept_positions(e2lsh, q_hat, k_hat, regions_h, ranks, raw_size)
    return hept_bucket_attention(q_hat, k_hat, v, q_pos, k_pos, block_size)
