"""Dispatcher entries for the two gated-delta forwards.

`torch.ops.lampa_b200.gdn_fwd` and `torch.ops.lampa_b200.hgdn_fwd` are `torch.library` custom ops around the same
C-ABI calls the eager functions make, with shape functions registered for fake tensors.  They exist so that code
calling `chunk_gated_delta_rule` / `chunk_h_gated_delta_rule` can be traced (torch.compile, export): while a
trace is being taken the public functions route through these ops, so the graph holds one opaque node per call
instead of a graph break at the ctypes boundary.  Eager calls do not pay the dispatcher's per-call overhead.
Forward only, like the eager functions (no autograd formula is registered).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import gated_delta as _gd


@torch.library.custom_op("lampa_b200::gdn_fwd", mutates_args=(), device_types="cuda")
def gdn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor, scale: float,
            initial_state: Optional[torch.Tensor], cu_seqlens: Optional[torch.Tensor],
            use_l2norm: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    """Plain rule: (o [B,T,H,V] in q's dtype, final state [N,H,K,V] fp32)."""
    o, ht = _gd._gdn_plain(q, k, v, g, beta, scale, initial_state, True, cu_seqlens, use_l2norm)
    return o, ht


@gdn_fwd.register_fake
def _(q, k, v, g, beta, scale, initial_state, cu_seqlens, use_l2norm):
    B, T, H, K = q.shape
    V = v.shape[-1]
    N = B if cu_seqlens is None else cu_seqlens.shape[0] - 1
    return q.new_empty(B, T, H, V), q.new_empty(N, H, K, V, dtype=torch.float32)


@torch.library.custom_op("lampa_b200::hgdn_fwd", mutates_args=(), device_types="cuda")
def hgdn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
             lam: torch.Tensor, cu_seqlens: Optional[torch.Tensor], use_l2norm: bool) -> torch.Tensor:
    """Hierarchical rule: o [B,T,H,V] in q's dtype."""
    return _gd._hgdn(q, k, v, g, beta, lam, cu_seqlens, use_l2norm)


@hgdn_fwd.register_fake
def _(q, k, v, g, beta, lam, cu_seqlens, use_l2norm):
    B, T, H, _ = q.shape
    return q.new_empty(B, T, H, v.shape[-1])
