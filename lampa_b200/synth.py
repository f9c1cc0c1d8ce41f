"""Seeded synthetic inputs with the shapes and value ranges of the benchmark configurations.

The reference evaluates on TrackML events (6k-60k hits, README.md:57); that dataset is not
available offline, so these generators stand in for it: hits on 10 cylindrical layers
(r = 30..1000 mm, phi ~ U(-pi, pi), z ~ U(-3000, 3000) mm) with a 24-float feature row
[x, y, z, r, phi, eta, 18 x N(0,1)], and mixer inputs drawn as the benchmark configuration
states (unit-norm q/k, v ~ N(0,1), beta = sigmoid(N), g = -softplus(N + shift), lambda = softplus(N)).
Everything is drawn on the CPU from one torch.Generator so the CPU checker and the GPU see the
same numbers.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn.functional as F


def gdn_inputs(seed: int, T: int, H: int, K: int, V: int, L: Optional[int] = None, g_shift: float = 2.0,
               h0: bool = False, dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Draw order: q, k, v, beta, g, lambda, h0 (all [1, T, H, .])."""
    gen = torch.Generator().manual_seed(seed)
    q = F.normalize(torch.randn(1, T, H, K, generator=gen), dim=-1)
    k = F.normalize(torch.randn(1, T, H, K, generator=gen), dim=-1)
    v = torch.randn(1, T, H, V, generator=gen)
    beta = torch.sigmoid(torch.randn(1, T, H, generator=gen))
    g = -F.softplus(torch.randn(1, T, H, generator=gen) + g_shift)
    out = {"q": q.to(dtype), "k": k.to(dtype), "v": v.to(dtype), "beta": beta, "g": g}
    if L is not None:
        out["lam"] = F.softplus(torch.randn(1, T, H, L, generator=gen))
    if h0:
        out["h0"] = 0.1 * torch.randn(1, H, K, V, generator=gen)
    return out


def detector_hits(seed: int, N: int, extra: int = 18) -> torch.Tensor:
    """[N, 6 + extra] fp32 rows: x, y, z, r, phi, eta, then N(0,1) features."""
    gen = torch.Generator().manual_seed(seed)
    layer = torch.randint(0, 10, (N,), generator=gen).float()
    r = 30.0 + layer * (970.0 / 9.0)
    phi = (torch.rand(N, generator=gen) * 2 - 1) * math.pi
    z = (torch.rand(N, generator=gen) * 2 - 1) * 3000.0
    eta = torch.asinh(z / r)
    coords = torch.stack([r * torch.cos(phi), r * torch.sin(phi), z, r, phi, eta], -1)
    feats = torch.randn(N, extra, generator=gen)
    return torch.cat([coords, feats], -1).contiguous()


def lsh_params(seed: int, heads: int = 8, dim: int = 6, rounds: int = 3, w: float = 1.0):
    """alpha ~ N(0,1) [heads, dim, rounds], beta ~ U(0, w) [rounds]."""
    gen = torch.Generator().manual_seed(seed)
    alpha = torch.randn(heads, dim, rounds, generator=gen)
    beta = torch.rand(rounds, generator=gen) * w
    return alpha, beta


def event_sizes(seed: int, n_events: int, lo: int = 6000, hi: int = 60000) -> torch.Tensor:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi + 1, (n_events,), generator=gen)
