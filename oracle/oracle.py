"""ctypes front end of the CPU oracle (``oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the
CPU-baseline legs of the benchmark.  The product package never imports it.

All functions take and return numpy arrays (fp32 / int32 / int64, C-contiguous)
in the reference's token-major layouts.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liblampa_oracle.so")
_LIB = None


def build(force: bool = False) -> str:
    """Compile ``oracle.c`` next to itself (gcc; OpenMP when available)."""
    src = os.path.join(_HERE, "oracle.c")
    if not force and os.path.exists(_SO) and os.path.getmtime(_SO) >= os.path.getmtime(src):
        return _SO
    base = ["-O2", "-ffp-contract=off", "-fPIC", "-shared", src, "-o", _SO, "-lm"]
    last = None
    for cc in ("/usr/bin/gcc", "gcc", "cc"):
        for omp in (["-fopenmp"], []):
            try:
                subprocess.run([cc] + omp + base, check=True, capture_output=True)
                return _SO
            except (subprocess.CalledProcessError, FileNotFoundError) as e:  # try next
                last = e
    raise RuntimeError(f"could not build the oracle: {last}")


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        build()
        _LIB = ctypes.CDLL(_SO)
    return _LIB


def set_threads(n: int) -> int:
    """Set the OpenMP thread count of the oracle's loops; returns the count in effect."""
    return int(lib().oracle_set_threads(ctypes.c_int(int(n))))


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


def _p(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def gdn_plain(q, k, v, g, beta, scale: Optional[float] = None, h0=None, cu_seqlens=None,
              use_l2norm: bool = False) -> Tuple[np.ndarray, np.ndarray]:
    """Plain gated-delta rule. q,k [T,H,K]; v [T,H,V]; g,beta [T,H]; h0 [N,H,K,V].

    Returns (o [T,H,V], final_state [N,H,K,V]) in fp32.
    """
    q, k, v, g, beta = map(_f32, (q, k, v, g, beta))
    T, H, K = q.shape
    V = v.shape[-1]
    if scale is None:
        scale = K ** -0.5
    cu = None if cu_seqlens is None else np.ascontiguousarray(np.asarray(cu_seqlens, dtype=np.int64))
    nseq = 1 if cu is None else len(cu) - 1
    h0 = None if h0 is None else _f32(h0).reshape(nseq, H, K, V)
    o = np.empty((T, H, V), np.float32)
    ht = np.empty((nseq, H, K, V), np.float32)
    rc = lib().oracle_gdn_plain(_p(q), _p(k), _p(v), _p(g), _p(beta), _p(h0), _p(cu),
                                ctypes.c_int(nseq), _p(o), _p(ht), ctypes.c_int(T), ctypes.c_int(H),
                                ctypes.c_int(K), ctypes.c_int(V), ctypes.c_float(scale),
                                ctypes.c_int(int(use_l2norm)))
    if rc != 0:
        raise RuntimeError(f"oracle_gdn_plain failed: {rc}")
    return o, ht


def hgdn(q, k, v, g, beta, lam, cu_seqlens=None, use_l2norm: bool = True):
    """Hierarchical gated-delta rule. lam [T,H,L].

    Returns (o [T,H,V], states [H,K,V,L], counts [L]); states/counts describe the
    last sequence.
    """
    q, k, v, g, beta, lam = map(_f32, (q, k, v, g, beta, lam))
    T, H, K = q.shape
    V = v.shape[-1]
    L = lam.shape[-1]
    cu = None if cu_seqlens is None else np.ascontiguousarray(np.asarray(cu_seqlens, dtype=np.int64))
    nseq = 1 if cu is None else len(cu) - 1
    o = np.empty((T, H, V), np.float32)
    states = np.zeros((H, K, V, L), np.float32)
    counts = np.zeros((L,), np.int32)
    rc = lib().oracle_hgdn(_p(q), _p(k), _p(v), _p(g), _p(beta), _p(lam), _p(cu), ctypes.c_int(nseq),
                           _p(o), _p(states), _p(counts), ctypes.c_int(T), ctypes.c_int(H),
                           ctypes.c_int(K), ctypes.c_int(V), ctypes.c_int(L),
                           ctypes.c_int(int(use_l2norm)))
    if rc != 0:
        raise RuntimeError(f"oracle_hgdn failed: {rc} (not enough levels for this length?)")
    return o, states, counts


def lsh_ids(x, alpha, beta, w: float = 1.0, dim: Optional[int] = None, want_keys: bool = False):
    """x [N, row] fp32 (coordinates first); alpha [heads, dim, rounds]; beta [rounds].

    Returns ids int32 [rounds, heads, N] (and the float projections when want_keys).
    """
    x = _f32(x)
    alpha = _f32(alpha)
    beta = _f32(beta).reshape(-1)
    heads, d, rounds = alpha.shape
    dim = d if dim is None else dim
    assert dim == d and x.shape[1] >= dim and beta.shape[0] == rounds
    N = x.shape[0]
    ids = np.empty((rounds, heads, N), np.int32)
    keys = np.empty((rounds, heads, N), np.float32) if want_keys else None
    lib().oracle_lsh_ids(_p(x), ctypes.c_int64(x.shape[1]), _p(alpha), _p(beta), ctypes.c_float(w),
                         ctypes.c_int64(N), ctypes.c_int(heads), ctypes.c_int(rounds), ctypes.c_int(dim),
                         _p(ids), _p(keys))
    return (ids, keys) if want_keys else ids


def segsort(keys, seg=None, init=None) -> np.ndarray:
    """Stable ascending sort per segment; keys 1-D int32 or fp32; returns int64 local indices."""
    keys = np.ascontiguousarray(keys)
    n = keys.shape[0]
    seg = np.array([0, n], np.int64) if seg is None else np.ascontiguousarray(np.asarray(seg, np.int64))
    init = None if init is None else np.ascontiguousarray(np.asarray(init, np.int64))
    perm = np.empty((n,), np.int64)
    if keys.dtype == np.int32:
        fn = lib().oracle_segsort_i32
    elif keys.dtype == np.float32:
        fn = lib().oracle_segsort_f32
    else:
        raise TypeError(keys.dtype)
    fn(_p(keys), _p(seg), ctypes.c_int(len(seg) - 1), _p(init), _p(perm))
    return perm


def invert_perm(perm, seg=None) -> np.ndarray:
    perm = np.ascontiguousarray(np.asarray(perm, np.int64))
    n = perm.shape[0]
    seg = np.array([0, n], np.int64) if seg is None else np.ascontiguousarray(np.asarray(seg, np.int64))
    inv = np.empty_like(perm)
    rc = lib().oracle_invert_perm(_p(perm), _p(seg), ctypes.c_int(len(seg) - 1), _p(inv))
    if rc != 0:
        raise ValueError("not a permutation")
    return inv


def permute_rows(src, perm, seg=None) -> np.ndarray:
    src = np.ascontiguousarray(src)
    perm = np.ascontiguousarray(np.asarray(perm, np.int64))
    n = perm.shape[0]
    seg = np.array([0, n], np.int64) if seg is None else np.ascontiguousarray(np.asarray(seg, np.int64))
    dst = np.empty_like(src)
    row_bytes = src.strides[0]
    lib().oracle_permute_rows(_p(src), _p(perm), _p(seg), ctypes.c_int(len(seg) - 1), _p(dst),
                              ctypes.c_int64(row_bytes))
    return dst


def lsh_ordering_keys(coords, alpha) -> np.ndarray:
    """Float bucket key of LSHOrdering (models/baselines/hmamba.py:316-333) for one event.

    coords [N, C] fp32; alpha [1, C, n_hashes].  With a single head the reference's
    shift (max - min over a size-1 axis) is zero, so key = sum_i 2^i * (coords @ alpha[0,:,i]).
    """
    coords = _f32(coords)
    alpha = _f32(alpha)
    proj = coords @ alpha[0]                    # [N, n_hashes]
    expo = (2 ** np.arange(alpha.shape[-1])).astype(np.float32)
    return (proj * expo).sum(-1).astype(np.float32)


def lsh_ordering(coords, alpha) -> np.ndarray:
    """Permutation of LSHOrdering.forward for one event: norm pre-sort, then stable key sort."""
    coords = _f32(coords)
    key = lsh_ordering_keys(coords, alpha)
    norm = np.sqrt((coords.astype(np.float32) ** 2).sum(-1, dtype=np.float32)).astype(np.float32)
    norm_idx = segsort(norm)
    return segsort(key, init=norm_idx)


# ---- region (geo) shift of the LSH keys: numpy fp32, one rounding per elementwise op ------------

def quantile_regions(sorted_idx, num_regions) -> np.ndarray:
    """quantile_partition (models/model_utils/hash_utils.py:14-27): sorted_idx [N] is the argsort
    of one coordinate, num_regions [R] fp32.  Returns fp32 [R, N]:
    floor(rank / ceil(N / R_r)) + 1 with rank = inverse permutation of sorted_idx."""
    sorted_idx = np.asarray(sorted_idx, np.int64)
    n = sorted_idx.shape[0]
    rank = np.empty(n, np.int64)
    rank[sorted_idx] = np.arange(n, dtype=np.int64)
    rs = np.ceil(np.float32(n) / np.asarray(num_regions, np.float32).reshape(-1))     # [R]
    return (np.floor_divide(rank[None, :].astype(np.float32), rs[:, None]) + np.float32(1)).astype(np.float32)


def geo_shift(regions_eta, hash_shift, reg_eta, reg_phi) -> np.ndarray:
    """get_geo_shift (models/attention/hept.py:78-88) for one of its two identical halves:
    (reg_phi * range) * (ceil(R_eta) + 1) + reg_eta * range, fp32 [R, N]."""
    hs = np.asarray(hash_shift, np.float32).reshape(-1, 1)
    stride = (np.ceil(np.asarray(regions_eta, np.float32)).reshape(-1, 1) + np.float32(1)).astype(np.float32)
    phi = (np.asarray(reg_phi, np.float32) * hs).astype(np.float32) * stride
    eta = (np.asarray(reg_eta, np.float32) * hs).astype(np.float32)
    return (phi.astype(np.float32) + eta).astype(np.float32)


def row_range(a, b=None) -> np.ndarray:
    """hash_shift of lsh_mapping (hash_utils.py:333-340): max - min over the last axis of a
    (and b), fp32 [R]."""
    a = np.asarray(a, np.float32).reshape(-1, a.shape[-1])
    mx, mn = a.max(-1), a.min(-1)
    if b is not None:
        b = np.asarray(b, np.float32).reshape(-1, b.shape[-1])
        mx, mn = np.maximum(mx, b.max(-1)), np.minimum(mn, b.min(-1))
    return (mx - mn).astype(np.float32)


def geo_keys(proj, shift, raw_size: int) -> np.ndarray:
    """Shifted sort keys (hept.py:130-136): padded hits get +inf before the shift is added."""
    k = np.array(proj, np.float32).reshape(shift.shape)
    k[:, raw_size:] = np.inf
    return (k + shift).astype(np.float32)


def e2lsh_proj(vecs, alpha) -> np.ndarray:
    """E2LSH.forward (hash_utils.py:366-371): vecs [heads, N, dim], alpha [heads, dim, rounds]
    -> fp32 [rounds, heads, N], accumulated in the frozen order of oracle_lsh_ids."""
    vecs = _f32(vecs)
    alpha = _f32(alpha)
    heads, N, dim = vecs.shape
    rounds = alpha.shape[-1]
    out = np.empty((rounds, heads, N), np.float32)
    for h in range(heads):
        acc = vecs[h, :, 0:1] * alpha[h, 0][None, :]
        for d in range(1, dim):
            acc = (acc + (vecs[h, :, d:d + 1] * alpha[h, d][None, :]).astype(np.float32)).astype(np.float32)
        out[:, h, :] = acc.T
    return out


# ---- producers / consumers of the op inside one layer (numpy fp32) ------------------------------

def _softplus(x):
    x = np.asarray(x, np.float32)
    return np.where(x > 20, x, np.log1p(np.exp(np.minimum(x, 20)))).astype(np.float32)


def _sigmoid(x):
    return (1.0 / (1.0 + np.exp(-np.asarray(x, np.float32)))).astype(np.float32)


def gate_inputs(a, b, dl, A_log, dt_bias, Lw, mode="positive"):
    """g, beta, lambda of the hierarchical layer (models/hattention/modeling_h_gated_deltanet.py:
    429-437, compute_lambda 151-166).  a, b [..., H]; dl [..., H, L]."""
    g = (-np.exp(np.asarray(A_log, np.float32)) * _softplus(np.asarray(a, np.float32) + np.asarray(dt_bias, np.float32))).astype(np.float32)
    beta = _sigmoid(b)
    Lw = np.asarray(Lw, np.float32)
    dl = np.asarray(dl, np.float32)
    if mode == "positive":
        lam = _softplus(Lw * dl)
    elif mode == "bounded":
        lam = np.exp(-np.exp(Lw) * _softplus(dl)).astype(np.float32)
    else:
        lam = (Lw * dl).astype(np.float32)
    return g, beta, lam


def short_conv(x, w, bias=None, residual=None, cu=None, silu=True):
    """Causal depthwise convolution of ShortConvolution (models/hattention/short_convolution.py:
    39-112): x [B, T, D], w [D, W]; y[t] = act(bias + sum_i w[:, i] x[t - (W-1) + i]) + residual,
    taps before the sequence start are zero.  cu: sequence offsets over the flattened tokens (B = 1)."""
    x = np.asarray(x, np.float32)
    w = np.asarray(w, np.float32)
    B, T, D = x.shape
    W = w.shape[1]
    y = np.zeros_like(x)
    bounds = [(bi, 0, T) for bi in range(B)] if cu is None else [(0, int(s), int(e)) for s, e in zip(cu[:-1], cu[1:])]
    for bi, s, e in bounds:
        seg = x[bi, s:e]
        acc = np.zeros_like(seg)
        for i in range(W):
            sh = W - 1 - i
            if sh < seg.shape[0]:
                acc[sh:] += seg[:seg.shape[0] - sh] * w[:, i]
        y[bi, s:e] = acc
    if bias is not None:
        y = y + np.asarray(bias, np.float32)
    if silu:
        y = y * _sigmoid(y)
    if residual is not None:
        y = y + np.asarray(residual, np.float32)
    return y.astype(np.float32)


def short_conv_state(x, W, cu=None):
    """Last W tokens of each sequence as [N, D, W], zero where the sequence is shorter
    (short_convolution.py:484-502, 617-626)."""
    x = np.asarray(x, np.float32)
    B, T, D = x.shape
    bounds = [(bi, 0, T) for bi in range(B)] if cu is None else [(0, int(s), int(e)) for s, e in zip(cu[:-1], cu[1:])]
    out = np.zeros((len(bounds), D, W), np.float32)
    for n, (bi, s, e) in enumerate(bounds):
        m = min(W, e - s)
        if m > 0:
            out[n, :, W - m:] = x[bi, e - m:e].T
    return out


def short_conv_step(x, cache, w, bias=None, silu=True):
    """Decode step (short_convolution.py:203-253): returns (y [N, D], new cache [N, D, W])."""
    cache = np.roll(np.asarray(cache, np.float32), -1, axis=-1)
    cache[:, :, -1] = np.asarray(x, np.float32)
    y = (cache * np.asarray(w, np.float32)).sum(-1)
    if bias is not None:
        y = y + np.asarray(bias, np.float32)
    if silu:
        y = y * _sigmoid(y)
    return y.astype(np.float32), cache


def rmsnorm_gate(x, g, w=None, eps=1e-5, sigmoid_only=False):
    """Gated RMS norm of the layer output (models/hattention/fused_norm.py:40-112)."""
    x = np.asarray(x, np.float32)
    g = np.asarray(g, np.float32)
    rstd = 1.0 / np.sqrt((x * x).mean(-1, keepdims=True) + np.float32(eps))
    y = x * rstd
    if w is not None:
        y = y * np.asarray(w, np.float32)
    y = y * _sigmoid(g) if sigmoid_only else y * g * _sigmoid(g)
    return y.astype(np.float32)


# ---- bucketed RBF-kernel attention of the HEPT layer (numpy, float64 accumulation) --------------

def qkv_res(s_query, s_key, s_value):
    """models/attention/hept.py:22-33 on rows already in bucket order [..., bucketsz, d]:
    p = exp(min(0, q.k - |q|^2/2 - |k|^2/2)), denom = sum_j p + 1e-20, so = p @ v.  Computed in
    float64 from the fp32 inputs: the exponent is a difference of large terms, and the test
    tolerance is stated against this value."""
    q = np.asarray(s_query, np.float64)
    k = np.asarray(s_key, np.float64)
    v = np.asarray(s_value, np.float64)
    qs = -0.5 * (q * q).sum(-1, keepdims=True)
    ks = -0.5 * (k * k).sum(-1, keepdims=True)
    d = np.einsum("...id,...jd->...ij", q, k) + qs + np.swapaxes(ks, -1, -2)
    p = np.exp(np.minimum(d, 0.0))
    return p.sum(-1, keepdims=True) + 1e-20, np.einsum("...ij,...jd->...id", p, v)


def hept_prep_qk(query, key, w, coords, raw_size=None):
    """prep_qk (hept.py:55-63) followed by the head-major rearrange and the zeroing of padded rows
    (hept.py:121-126), fp32 with one rounding per elementwise op: returns q_hat, k_hat
    [heads, N, d + coords_dim]."""
    query = np.asarray(query, np.float32)
    key = np.asarray(key, np.float32)
    w = np.asarray(w, np.float32)
    coords = np.asarray(coords, np.float32)
    qw = np.exp(np.minimum(w.sum(1), np.float32(50))).sum(-1).astype(np.float32)          # [heads, r]
    scale = np.sqrt(np.float32(2) * np.concatenate([qw[:, :1], qw], -1)).astype(np.float32)
    r = (scale[None] * coords[:, None]).astype(np.float32)                                  # [N, heads, cd]
    q_hat = np.concatenate([query, r], -1).transpose(1, 0, 2).copy()
    k_hat = np.concatenate([key, r], -1).transpose(1, 0, 2).copy()
    if raw_size is not None:
        q_hat[:, raw_size:] = 0
        k_hat[:, raw_size:] = 0
    return q_hat, k_hat


def hept_bucket_attention(q_hat, k_hat, value, q_pos, k_pos, block: int):
    """hept.py:141-151: gather into bucket order per (round, head), qkv_res, scatter back to hit
    order, sum the rounds, so / denom.  q_hat, k_hat [heads, N, dq], value [heads, N, dv],
    positions [rounds, heads, N].  Returns (out [heads, N, dv], o [rounds, heads, N, dv],
    logits [rounds, heads, N, 1]) in float64."""
    q_hat = np.asarray(q_hat, np.float32)
    k_hat = np.asarray(k_hat, np.float32)
    value = np.asarray(value, np.float32)
    C, H, N = q_pos.shape
    o = np.zeros((C, H, N, value.shape[-1]), np.float64)
    lg = np.zeros((C, H, N, 1), np.float64)
    for c in range(C):
        for h in range(H):
            sq = q_hat[h][q_pos[c, h]].reshape(N // block, block, -1)
            sk = k_hat[h][k_pos[c, h]].reshape(N // block, block, -1)
            sv = value[h][k_pos[c, h]].reshape(N // block, block, -1)
            den, so = qkv_res(sq, sk, sv)
            o[c, h, q_pos[c, h]] = so.reshape(N, -1)
            lg[c, h, q_pos[c, h]] = den.reshape(N, 1)
    return o.sum(0) / lg.sum(0), o, lg
