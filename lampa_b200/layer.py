"""Producers and consumers of the gated-delta op inside one mixer layer, host side.

Same names and argument meaning as the reference:
  ShortConvolution                       models/hattention/short_convolution.py:528-720
  compute_lambda                         models/hattention/modeling_h_gated_deltanet.py:151-166
  FusedRMSNormGated / rms_norm_gated     models/hattention/fused_norm.py:1003-1064, 858-880
plus `gate_inputs`, the three statements that turn the a/b/l projections into g, beta and lambda
(modeling_h_gated_deltanet.py:429-450) as one call.  Forward only; everything runs in the CUDA
library on the current stream.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

from . import _lib as L

_LAMBDA_MODES = {"positive": 0, "bounded": 1, None: 2}


class ShortConvolution(nn.Module):
    """Depthwise causal convolution over the token axis of [B, T, D] with an optional SiLU.

    Parameters are those of the reference's nn.Conv1d subclass: `weight` [D, 1, W] and `bias` [D]
    or None.  forward(x, residual, mask, cache, output_final_state, cu_seqlens) -> (y, cache);
    a call with one token per sequence and a cache is the decode step, which updates the cache
    [N, D, W] in place.
    """

    def __init__(self, hidden_size: int, kernel_size: int, bias: bool = False, activation: Optional[str] = "silu",
                 use_fast_conv1d: Optional[bool] = True, device=None, dtype=None, **kwargs):
        super().__init__()
        if kernel_size % 2 != 0:
            raise ValueError("Kernel size must be the power of 2")
        if activation is not None:
            assert activation in ["silu", "swish"], f"Activation `{activation}` not supported yet."
        self.hidden_size = hidden_size
        self.kernel_size = (kernel_size,)
        self.activation = activation
        conv = nn.Conv1d(hidden_size, hidden_size, kernel_size, groups=hidden_size, bias=bias,
                         padding=kernel_size - 1, device=device, dtype=dtype)      # same initialisation
        self.weight = conv.weight
        self.bias = conv.bias

    @property
    def state_size(self) -> int:
        return self.hidden_size * self.kernel_size[0]

    def _params(self):
        w = self.weight.detach().reshape(self.hidden_size, self.kernel_size[0]).contiguous()
        b = None if self.bias is None else self.bias.detach().contiguous()
        return w, b

    @torch.no_grad()
    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, mask: Optional[torch.Tensor] = None,
                cache: Optional[torch.Tensor] = None, output_final_state: bool = False,
                cu_seqlens: Optional[torch.LongTensor] = None, **kwargs) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        B, T, D = x.shape
        W = self.kernel_size[0]
        N = B if cu_seqlens is None else len(cu_seqlens) - 1
        if mask is not None:
            if cu_seqlens is not None:
                raise ValueError("`mask` and `cu_seqlens` cannot be provided at the same time")
            x = x.mul_(mask.unsqueeze(-1))
        if output_final_state and cache is None:
            cache = x.new_zeros(N, D, W)
        if cache is not None and B * T == N:
            return self.step(x, residual, cache, cu_seqlens)
        dev = L.require_cuda(x, residual, cache, cu_seqlens)
        w, b = self._params()
        x = x.contiguous()
        residual = None if residual is None else residual.contiguous()
        cu = None if cu_seqlens is None else cu_seqlens.to(device=dev, dtype=torch.int64).contiguous()
        if cache is not None and (not cache.is_contiguous() or cache.dtype != x.dtype):
            raise ValueError("cache must be a contiguous [N, D, W] tensor of x's dtype")
        y = torch.empty_like(x)
        rc = L.lib().lampa_short_conv_fwd(L.ptr(x), L.ptr(w), L.ptr(b), L.ptr(residual), L.ptr(cu),
                                          0 if cu is None else N, B, T, D, W, L.dtype_code(x.dtype),
                                          L.dtype_code(w.dtype), int(self.activation is not None), L.ptr(y),
                                          L.ptr(cache), int(cu is not None), L.stream_ptr(dev))
        L.check(rc, "lampa_short_conv_fwd")
        return y, cache

    @torch.no_grad()
    def step(self, x: torch.Tensor, residual: Optional[torch.Tensor], cache: torch.Tensor,
             cu_seqlens: Optional[torch.LongTensor] = None):
        dev = L.require_cuda(x, residual, cache)
        shape = x.shape
        N, D, W = cache.shape
        w, b = self._params()
        xf = x.reshape(N, D).contiguous()
        rf = None if residual is None else residual.reshape(N, D).contiguous()
        if not cache.is_contiguous() or cache.dtype != x.dtype:
            raise ValueError("cache must be a contiguous [N, D, W] tensor of x's dtype")
        y = torch.empty_like(xf)
        rc = L.lib().lampa_short_conv_step(L.ptr(xf), L.ptr(cache), L.ptr(w), L.ptr(b), L.ptr(rf), N, D, W,
                                           L.dtype_code(x.dtype), L.dtype_code(w.dtype),
                                           int(self.activation is not None), L.ptr(y), L.stream_ptr(dev))
        L.check(rc, "lampa_short_conv_step")
        return y.view(shape), cache


@torch.no_grad()
def gate_inputs(a: Optional[torch.Tensor], b: Optional[torch.Tensor], dl: Optional[torch.Tensor],
                A_log: Optional[torch.Tensor], dt_bias: Optional[torch.Tensor], L_param: Optional[torch.Tensor],
                lambda_mode: Optional[str] = "positive", attention_mask: Optional[torch.Tensor] = None,
                lambda_dtype: Optional[torch.dtype] = None):
    """(g, beta, l) of the hierarchical layer: a, b [B,T,H] (outputs of a_proj / b_proj), dl
    [B,T,H,L] or [B,T,H*L] (output of l_proj), A_log / dt_bias [H], L_param [H,L];
    g = -exp(A_log) softplus(a + dt_bias) in fp32, beta = sigmoid(b) in b's dtype,
    l = compute_lambda(L_param, dl, lambda_mode) in `lambda_dtype` (default: dl's dtype), each
    multiplied by attention_mask [B,T] when given.  Inputs set to None skip their output."""
    ref = a if a is not None else (b if b is not None else dl)
    dev = L.require_cuda(a, b, dl, A_log, dt_bias, L_param, attention_mask)
    Bn, T = ref.shape[:2]
    H = (a if a is not None else b).shape[2] if (a is not None or b is not None) else L_param.shape[0]
    if lambda_mode not in _LAMBDA_MODES:
        raise ValueError
    g = beta = lam = None
    nl = 0
    if a is not None:
        a = a.contiguous()
        g = torch.empty(Bn, T, H, dtype=torch.float32, device=dev)
    if b is not None:
        b = b.to(ref.dtype).contiguous()
        beta = torch.empty(Bn, T, H, dtype=b.dtype, device=dev)
    if dl is not None:
        nl = L_param.shape[-1]
        dl = dl.to(ref.dtype).reshape(Bn, T, H, nl).contiguous()
        lam = torch.empty(Bn, T, H, nl, dtype=lambda_dtype or dl.dtype, device=dev)
    f32 = lambda t: None if t is None else t.detach().to(device=dev, dtype=torch.float32).contiguous()
    A_log, dt_bias, Lw = f32(A_log), f32(dt_bias), f32(L_param)
    m = None if attention_mask is None else attention_mask[:, -T:].to(torch.float32).contiguous()
    rc = L.lib().lampa_gate_inputs(L.ptr(a), L.ptr(b), L.ptr(dl), L.ptr(A_log), L.ptr(dt_bias), L.ptr(Lw), L.ptr(m),
                                   Bn * T, H, nl, L.dtype_code(ref.dtype),
                                   L.dtype_code(beta.dtype if beta is not None else ref.dtype),
                                   L.dtype_code(lam.dtype if lam is not None else ref.dtype),
                                   _LAMBDA_MODES[lambda_mode], L.ptr(g), L.ptr(beta), L.ptr(lam), L.stream_ptr(dev))
    L.check(rc, "lampa_gate_inputs")
    return g, beta, lam


def compute_lambda(L: torch.Tensor, dl: torch.Tensor, lambda_mode: Optional[str]) -> torch.Tensor:
    """softplus(L * dl) ("positive"), exp(-exp(L) * softplus(dl)) ("bounded") or L * dl (None);
    L broadcasts as [1, 1, H, levels] against dl [B, T, H, levels]."""
    if lambda_mode not in _LAMBDA_MODES:
        raise ValueError
    Lp = L.reshape(L.shape[-2], L.shape[-1])
    return gate_inputs(None, None, dl, None, None, Lp, lambda_mode,
                       lambda_dtype=torch.promote_types(L.dtype, dl.dtype))[2]


@torch.no_grad()
def rms_norm_gated(x: torch.Tensor, g: torch.Tensor, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor],
                   activation: str = "swish", residual: Optional[torch.Tensor] = None, prenorm: bool = False,
                   residual_in_fp32: bool = False, eps: float = 1e-6) -> torch.Tensor:
    """y = x / sqrt(mean(x^2) + eps) * weight * g * sigmoid(g) over the last axis (activation
    "sigmoid": ... * sigmoid(g)).  bias, residual and prenorm of the reference signature are not
    supported (the layer does not use them)."""
    if bias is not None or residual is not None or prenorm:
        raise NotImplementedError
    if activation not in ("swish", "silu", "sigmoid"):
        raise ValueError(f"Unsupported activation: {activation}")
    dev = L.require_cuda(x, g, weight)
    D = x.shape[-1]
    xf, gf = x.contiguous(), g.to(x.dtype).contiguous()
    w = None if weight is None else weight.detach().contiguous()
    y = torch.empty_like(xf)
    rc = L.lib().lampa_rmsnorm_gate(L.ptr(xf), L.ptr(gf), L.ptr(w), xf.numel() // D, D, L.dtype_code(x.dtype),
                                    L.dtype_code(w.dtype) if w is not None else L.LAMPA_F32, float(eps),
                                    int(activation == "sigmoid"), L.ptr(y), L.stream_ptr(dev))
    L.check(rc, "lampa_rmsnorm_gate")
    return y


@torch.no_grad()
def add_rms_norm(res: torch.Tensor, delta: Optional[torch.Tensor], weight: Optional[torch.Tensor], eps: float = 1e-6,
                 perm: Optional[torch.Tensor] = None, seg_offsets: Optional[torch.Tensor] = None, nseg: int = 1,
                 delta_at_r: bool = False, y_at_r: bool = False, out_dtype: Optional[torch.dtype] = torch.bfloat16):
    """Fused residual add + RMS norm (+ row permutation) on an fp32 residual stream `res` [rows, D],
    in place: the `RMSNorm(x, residual, prenorm=True)` of the reference's blocks
    (models/hattention/fused_norm.py:1288-1330, modeling_gated_deltaproduct.py:1169-1199) with the
    ordering layer's gather / un-gather (models/baselines/hmamba.py:428-455) folded in.

    For every j: r = perm[j] inside j's segment (r = j without perm);
    res[r] += delta[r if delta_at_r else j]; y[r if y_at_r else j] = rms_norm(res[r]) * weight.
    delta None: norm only.  out_dtype None: add only (returns None)."""
    dev = L.require_cuda(res, delta, weight, perm)
    if res.dtype != torch.float32 or not res.is_contiguous() or res.dim() != 2:
        raise ValueError("res must be a contiguous fp32 [rows, D] tensor (updated in place)")
    rows, D = res.shape
    if delta is not None:
        delta = delta.contiguous()
        if tuple(delta.shape) != (rows, D):
            raise ValueError("delta must match res")
    if perm is not None:
        perm = perm.to(torch.int64).contiguous().view(-1)
        if perm.numel() != rows:
            raise ValueError("perm must have one entry per row")
    if seg_offsets is not None:
        seg_offsets = seg_offsets.to(device=dev, dtype=torch.int64).contiguous()
        nseg = seg_offsets.numel() - 1
    w = None if weight is None else weight.detach().to(torch.float32).contiguous()
    y = None if out_dtype is None else torch.empty(rows, D, dtype=out_dtype, device=dev)
    rc = L.lib().lampa_add_rmsnorm(L.ptr(res), L.ptr(delta), L.dtype_code(delta.dtype) if delta is not None else 0,
                                   L.ptr(perm), L.ptr(seg_offsets), max(int(nseg), 1), rows, D, L.ptr(w), float(eps),
                                   int(delta_at_r), int(y_at_r), L.ptr(y), L.dtype_code(out_dtype) if y is not None else 0,
                                   L.ptr(L.status_word(dev)), L.stream_ptr(dev))
    L.check(rc, "lampa_add_rmsnorm")
    return y


class FusedRMSNormGated(nn.Module):
    """RMS norm over the last axis followed by a swish (or sigmoid) gate (fused_norm.py:1003-1064)."""

    def __init__(self, hidden_size: int, elementwise_affine: bool = True, eps: float = 1e-5,
                 activation: str = "swish", device=None, dtype=None):
        super().__init__()
        if activation not in ["swish", "silu", "sigmoid"]:
            raise ValueError(f"Unsupported activation: {activation}")
        self.hidden_size = hidden_size
        self.elementwise_affine = elementwise_affine
        self.eps = eps
        self.activation = activation
        if elementwise_affine:
            self.weight = nn.Parameter(torch.ones(hidden_size, device=device, dtype=dtype))
        else:
            self.register_parameter("weight", None)
        self.register_parameter("bias", None)

    def forward(self, x: torch.Tensor, g: torch.Tensor, residual: Optional[torch.Tensor] = None,
                prenorm: bool = False, residual_in_fp32: bool = False) -> torch.Tensor:
        return rms_norm_gated(x, g, self.weight, self.bias, self.activation, residual=residual, eps=self.eps,
                              prenorm=prenorm, residual_in_fp32=residual_in_fp32)
