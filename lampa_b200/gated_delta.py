"""Drop-in host side of the gated-delta forward ops.

Same names, argument meaning and error behaviour as the reference entry points:
  chunk_gated_delta_rule    models/hattention/gated_delta_rule_ori.py:235-357
  chunk_h_gated_delta_rule  models/hattention/gated_delta_rule_apis.py:20-134
  hattention_kernel         models/hattention/kernel.py:338-374
  hattention_prefill / hattention_step / HState   kernel.py:470-633, recurrent.py:9-131
Forward only: the ops are not differentiable, and a call whose inputs require grad while grad
mode is on raises instead of returning a silently detached result (the reference's forward-only
ops raise in backward: gated_delta_rule_ori.py:555-562).  Everything runs in the CUDA library
on the current torch stream; there is no PyTorch or CPU fallback.
"""
from __future__ import annotations

import ctypes
import enum
import math
import warnings
from typing import Optional, Tuple

import torch

from . import _lib as L


class HType(enum.Enum):
    """Hierarchy type (models/hattention/base.py); only WEAK is implemented, as in the GDELTA path."""
    WEAK = "weak"
    STRONG = "strong"


class HStruct(enum.Enum):
    """State structure (models/hattention/base.py); only GDELTA is implemented here."""
    MAMBA2 = "mamba2"
    GDELTA = "gdelta"


CHUNK = 64
ELL0 = 7   # intra-chunk levels: get_num_levels(64, 2) (models/hattention/base.py:37-38)


def num_levels_required(T: int) -> int:
    """Levels lambda must provide for a sequence of T tokens: 7 + ceil(log2(ceil(T/64)))
    (the check at models/hattention/chunkwise_hgdn.py:723-726)."""
    nt = (T + CHUNK - 1) // CHUNK
    return ELL0 + (math.ceil(math.log2(nt)) if nt > 1 else 0)


def _check_cu_seqlens(cu_seqlens, T: int, n_levels: Optional[int] = None) -> None:
    """Host-side validation of packed offsets when they are host-resident (the reference reads
    them on the host too, models/hattention/index.py:69-83).  Device-resident offsets are checked
    by the kernels instead: a bad entry empties that sequence and sets LAMPA_ERR_BOUNDS /
    LAMPA_ERR_LEVELS in the status word, which the caller reads with `check_status()` at its next
    synchronisation point (LAMPA_B200_CHECK=1 does so after every call)."""
    if cu_seqlens is None or cu_seqlens.is_cuda:
        return
    cu = cu_seqlens.tolist()
    if len(cu) < 2 or cu[0] != 0 or cu[-1] != T or any(b < a for a, b in zip(cu[:-1], cu[1:])):
        raise ValueError(f"cu_seqlens must rise from 0 to the number of tokens ({T}); got {cu[:4]}...{cu[-2:]}")
    if n_levels is not None:
        longest = max(b - a for a, b in zip(cu[:-1], cu[1:]))
        if n_levels < num_levels_required(longest):
            raise ValueError(f"l has {n_levels} levels, a sequence of {longest} tokens needs {num_levels_required(longest)}")


def _common_checks(q, k, v, beta, head_first, cu_seqlens, initial_state):
    assert q.dtype == k.dtype == v.dtype
    assert q.dtype != torch.float32, "ChunkGatedDeltaRuleFunction does not support float32. Please use bfloat16."
    assert len(beta.shape) == 3, "beta must be of shape [B, T, H] if head_first=False, or [B, H, T] otherwise."
    if head_first:
        raise DeprecationWarning(
            "head_first is deprecated and will be removed in a future version. "
            "Please use head_first=False for now instead."
        )
    if q.shape[1] < q.shape[2]:
        warnings.warn(
            f"Input tensor shape suggests potential format mismatch: seq_len ({q.shape[1]}) < num_heads ({q.shape[2]}). "
            "This may indicate the inputs were passed in head-first format [B, H, T, ...] "
            "when head_first=False was specified. "
            "Please verify your input tensor format matches the expected shape [B, T, H, ...]."
        )
    if cu_seqlens is not None:
        if q.shape[0] != 1:
            raise ValueError(
                f"The batch size is expected to be 1 rather than {q.shape[0]} when using `cu_seqlens`."
                f"Please flatten variable-length inputs before processing."
            )
        if initial_state is not None and initial_state.shape[0] != len(cu_seqlens) - 1:
            raise ValueError(
                f"The number of initial states is expected to be equal to the number of input sequences, "
                f"i.e., {len(cu_seqlens) - 1} rather than {initial_state.shape[0]}."
            )


def _forward_only(*tensors) -> None:
    if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors):
        raise NotImplementedError(
            "lampa_b200 implements the forward pass only: backward is not implemented; "
            "call under torch.no_grad() or detach the inputs")


def _desc(q, v, g, lam, cu_seqlens, use_l2norm, scale) -> L.GdnDesc:
    B, T, H, K = q.shape
    return L.GdnDesc(B=B, T=T, H=H, K=K, V=v.shape[-1], L=0 if lam is None else lam.shape[-1],
                     nseq=0 if cu_seqlens is None else len(cu_seqlens) - 1,
                     qkv_dtype=L.dtype_code(q.dtype), gb_dtype=L.dtype_code(g.dtype),
                     lam_dtype=L.LAMPA_F32 if lam is None else L.dtype_code(lam.dtype),
                     use_l2norm=int(bool(use_l2norm)), scale=float(scale))


def _workspace(desc: L.GdnDesc, dev: torch.device) -> torch.Tensor:
    n = ctypes.c_size_t(0)
    L.check(L.lib().lampa_gdn_workspace_bytes(ctypes.byref(desc), ctypes.byref(n)), "lampa_gdn_workspace_bytes")
    buf = torch.empty(max(n.value, 256) + 1024, dtype=torch.uint8, device=dev)
    skip = (-buf.data_ptr()) % 1024          # the library wants a 1024-byte aligned workspace
    return buf[skip: skip + max(n.value, 256)]


def _prep_inputs(q, k, v, g, beta, lam, cu_seqlens):
    dev = L.require_cuda(q, k, v, g, beta, lam)          # cu_seqlens may live on the host: it is copied over
    if v.shape[:3] != q.shape[:3] or k.shape != q.shape or g.shape != q.shape[:3] or beta.shape != q.shape[:3]:
        raise ValueError("q/k [B,T,H,K], v [B,T,H,V], g/beta [B,T,H] expected")
    q, k, v, g, beta = (x.contiguous() for x in (q, k, v, g, beta))
    if g.dtype != beta.dtype:
        beta = beta.to(g.dtype)
    if lam is not None:
        if lam.shape[:3] != q.shape[:3]:
            raise ValueError("l must be [B,T,H,L]")
        lam = lam.contiguous()
    if cu_seqlens is not None:
        cu_seqlens = cu_seqlens.to(device=dev, dtype=torch.int64).contiguous()
    return dev, q, k, v, g, beta, lam, cu_seqlens


def chunk_gated_delta_rule(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    beta: torch.Tensor,
    scale: float = None,
    initial_state: torch.Tensor = None,
    output_final_state: bool = False,
    cu_seqlens: Optional[torch.LongTensor] = None,
    head_first: bool = False,
    use_qk_l2norm_in_kernel: bool = False,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Chunkwise gated-delta-rule forward.

    q, k: [B,T,H,K]; v: [B,T,H,V]; g (log decay), beta: [B,T,H]; initial_state: [N,H,K,V];
    cu_seqlens: [N+1] with B == 1.  Returns (o [B,T,H,V] in q's dtype, final_state [N,H,K,V]
    fp32 or None).  fp32 q/k/v are rejected as in the reference (gated_delta_rule_ori.py:313):
    the tensor-core operands are bf16, so an fp32 call could not honour fp32 accuracy.
    """
    _common_checks(q, k, v, beta, head_first, cu_seqlens, initial_state)
    _forward_only(q, k, v, g, beta, initial_state)
    if scale is None:
        scale = k.shape[-1] ** -0.5
    if torch.compiler.is_compiling():          # one opaque node in the traced graph (see torch_ops.py)
        from . import torch_ops  # noqa: F401
        o, ht = torch.ops.lampa_b200.gdn_fwd(q, k, v, g, beta, float(scale), initial_state, cu_seqlens,
                                             bool(use_qk_l2norm_in_kernel))
        return o, (ht if output_final_state else None)
    _check_cu_seqlens(cu_seqlens, q.shape[1])
    with torch.no_grad():
        return _gdn_plain(q, k, v, g, beta, scale, initial_state, output_final_state, cu_seqlens,
                          use_qk_l2norm_in_kernel)


@torch.no_grad()
def _gdn_plain(q, k, v, g, beta, scale, initial_state, output_final_state, cu_seqlens, use_qk_l2norm_in_kernel):
    dev, q, k, v, g, beta, _, cu = _prep_inputs(q, k, v, g, beta, None, cu_seqlens)
    B, T, H, K = q.shape
    V = v.shape[-1]
    N = B if cu is None else len(cu) - 1
    h0 = None
    if initial_state is not None:
        L.require_cuda(initial_state)
        if tuple(initial_state.shape) != (N, H, K, V):
            raise ValueError(f"initial_state must be [{N},{H},{K},{V}]")
        h0 = initial_state.to(torch.float32).contiguous()
    desc = _desc(q, v, g, None, cu, use_qk_l2norm_in_kernel, scale)
    o = torch.empty(B, T, H, V, dtype=q.dtype, device=dev)
    ht = torch.empty(N, H, K, V, dtype=torch.float32, device=dev) if output_final_state else None
    ws = _workspace(desc, dev)
    st = L.status_word(dev)
    rc = L.lib().lampa_gdn_fwd(ctypes.byref(desc), L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(g), L.ptr(beta),
                               L.ptr(h0), L.ptr(cu), L.ptr(o), L.ptr(ht), L.ptr(ws), ws.numel(),
                               L.ptr(st), L.stream_ptr(dev))
    L.check(rc, "lampa_gdn_fwd")
    if L.debug_checks():
        L.check_status(dev)
    return o, ht


class HState:
    """Fenwick state of the hierarchical rule (models/hattention/recurrent.py:9-131): `states`
    [B,H,K,V,L] and `counts` [L] int32 (tokens held per level).  Always fp32 on the device; the
    cascade / insert / dot methods of the reference live in the library's step kernel."""

    def __init__(self, base: int, htype, hstruct, shape, dtype: torch.dtype, device, empty: bool = False) -> None:
        if getattr(htype, "name", htype) != "WEAK" or base != 2:
            raise NotImplementedError
        if dtype != torch.float32:
            raise NotImplementedError("states are kept in fp32")
        self.base = base
        self.htype = htype
        self.hstruct = hstruct
        self.shape = tuple(shape)
        self.dtype = dtype
        self.device = torch.device(device)
        self.max_num_levels = self.shape[-1]
        if empty:                      # the caller attaches tensors it already has
            self.states = self.counts = None
            return
        self.states = torch.zeros(self.shape, dtype=dtype, device=device)
        self.counts = torch.zeros(self.max_num_levels, dtype=torch.int32, device=device)

    def reset_states(self) -> None:
        self.states.zero_()

    def to(self, dtype: Optional[torch.dtype] = None, device=None) -> "HState":
        new = HState.__new__(HState)
        new.__dict__.update(self.__dict__)
        new.dtype = self.dtype if dtype is None else dtype
        new.device = self.device if device is None else torch.device(device)
        new.states = self.states.to(dtype=new.dtype, device=new.device)
        new.counts = self.counts.to(dtype=torch.int32, device=new.device)
        return new


@torch.no_grad()
def _hgdn(q, k, v, g, beta, lam, cu_seqlens, use_l2norm, want_state: bool = False, out_perm=None):
    _check_cu_seqlens(cu_seqlens, q.shape[1], lam.shape[-1])
    dev, q, k, v, g, beta, lam, cu = _prep_inputs(q, k, v, g, beta, lam, cu_seqlens)
    B, T, H, K = q.shape
    V = v.shape[-1]
    if cu is None and lam.shape[-1] < num_levels_required(T):
        raise ValueError(f"l has {lam.shape[-1]} levels, a sequence of {T} tokens needs {num_levels_required(T)}")
    if K > 256:
        raise NotImplementedError("current kernel does not support head dimension larger than 256.")
    desc = _desc(q, v, g, lam, cu, use_l2norm, 1.0)
    o = torch.empty(B, T, H, V, dtype=q.dtype, device=dev)
    ws = _workspace(desc, dev)
    st = L.status_word(dev)
    if out_perm is None:
        rc = L.lib().lampa_hgdn_fwd(ctypes.byref(desc), L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(g), L.ptr(beta),
                                    L.ptr(lam), L.ptr(cu), L.ptr(o), L.ptr(ws), ws.numel(), L.ptr(st),
                                    L.stream_ptr(dev))
    else:
        L.require_cuda(out_perm)
        if out_perm.dtype != torch.int64 or out_perm.dim() != 1 or not out_perm.is_contiguous() or out_perm.numel() > B * T:
            raise ValueError("out_perm must be a contiguous int64 vector of at most B*T row indices")
        rc = L.lib().lampa_hgdn_fwd_scatter(ctypes.byref(desc), L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(g), L.ptr(beta),
                                            L.ptr(lam), L.ptr(cu), L.ptr(out_perm), out_perm.numel(), L.ptr(o),
                                            L.ptr(ws), ws.numel(), L.ptr(st), L.stream_ptr(dev))
    L.check(rc, "lampa_hgdn_fwd")
    states = counts = None
    if want_state:
        N = B if cu is None else len(cu) - 1
        Lv = lam.shape[-1]
        states = torch.empty(N, H, K, V, Lv, dtype=torch.float32, device=dev)
        counts = torch.empty(N, Lv, dtype=torch.int32, device=dev)
        rc = L.lib().lampa_hgdn_final_state(ctypes.byref(desc), L.ptr(k), L.ptr(v), L.ptr(g), L.ptr(beta),
                                            L.ptr(cu), L.ptr(ws), ws.numel(), L.ptr(states), L.ptr(counts),
                                            L.ptr(st), L.stream_ptr(dev))
        L.check(rc, "lampa_hgdn_final_state")
    if L.debug_checks():
        L.check_status(dev)
    return (o, states, counts) if want_state else o


@torch.no_grad()
def _hgdn_step(hstate: HState, q, k, v, g, beta, lam, use_l2norm: bool = True) -> torch.Tensor:
    """One token per batch row: q,k [B,H,K]; v [B,H,V]; g,beta [B,H]; lam [B,H,L] (as given to
    the kernel, i.e. not divided by scale).  Updates hstate in place, returns o [B,H,V]."""
    dev = L.require_cuda(q, k, v, g, beta, lam, hstate.states, hstate.counts)
    B, H, K = q.shape
    V = v.shape[-1]
    Lv = lam.shape[-1]
    if tuple(hstate.states.shape) != (B, H, K, V, Lv) or hstate.states.dtype != torch.float32:
        raise ValueError(f"state must be fp32 [{B},{H},{K},{V},{Lv}]")
    if not hstate.states.is_contiguous():
        hstate.states = hstate.states.contiguous()
    q, k, v, g, lam = (x.contiguous() for x in (q, k, v, g, lam))
    beta = beta.to(g.dtype).contiguous()
    desc = L.GdnDesc(B=B, T=1, H=H, K=K, V=V, L=Lv, nseq=0, qkv_dtype=L.dtype_code(q.dtype),
                     gb_dtype=L.dtype_code(g.dtype), lam_dtype=L.dtype_code(lam.dtype),
                     use_l2norm=int(bool(use_l2norm)), scale=1.0)
    o = torch.empty(B, H, V, dtype=q.dtype, device=dev)
    st = L.status_word(dev)
    rc = L.lib().lampa_hgdn_step(ctypes.byref(desc), L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(g), L.ptr(beta),
                                 L.ptr(lam), L.ptr(hstate.states), L.ptr(hstate.counts), L.ptr(o),
                                 L.ptr(st), L.stream_ptr(dev))
    L.check(rc, "lampa_hgdn_step")
    if L.debug_checks():
        L.check_status(dev)
    return o


@torch.no_grad()
def _hgdn_prefill(q, k, v, g, beta, lam, use_l2norm: bool = True):
    """(o, HState) after all T tokens: whole chunks through the chunkwise kernels, the remaining
    T mod 64 tokens through the step kernel — the split hattention_prefill makes
    (models/hattention/kernel.py:470-560)."""
    B, T, H, K = q.shape
    V, Lv = v.shape[-1], lam.shape[-1]
    dev = L.require_cuda(q, k, v, g, beta, lam)
    T0 = T - T % CHUNK
    hstate = HState(2, HType.WEAK, HStruct.GDELTA, (B, H, K, V, Lv), torch.float32, dev)
    o = torch.empty(B, T, H, V, dtype=q.dtype, device=dev)
    if T0 > 0:
        o0, states, counts = _hgdn(q[:, :T0], k[:, :T0], v[:, :T0], g[:, :T0], beta[:, :T0], lam[:, :T0],
                                   None, use_l2norm, want_state=True)
        o[:, :T0] = o0
        hstate.states = states
        hstate.counts = counts[0].contiguous()
    for t in range(T0, T):
        o[:, t] = _hgdn_step(hstate, q[:, t], k[:, t], v[:, t], g[:, t], beta[:, t], lam[:, t], use_l2norm)
    return o, hstate


def chunk_h_gated_delta_rule(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    l: torch.Tensor,
    beta: torch.Tensor,
    scale: float = None,
    initial_state: Optional[HState] = None,
    output_final_state: bool = False,
    cu_seqlens: Optional[torch.LongTensor] = None,
    head_first: bool = False,
    use_qk_l2norm_in_kernel: bool = False,
    out_perm: Optional[torch.LongTensor] = None,
):
    """Hierarchical (Fenwick-level) chunkwise gated-delta-rule forward.

    l: [B,T,H,L] level weights.  The reference divides l by `scale` and multiplies the
    normalised q by it (gated_delta_rule_apis.py:68-70, kernel.py:109-111); the two cancel, so
    the kernels take l as given and the result does not depend on `scale`.
    The three branches of the reference (gated_delta_rule_apis.py:72-129):
      output_final_state=False                  -> (o, None)
      output_final_state=True, no initial_state -> (o, HState) after all T tokens (prefill)
      output_final_state=True, initial_state    -> T must be 1: one decode step on the state
                                                   (updated in place and returned)
    Beyond the reference: `cu_seqlens` and T not a multiple of 64 are accepted by the first branch,
    and `cu_seqlens` by the second: the returned HState then holds one state per sequence
    (`states` [N,H,K,V,L], `counts` [N,L]); a sequence whose length is not a multiple of 64 is
    completed by null tokens (k = v = 0, beta = 0, g = 0), which its counts include.
    `out_perm` (int64 [n <= B*T], first branch only) folds the un-ordering of a sorted event into the output store:
    row t of the result lands in o.view(B*T, H, V)[out_perm[t]] for t < n (hmamba.py:451-455 gathers with the inverse
    permutation in a second pass); rows from n on stay where they are.
    Device-side problems (a wait that ran out, device-resident cu_seqlens that are malformed or
    need more levels than l has) are reported through `check_status()`.
    """
    _common_checks(q, k, v, beta, head_first, cu_seqlens, None)
    assert use_qk_l2norm_in_kernel is True
    _forward_only(q, k, v, g, l, beta)
    if output_final_state is False:
        if initial_state is not None:
            raise NotImplementedError
        if torch.compiler.is_compiling() and out_perm is None:      # one opaque node in the traced graph (see torch_ops.py)
            from . import torch_ops  # noqa: F401
            return torch.ops.lampa_b200.hgdn_fwd(q, k, v, g, beta, l, cu_seqlens, True), None
        return _hgdn(q, k, v, g, beta, l, cu_seqlens, True, out_perm=out_perm), None
    if cu_seqlens is not None:
        if initial_state is not None:
            raise NotImplementedError("a decode step takes one token per batch row, not packed sequences")
        o, states, counts = _hgdn(q, k, v, g, beta, l, cu_seqlens, True, want_state=True)
        hs = HState(2, HType.WEAK, HStruct.GDELTA, tuple(states.shape), torch.float32, states.device, empty=True)
        hs.states, hs.counts = states, counts
        return o, hs
    if initial_state is None:
        return _hgdn_prefill(q, k, v, g, beta, l, True)
    if not all([q.ndim == 4, q.shape[1] == 1, k.ndim == 4, k.shape[1] == 1, v.ndim == 4, v.shape[1] == 1,
                beta.ndim == 3, beta.shape[1] == 1, g.ndim == 3, g.shape[1] == 1,
                l.ndim == 4, l.shape[1] == 1]):
        raise ValueError
    o = _hgdn_step(initial_state, q[:, 0], k[:, 0], v[:, 0], g[:, 0], beta[:, 0], l[:, 0], True)
    return o.unsqueeze(1), initial_state


def hattention_prefill(q, k, v, b, g, l, scale, head_first, level_base, htype, hstruct,
                       chunk_size: Optional[int] = None, use_qk_l2norm_in_kernel: bool = False):
    """hattention_prefill of models/hattention/kernel.py:470-560 for GDELTA / WEAK / base 2:
    returns (o, HState).  `l` is the weight the reference kernel sees (already divided by scale)."""
    if getattr(hstruct, "name", hstruct) != "GDELTA" or getattr(htype, "name", htype) != "WEAK" or level_base != 2:
        raise NotImplementedError
    if head_first or (chunk_size is not None and chunk_size != CHUNK):
        raise NotImplementedError
    if not use_qk_l2norm_in_kernel or scale is None or b is None:
        raise NotImplementedError
    return _hgdn_prefill(q, k, v, g, b, l * scale, True)


def hattention_step(hstate: HState, q, k, v, b, g, l, scale, level_base, htype, hstruct,
                    use_qk_l2norm_in_kernel: bool = False):
    """hattention_step of models/hattention/kernel.py:570-633: q,k [B,H,K]; v [B,H,V]; b,g [B,H];
    l [B,H,L].  Returns (o [B,H,V], hstate) with hstate updated in place."""
    if not all([q.ndim == 3, k.ndim == 3, v.ndim == 3, b.ndim == 2 if b is not None else True,
                g.ndim == 2, l.ndim == 3, q.dtype == k.dtype, q.dtype == v.dtype,
                hstate.base == level_base]):
        raise TypeError
    if getattr(hstruct, "name", hstruct) != "GDELTA" or getattr(htype, "name", htype) != "WEAK" or level_base != 2:
        raise NotImplementedError
    if not use_qk_l2norm_in_kernel or scale is None or b is None:
        raise NotImplementedError
    return _hgdn_step(hstate, q, k, v, g, b, l * scale, True), hstate


def hattention_kernel(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    b: Optional[torch.Tensor],
    g: torch.Tensor,
    l: torch.Tensor,
    scale: Optional[float],
    head_first: bool,
    level_base: int,
    htype,
    hstruct,
    chunk_sizes=None,
    chunkwise: bool = True,
    use_qk_l2norm_in_kernel: bool = False,
) -> torch.Tensor:
    """The GDELTA / WEAK / base-2 / chunkwise branch of hattention_kernel (kernel.py:100-120):
    o = sum over levels of l * (l2norm(q) * scale)^T (...).  Other branches raise, as there."""
    if getattr(hstruct, "name", hstruct) != "GDELTA" or not chunkwise:
        raise NotImplementedError
    if getattr(htype, "name", htype) != "WEAK" or level_base != 2:
        raise NotImplementedError
    if b is None:
        raise ValueError
    if chunk_sizes is not None and (chunk_sizes[0] != chunk_sizes[1] or chunk_sizes[0] != CHUNK):
        raise NotImplementedError
    if not use_qk_l2norm_in_kernel or scale is None or head_first:
        raise NotImplementedError
    return _hgdn(q, k, v, g, b, l * scale, None, True)
