"""ctypes binding of liblampa_b200.so (see include/lampa_b200.h).

There is no fallback: if the library is missing or no CUDA device is present the
public ops raise.  torch is used only for device memory and streams.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(_HERE, "liblampa_b200.so")

LAMPA_BF16, LAMPA_F16, LAMPA_F32 = 0, 1, 2
LAMPA_KEY_I32, LAMPA_KEY_F32 = 0, 1
ERR_TIMEOUT, ERR_LEVELS, ERR_BOUNDS, ERR_TOO_LARGE = -5, -6, -7, -8
SEGSORT_STATIC_MAX_KEYS = 1572864

_DTYPES = {torch.bfloat16: LAMPA_BF16, torch.float16: LAMPA_F16, torch.float32: LAMPA_F32}


class LampaError(RuntimeError):
    pass


class GdnDesc(ctypes.Structure):
    _fields_ = [("B", ctypes.c_int32), ("T", ctypes.c_int32), ("H", ctypes.c_int32), ("K", ctypes.c_int32),
                ("V", ctypes.c_int32), ("L", ctypes.c_int32), ("nseq", ctypes.c_int32),
                ("qkv_dtype", ctypes.c_int32), ("gb_dtype", ctypes.c_int32), ("lam_dtype", ctypes.c_int32),
                ("use_l2norm", ctypes.c_int32), ("scale", ctypes.c_float)]


_lib: Optional[ctypes.CDLL] = None
EXPORTS = ["lampa_version", "lampa_error_string", "lampa_gdn_workspace_bytes", "lampa_gdn_workspace_layout",
           "lampa_gdn_fwd", "lampa_hgdn_fwd", "lampa_hgdn_fwd_scatter", "lampa_hgdn_final_state", "lampa_hgdn_step", "lampa_lsh_hash", "lampa_segsort_workspace_bytes",
           "lampa_segsort_stable", "lampa_permute_rows", "lampa_invert_perm", "lampa_segsort_stable_static",
           "lampa_short_conv_fwd", "lampa_short_conv_step", "lampa_gate_inputs", "lampa_rmsnorm_gate", "lampa_add_rmsnorm",
           "lampa_row_range", "lampa_quantile_regions", "lampa_geo_keys",
           "lampa_bucket_rbf_attn", "lampa_bucket_attn_combine", "lampa_hept_prep_qk",
           "lampa_profile_enable",
           "lampa_profile_read", "lampa_debug_set_poll_budget", "lampa_debug_set_tick_buffer",
           "lampa_debug_force_mma_sync"]


def lib() -> ctypes.CDLL:
    """Load the CUDA library; raises LampaError when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(SO_PATH):
            raise LampaError(f"{SO_PATH} is missing: build it with `python -m lampa_b200.build` "
                             "(there is no CPU or PyTorch fallback)")
        L = ctypes.CDLL(SO_PATH)
        L.lampa_error_string.restype = ctypes.c_char_p
        L.lampa_error_string.argtypes = [ctypes.c_int]
        vp, i32, i64, sz = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_size_t
        L.lampa_gdn_workspace_bytes.argtypes = [ctypes.POINTER(GdnDesc), ctypes.POINTER(sz)]
        L.lampa_gdn_workspace_layout.argtypes = [ctypes.POINTER(GdnDesc), ctypes.POINTER(sz)]
        L.lampa_gdn_fwd.argtypes = [ctypes.POINTER(GdnDesc)] + [vp] * 10 + [sz, vp, vp]
        L.lampa_hgdn_fwd.argtypes = [ctypes.POINTER(GdnDesc)] + [vp] * 9 + [sz, vp, vp]
        L.lampa_hgdn_fwd_scatter.argtypes = [ctypes.POINTER(GdnDesc)] + [vp] * 8 + [i64, vp, vp, sz, vp, vp]
        L.lampa_hgdn_final_state.argtypes = [ctypes.POINTER(GdnDesc)] + [vp] * 6 + [sz, vp, vp, vp, vp]
        L.lampa_hgdn_step.argtypes = [ctypes.POINTER(GdnDesc)] + [vp] * 11
        L.lampa_lsh_hash.argtypes = [vp, i64, i64, vp, vp, ctypes.c_float, i64, i32, i32, i32, vp, vp, vp, vp]
        L.lampa_segsort_workspace_bytes.argtypes = [i64, ctypes.POINTER(sz)]
        L.lampa_segsort_stable.argtypes = [vp, i32, i64, vp, i32, vp, vp, vp, sz, vp, vp]
        L.lampa_segsort_stable_static.argtypes = [vp, i32, i64, vp, i32, vp, vp, vp, vp]
        L.lampa_permute_rows.argtypes = [vp, vp, vp, i32, i64, i64, i32, vp, vp, vp]
        L.lampa_invert_perm.argtypes = [vp, vp, i32, i64, vp, vp, vp]
        L.lampa_row_range.argtypes = [vp, vp, i32, i64, vp, vp, vp, vp]
        L.lampa_quantile_regions.argtypes = [vp, vp, i32, i64, vp, vp]
        L.lampa_geo_keys.argtypes = [vp] * 8 + [i32, i64, i64, vp, vp]
        L.lampa_bucket_rbf_attn.argtypes = [vp] * 5 + [i32, i32, i64, i32, i32, i32, i32, i32, i32, i32, vp, vp, vp]
        L.lampa_bucket_attn_combine.argtypes = [vp, vp, i32, i64, i32, vp, vp]
        L.lampa_hept_prep_qk.argtypes = [vp] * 5 + [i64, i32, i32, i32, i32, i64, vp, vp, vp, vp]
        L.lampa_short_conv_fwd.argtypes = [vp, vp, vp, vp, vp, i32, i64, i64, i32, i32, i32, i32, i32, vp, vp, i32, vp]
        L.lampa_short_conv_step.argtypes = [vp, vp, vp, vp, vp, i64, i32, i32, i32, i32, i32, vp, vp]
        L.lampa_gate_inputs.argtypes = [vp] * 7 + [i64, i32, i32, i32, i32, i32, i32, vp, vp, vp, vp]
        L.lampa_rmsnorm_gate.argtypes = [vp, vp, vp, i64, i32, i32, i32, ctypes.c_float, i32, vp, vp]
        L.lampa_add_rmsnorm.argtypes = [vp, vp, i32, vp, vp, i32, i64, i32, vp, ctypes.c_float, i32, i32, vp, i32, vp, vp]
        L.lampa_profile_enable.argtypes = [ctypes.c_int]
        L.lampa_debug_set_poll_budget.argtypes = [ctypes.c_int]
        L.lampa_debug_force_mma_sync.argtypes = [ctypes.c_int]
        L.lampa_debug_set_tick_buffer.argtypes = [vp, ctypes.c_int]
        L.lampa_profile_read.argtypes = [ctypes.c_char_p, sz, ctypes.POINTER(ctypes.c_float),
                                         ctypes.POINTER(i32), i32, ctypes.POINTER(i32)]
        for name in EXPORTS:
            if name != "lampa_error_string":
                getattr(L, name).restype = ctypes.c_int
        _lib = L
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise LampaError(f"{what}: {lib().lampa_error_string(rc).decode()} ({rc})")


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise TypeError(f"unsupported dtype {dt}") from None


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise LampaError("lampa_b200 ops run on CUDA tensors only (no CPU path)")
        if dev is not None and t.device != dev:
            raise LampaError("all tensors must be on the same device")
        dev = t.device
    return dev


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_ptr(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


_status: Dict[int, torch.Tensor] = {}


def status_word(dev: torch.device) -> torch.Tensor:
    """Device int32[4] the kernels report into (code, where, detail, -)."""
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(4, dtype=torch.int32, device=dev)
    return _status[idx]


def check_status(dev: Optional[torch.device] = None) -> None:
    """Synchronise and raise if a kernel reported a device-side error since the last check."""
    devs = list(_status) if dev is None else [dev.index if dev.index is not None else torch.cuda.current_device()]
    for idx in devs:
        if idx not in _status:
            continue
        vals = _status[idx].tolist()
        if vals[0] != 0:
            _status[idx].zero_()
            raise LampaError(f"device-side error: {lib().lampa_error_string(vals[0]).decode()} "
                             f"(code {vals[0]}, where {vals[1]}, detail {vals[2]})")


def debug_checks() -> bool:
    return os.environ.get("LAMPA_B200_CHECK", "0") not in ("", "0")


def profile_enable(on: bool) -> None:
    """Turn per-kernel CUDA-event timing inside the library on or off (clears earlier records)."""
    check(lib().lampa_profile_enable(int(on)), "lampa_profile_enable")


def profile_read() -> Dict[str, Dict[str, float]]:
    """{kernel name: {"ms": summed milliseconds, "launches": count}} since profiling was enabled."""
    names = ctypes.create_string_buffer(4096)
    ms = (ctypes.c_float * 64)()
    cnt = (ctypes.c_int32 * 64)()
    n = ctypes.c_int32(0)
    check(lib().lampa_profile_read(names, 4096, ms, cnt, 64, ctypes.byref(n)), "lampa_profile_read")
    out = {}
    for i, nm in enumerate(names.value.decode().split("\n")[: n.value]):
        out[nm] = {"ms": float(ms[i]), "launches": int(cnt[i])}
    return out
