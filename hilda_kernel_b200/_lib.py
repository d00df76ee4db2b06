"""ctypes binding of libhilda_b200.so (the C ABI declared in include/hilda_b200.h).

There is no CPU or PyTorch fallback: if the library is missing or a call returns an error the
operator raises.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("HILDA_LIB_PATH") or os.path.join(_PKG, "libhilda_b200.so")  # HILDA_LIB_PATH: another build of the same ABI
# HILDA_DEBUG=1 prefers the library built with -DHILDA_DEBUG (python -m hilda_kernel_b200._build --debug)
if os.environ.get("HILDA_DEBUG", "0") not in ("", "0") and os.path.exists(os.path.join(_PKG, "libhilda_b200_debug.so")):
    LIB_PATH = os.path.join(_PKG, "libhilda_b200_debug.so")

F32, BF16, F16 = 0, 1, 2
_DT = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}

_ERR = {
    -1: "unsupported dtype", -2: "misaligned pointer", -3: "unsupported size", -4: "CUDA launch/runtime error",
    -5: "null pointer", -6: "device status: a bounded wait ran out", -7: "inconsistent arguments",
}

# Device status words (written by kernels, never read on the default path because reading one is a
# host synchronisation). HILDA_DEBUG=1 in the environment, or DEBUG = True here, makes every operator
# that has a status word read it after the call and raise.
DEBUG = os.environ.get("HILDA_DEBUG", "0") not in ("", "0")
_STATUS = {31: "a target / token id outside [0, V)"}

_p, _i64, _i32, _f32 = C.c_void_p, C.c_int64, C.c_int, C.c_float

# name -> (restype, argtypes); must list every symbol include/hilda_b200.h declares
SIGNATURES = {
    "hilda_rms_norm_fwd": (_i32, [_p, _p, _p, _p, _i64, _i64, _f32, _i32, _i32, _p]),
    "hilda_fused_add_rms_norm_fwd": (_i32, [_p, _p, _p, _p, _p, _p, _i64, _i64, _f32, _i32, _i32, _p]),
    "hilda_norm_bwd_workspace_bytes": (_i64, [_i64, _i64, _i32]),
    "hilda_norm_bwd": (_i32, [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i32, _i32, _p]),
    "hilda_norm_bwd_set_path": (_i32, [_i32]),
    "hilda_norm_bwd_noalloc_max_bytes": (_i64, []),
    "hilda_norm_bwd_noalloc": (_i32, [_p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i32, _i32, _p]),
    "hilda_rope": (_i32, [_p, _p, _p, _i32, _p, _p, _p, _i32, _p, _p, _i64, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _p]),
    "hilda_swiglu_fwd": (_i32, [_p, _p, _p, _i64, _i32, _p]),
    "hilda_swiglu_bwd": (_i32, [_p, _p, _p, _p, _p, _i64, _i32, _p]),
    "hilda_geglu_fwd": (_i32, [_p, _p, _p, _i64, _i32, _p]),
    "hilda_geglu_bwd": (_i32, [_p, _p, _p, _p, _p, _i64, _i32, _p]),
    "hilda_cross_entropy_workspace_bytes": (_i64, [_i64]),
    "hilda_cross_entropy_fwd": (_i32, [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i32, _i32, _p]),
    "hilda_scale_rows": (_i32, [_p, _p, _p, _i32, _i64, _i64, _i32, _p]),
    "hilda_grpo_workspace_bytes": (_i64, [_i64]),
    "hilda_grpo_loss_fwd": (_i32, [_p] * 13 + [_i64, _i64, _i64, _i64, _f32, _f32, _f32, _f32, _i32, _p]),
    "hilda_selective_log_softmax": (_i32, [_p, _p, _p, _p, _i64, _i64, _i64, _f32, _i32, _p]),
    "hilda_row_engine_force": (None, [_i32, _i32, _i32]),
    "hilda_row_engine_plan": (_i32, [_i64, _i32, _p]),
    "hilda_row_engine_has_kernel": (_i32, [_i32, _i32, _i32, _i32]),
    "hilda_count_valid": (_i32, [_p, _i64, _i64, _p, _p]),
    "hilda_flce_logits_pitch": (_i64, [_i64]),
    "hilda_flce_padded_rows": (_i64, [_i64]),
    "hilda_flce_stat_tiles": (_i64, [_i64]),
    "hilda_flce_logits": (_i32, [_p, _p, _p, _p, _i64, _i64, _i64, _i32, _p, _p, _i64, _p]),
    "hilda_flce_logits_scaled": (_i32, [_p, _p, _p, _p, _i64, _i64, _i64, _f32, _i32, _p, _p]),
    "hilda_kl_div_fwd": (_i32, [_p, _p, _p, _p, _i64, _i64, _i32, _i32, _f32, _i32, _p]),
    "hilda_kl_div_bwd": (_i32, [_p, _p, _p, _i64, _i64, _i32, _i32, _i32, _p]),
    "hilda_jsd_fwd": (_i32, [_p, _p, _p, _p, _p, _p, _i64, _p, _i64, _i64, _f32, _i32, _p]),    "hilda_paged_attention_fp8_workspace_bytes": (_i64, [_i64] * 5),
    "hilda_paged_attention_fp8_decode": (_i32, [_p, _i64, _i64, _p, _i64, _i64, _i64, _p, _i64, _i64, _i64, _p, _i64, _i64,
                                                _p, _i64, _p, _p, _f32, _i64, _i64, _i64, _i64, _i64, _i64, _p]),

    "hilda_attn_res_fwd": (_i32, [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _f32, _i32, _i32, _i32, _p]),
    "hilda_attn_res_set_path": (_i32, [_i32]),
    "hilda_attn_res_bwd_workspace_bytes": (_i64, [_i64, _i64]),
    "hilda_attn_res_bwd": (_i32, [_p] * 10 + [_i64, _i64, _i64, _i32, _i32, _i32, _p]),
    "hilda_fljsd_dlogits": (_i32, [_p, _p, _p, _p, _p, _i64, _p, _i64, _p, _i64, _i64, _f32, _f32, _i32, _p]),
    "hilda_flce_row_stats": (_i32, [_p, _p, _p, _p, _i64, _i64, _i64, _i32, _p, _i64, _p]),
    "hilda_flce_finalize": (_i32, [_p, _i32, _p, _i64, _p, _p, _i64, _p, _i64, _p]),
    "hilda_flce_dlogits": (_i32, [_p, _p, _p, _i64, _p, _i64, _i64, _i64, _i32, _p, _i64, _p]),
    "hilda_flce_grad_hidden": (_i32, [_p, _p, _p, _p, _i64, _i64, _i64, _i32, _p, _p, _i64, _p]),
    "hilda_flce_grad_weight": (_i32, [_p, _p, _p, _p, _i32, _i64, _i64, _i64, _i32, _p, _p, _i64, _p]),
    "hilda_flce_sum_loss": (_i32, [_p, _i64, _p, _i32, _p, _p, _p]),
    "hilda_flce_compact": (_i32, [_p, _i64, _i64, _p, _p, _p, _p, _p]),
    "hilda_gather_valid_rows": (_i32, [_p, _p, _p, _p, _i64, _i64, _p]),
    "hilda_scatter_valid_rows": (_i32, [_p, _p, _p, _i64, _i64, _p]),
    "hilda_scatter_valid_f32": (_i32, [_p, _p, _p, _i64, _p]),
    "hilda_flce_default_chunk_rows": (_i64, [_i64, _i64, _i64]),
    "hilda_flce_workspace_bytes": (_i64, [_i64, _i64, _i64, _i64, _i32, _i32]),
    "hilda_fused_linear_cross_entropy_fwd": (_i32, [_p] * 8 + [_i64, _i64, _i64, _i64, _i32, _i64, _i32, _i32, _p]),
    "hilda_flce_profile": (None, [_i32]),
    "hilda_flce_profile_collect": (_i32, [_p, _p]),
    "hilda_flce_profile_entry": (_i32, [_i32, _p, _p]),
    "hilda_gather_rows": (_i32, [_p, _p, _p, _i64, _i64, _p]),
    "hilda_scatter_rows": (_i32, [_p, _p, _p, _i64, _i64, _i64, _p]),
    "hilda_gemm_set_pair": (None, [_i32]),
    "hilda_gemm_get_pair": (_i32, []),
    "hilda_gemm_set_sm_limit": (None, [_i32]),
    "hilda_gemm_set_wait_cap": (None, [C.c_uint]),
    "hilda_debug_gemm_set_order": (None, [_i32]),
    "hilda_gemm_set_probe": (None, [_p, _i32]),
    "hilda_debug_gemm": (_i32, [_p, _i64, _p, _i64, _p, _p, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _p, _p]),
}

_lib = None


def lib() -> C.CDLL:
    """Load the library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} not found: build it with `python -m hilda_kernel_b200._build` "
                "(there is no fallback path)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def dt(t: torch.Tensor | torch.dtype) -> int:
    d = t.dtype if isinstance(t, torch.Tensor) else t
    if d not in _DT:
        raise TypeError(f"hilda_kernel_b200: unsupported dtype {d} (float32, bfloat16, float16 only)")
    return _DT[d]


def ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"hilda_kernel_b200.{what} failed: {_ERR.get(rc, 'error')} (code {rc})")


def check_status(word: torch.Tensor, what: str, force: bool = False) -> None:
    """Read a device status word (synchronises) when DEBUG or force; raise if it is non-zero."""
    if not (DEBUG or force):
        return
    code = int(word)
    if code != 0:
        why = _STATUS.get(code, "a bounded device-side wait ran out")
        raise RuntimeError(f"hilda_kernel_b200.{what}: device status {code} ({why})")


def require_cuda(*tensors: torch.Tensor | None) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("hilda_kernel_b200 operators run on CUDA tensors only (no CPU fallback)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"tensors on different devices: {dev} vs {t.device}")
    return dev


class device_guard:
    """Make `dev` the current CUDA device for the duration of a launch (cheap when it already is)."""

    def __init__(self, dev):
        self.idx = dev.index if dev.index is not None else torch.cuda.current_device()
        self.prev = None

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.idx:
            self.prev = cur
            torch.cuda.set_device(self.idx)
        return self

    def __exit__(self, *exc):
        if self.prev is not None:
            torch.cuda.set_device(self.prev)
        return False
