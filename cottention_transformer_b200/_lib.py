"""ctypes binding of ``libcottention_b200.so`` (the C ABI declared in ``include/cottention_b200.h``).

There is no fallback: if the library is missing or a call fails, a ``RuntimeError`` is raised.
"""
from __future__ import annotations

import ctypes
import os

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libcottention_b200.so")

COTT_F32, COTT_F64, COTT_F16, COTT_BF16 = 0, 1, 2, 3
DTYPE_CODE = {
    torch.float32: COTT_F32,
    torch.float64: COTT_F64,
    torch.float16: COTT_F16,
    torch.bfloat16: COTT_BF16,
}

_P, _I, _L = ctypes.c_void_p, ctypes.c_int, ctypes.c_long

# name -> argtypes; restype is int (status) unless listed in _STR
_SIGNATURES = {
    "cott_scan": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "cott_scan_bwd": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "cott_cos_attn_fwd": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "cott_cos_attn_bwd": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "cott_cos_attn_bwd_dq": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "cott_cos_attn_bwd_dkdv": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "cott_cos_attn_seg_count": [_I, _I, _I],
    "cott_cos_attn_fwd_seg": [_P, _P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _P],
    "cott_cos_attn_bwd_seg": [_P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "cott_cos_attn_fwd_train": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _P],
    "cott_cos_attn_bwd_train": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "cott_cos_attn_wide_fwd": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "cott_cos_attn_wide_bwd": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "cott_cos_attn_prefill_state": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "cott_decode_step": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, ctypes.c_longlong, _P, _P],
    "cott_decode_steps": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, ctypes.c_longlong, _P, _P],
    "cott_bidir_fwd": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "cott_bidir_bwd": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "cott_bidir_fwd_strided": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "cott_bidir_bwd_strided": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "cott_bidir_fwd_static": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "cott_rotary": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, ctypes.c_longlong, _I, _I, _P],
    "cott_cos_attn_fwd_rotary": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "cott_cos_attn_bwd_rotary": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "cott_check_status": [ctypes.POINTER(ctypes.c_int)],
    "cott_selftest_device_wait": [_I, _I, _I, _P],
}
_STR = {"cott_version": [], "cott_last_error": [], "cott_status_string": [_I]}
_SIZE = {"cott_bidir_scratch_bytes": [_I, _I, _I, _I, _I, _I], "cott_cos_attn_saved_bytes": [_I, _I, _I],
         "cott_cos_attn_wide_workspace_bytes": [_I, _I, _I], "cott_cos_attn_seg_workspace_bytes": [_I, _I, _I, _I]}

class CottRotaryTables(ctypes.Structure):
    """``cott_rotary_tables``: fp32 sin / cos tables, the rotary dim and the element stride between batch entries."""
    _fields_ = [("sin_table", ctypes.c_void_p), ("cos_table", ctypes.c_void_p), ("rot_dim", ctypes.c_int),
                ("table_batch_stride", ctypes.c_longlong)]


class CottLayout(ctypes.Structure):
    """``cott_layout``: element strides (batch, head, position) of q/k/v/dq/dk/dv and of out/dout."""
    _fields_ = [(n, ctypes.c_longlong) for n in ("in_b", "in_h", "in_n", "out_b", "out_h", "out_n")]


_lib = None
launch_count = 0  # kernels launched through this binding (bookkeeping for the benchmark)


def exported_symbols() -> list[str]:
    return sorted(list(_SIGNATURES) + list(_STR) + list(_SIZE))


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} not found: build it with `python -m cottention_transformer_b200.build` "
                "(there is no CPU or PyTorch fallback)"
            )
        L = ctypes.CDLL(LIB_PATH)
        for name, args in _SIGNATURES.items():
            fn = getattr(L, name)
            fn.argtypes, fn.restype = args, _I
        for name, args in _STR.items():
            fn = getattr(L, name)
            fn.argtypes, fn.restype = args, ctypes.c_char_p
        for name, args in _SIZE.items():
            fn = getattr(L, name)
            fn.argtypes, fn.restype = args, ctypes.c_size_t
        _lib = L
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        L = lib()
        raise RuntimeError(
            f"{what}: {L.cott_status_string(status).decode()} ({status}): {L.cott_last_error().decode()}"
        )


def check_device_status() -> None:
    """Synchronise and raise if a tensor-core kernel recorded a bounded wait that gave up."""
    detail = ctypes.c_int(0)
    check(lib().cott_check_status(ctypes.byref(detail)), "cott_check_status")


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()
