"""Drop-in for the reference's extension module ``FastAttention2.kernel``.

The reference builds ``FastAttention2.kernel`` from ``Cuda_Kernel/combined_kernel_general.cu``
(``Cuda_Kernel/setup.py:13-15``) and exports four functions with one signature
(``combined_kernel_general.cu:353,444-454``):

    float32 / float64 / float16 / bfloat16 (Q, K, V, block_size, inplace=False, reversed=False) -> Tensor

This module exports the same four names with the same argument meaning and error behaviour,
implemented by ``cott_scan`` of ``libcottention_b200.so``:

* ``out[b,h,s,:] = sum_{t<=s} (Q_s . K_t) V_t`` (``t>=s`` when ``reversed``), ``:126-168``;
* the entry-point name only selects the autocast target: the working dtype is
  ``autocast on and Q is float32 ? (float16 for float16, else bfloat16) : Q.dtype`` and K, V are
  cast to it (``:377-399``);
* inputs are made contiguous (``:397-399``); ``block_size`` is ignored (``:353``);
  ``inplace=True`` returns the (re-cast, contiguous) V holding the result (``:403-404``);
* the checks of ``:355-374`` raise ``RuntimeError`` with the reference's messages.

When the compiled torch binding has been built (``cott_torch_binding.so``, ``csrc_torch/torch_binding.cpp``) the four
names are its functions -- the reference's pybind signature in C++ -- and the Python statement of the same checks
below is the route without it.

Differences, on purpose: sums are kept in fp32/fp64 rather than the storage type, and the launch
goes to torch's current stream rather than the legacy default stream (``:262``).
"""
from __future__ import annotations

import torch

from . import _binding, _lib

__all__ = ["float32", "float64", "float16", "bfloat16", "scan"]


def scan(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, reversed: bool = False,
         out: torch.Tensor | None = None) -> torch.Tensor:
    """``cott_scan`` on contiguous CUDA tensors of one dtype; allocates ``out`` unless given."""
    B, H, N, Dk = Q.shape
    Dv = V.shape[3]
    if out is None:
        out = torch.empty((B, H, N, Dv), dtype=Q.dtype, device=Q.device)
    with torch.cuda.device(Q.device):
        st = _lib.lib().cott_scan(
            _lib.ptr(Q), _lib.ptr(K), _lib.ptr(V), _lib.ptr(out), B, H, N, Dk, Dv,
            _lib.DTYPE_CODE[Q.dtype], int(bool(reversed)), _lib.stream_ptr(Q.device),
        )
    _lib.check(st, "cott_scan")
    return out


def _forward(autocast_dtype: torch.dtype, Q, K, V, block_size, inplace=False, reversed=False):
    # combined_kernel_general.cu:355-357
    if not Q.is_cuda:
        raise RuntimeError("Q must be a CUDA tensor")
    if not K.is_cuda:
        raise RuntimeError("K must be a CUDA tensor")
    if not V.is_cuda:
        raise RuntimeError("V must be a CUDA tensor")
    if Q.dim() != 4 or K.dim() != 4 or V.dim() != 4:
        raise RuntimeError("Q, K and V must be 4-dimensional [N, H, S, D]")
    # :365
    if Q.size(3) != K.size(3):
        raise RuntimeError("Q and K must have the same dimension")
    D_attn = Q.size(3)
    # :372-374
    if D_attn % 16 != 0:
        raise RuntimeError("D_attn must be divisible by 16")
    if D_attn < 32:
        raise RuntimeError("D_attn must be greater than or equal to 16*2")
    if K.shape[:3] != Q.shape[:3] or V.shape[:3] != Q.shape[:3]:
        raise RuntimeError("Q, K and V must agree in their first three dimensions")
    int(block_size)  # accepted and ignored, as in the reference
    # :377-389
    if torch.is_autocast_enabled() and Q.dtype == torch.float32:
        data_type = autocast_dtype
    else:
        data_type = Q.dtype
    if data_type not in _lib.DTYPE_CODE:
        raise RuntimeError(f"\"forward_cuda\" not implemented for '{data_type}'")
    # :397-399
    Q = Q.contiguous().to(data_type)
    K = K.contiguous().to(data_type)
    V = V.contiguous().to(data_type)
    # :402-407
    out = V if inplace else None
    return scan(Q, K, V, reversed, out=out)


def float32(Q, K, V, block_size, inplace=False, reversed=False):
    m = _binding.module()
    if m is not None:  # the compiled entry point (same checks, same C call)
        return m.float32(Q, K, V, block_size, inplace, reversed)
    return _forward(torch.bfloat16, Q, K, V, block_size, inplace, reversed)


def float64(Q, K, V, block_size, inplace=False, reversed=False):
    m = _binding.module()
    if m is not None:  # the compiled entry point (same checks, same C call)
        return m.float64(Q, K, V, block_size, inplace, reversed)
    return _forward(torch.bfloat16, Q, K, V, block_size, inplace, reversed)


def float16(Q, K, V, block_size, inplace=False, reversed=False):
    m = _binding.module()
    if m is not None:  # the compiled entry point (same checks, same C call)
        return m.float16(Q, K, V, block_size, inplace, reversed)
    return _forward(torch.float16, Q, K, V, block_size, inplace, reversed)


def bfloat16(Q, K, V, block_size, inplace=False, reversed=False):
    m = _binding.module()
    if m is not None:  # the compiled entry point (same checks, same C call)
        return m.bfloat16(Q, K, V, block_size, inplace, reversed)
    return _forward(torch.bfloat16, Q, K, V, block_size, inplace, reversed)
