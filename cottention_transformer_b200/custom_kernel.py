"""Drop-in for ``Cuda_Kernel/Custom_Kernel.py``: the ``CustomAttention`` autograd Function.

Same contract as the reference (``Custom_Kernel.py:7-141``): ``forward(ctx, Q, K, V)`` makes the
inputs contiguous, saves them, and dispatches on ``Q.dtype`` to ``kernel.<dtype>(Q, K, V, 1, False,
False)`` (``:9-32``); ``backward`` runs the three permuted scans (``:106-108``)

    grad_Q = kernel(grad_output, V, K, rev=False)
    grad_K = kernel(V, grad_output, Q, rev=True)
    grad_V = kernel(K, Q, grad_output, rev=True)

each through the same name-dispatch, so the autocast rules of the entry points apply to the
backward exactly as they do in the reference.  Passes ``torch.autograd.gradcheck`` in float64, the
reference's only correctness check (``:184-188``).
"""
from __future__ import annotations

import torch

from . import kernel

_BY_DTYPE = {
    torch.float32: kernel.float32,
    torch.float64: kernel.float64,
    torch.float16: kernel.float16,
    torch.bfloat16: kernel.bfloat16,
}


class CustomAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, Q, K, V):
        Q = Q.contiguous()
        K = K.contiguous()
        V = V.contiguous()
        ctx.save_for_backward(Q, K, V)
        fn = _BY_DTYPE.get(Q.dtype)
        if fn is None:
            raise ValueError("Only float32, float64, float16, and bfloat16 are supported")
        return fn(Q, K, V, 1, False, False)

    @staticmethod
    def backward(ctx, grad_output):
        Q, K, V = ctx.saved_tensors
        Q = Q.contiguous()
        K = K.contiguous()
        V = V.contiguous()
        grad_output = grad_output.contiguous()
        fn = _BY_DTYPE.get(Q.dtype)
        if fn is None:
            raise ValueError("Only float32, float64, float16, and bfloat16 are supported")
        grad_Q = fn(grad_output, V, K, 1, False, False)
        grad_K = fn(V, grad_output, Q, 1, False, True)
        grad_V = fn(K, Q, grad_output, 1, False, True)
        return grad_Q, grad_K, grad_V
