"""Recurrent decode state for cosine attention: the B200 replacement of the reference's
``fast_inference`` branch (``GPT_Trainer/GPTCosAttention.py:76-85,235-272``).

The reference keeps, per attention module, ``past_KV`` (float64 ``[1, H, d, d]``, V index first)
and ``cur_s`` (1-based position) as module attributes and loops over tokens in Python on the CPU.
``CosAttnDecodeState`` holds the same two things on the GPU -- float32 ``[B, H, d_v, d_k]`` plus a
position counter -- and advances them with ``cott_decode_step`` / ``cott_decode_steps``.
"""
from __future__ import annotations

import torch

from . import _lib


class CosAttnDecodeState:
    def __init__(self, batch: int, heads: int, d_k: int, d_v: int | None = None, device="cuda"):
        d_v = d_k if d_v is None else d_v
        self.state = torch.zeros(batch, heads, d_v, d_k, dtype=torch.float32, device=device)
        self.cur_s = 1  # GPTCosAttention.py:82

    def reset(self):
        self.state.zero_()
        self.cur_s = 1

    def prefill(self, q, k, v, norm_const):
        """Absorb a whole prompt at once (fresh state only): the outputs come from the fused causal kernels and the
        state from the segment-state kernels, instead of T recurrent steps.  bf16 / fp16, head dim 64 or 128; anything
        else falls back to ``step``.  Returns ``[B, H, T, d_v]``."""
        from .cos_attention import cos_attn_causal, fused_supported, wide_supported
        wide = wide_supported(q, k, v) and q.shape[-1] == 128
        if self.cur_s != 1 or not (wide or fused_supported(q, k, v)):
            return self.step(q, k, v, norm_const)
        B, H, T, D = q.shape
        k, v = k.contiguous(), v.contiguous()
        with torch.no_grad():
            out = cos_attn_causal(q, k, v, norm_const)
        L = _lib.lib()
        nc = norm_const.detach().reshape(-1).to(device=q.device, dtype=torch.float32).contiguous()
        with torch.cuda.device(q.device):
            nseg = 1 if wide else L.cott_cos_attn_seg_count(B, H, T)
            nbytes = L.cott_cos_attn_wide_workspace_bytes(B, H, T) if wide else L.cott_cos_attn_seg_workspace_bytes(B, H, T, nseg)
            ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=q.device)
            st = L.cott_cos_attn_prefill_state(_lib.ptr(k), _lib.ptr(v), _lib.ptr(nc), _lib.ptr(self.state), _lib.ptr(ws), nseg,
                                               0, B, H, T, D, D, _lib.DTYPE_CODE[q.dtype], _lib.stream_ptr(q.device))
        _lib.check(st, "cott_cos_attn_prefill_state")
        self.cur_s += T
        return out

    def step(self, q, k, v, norm_const):
        """q, k: ``[B, H, T, d_k]``; v: ``[B, H, T, d_v]`` (T >= 1 tokens, e.g. a prompt or one new
        token).  Returns ``[B, H, T, d_v]`` and advances the state and the position by T."""
        if not q.is_cuda:
            raise RuntimeError("decode needs CUDA tensors (there is no CPU path)")
        B, H, T, Dk = q.shape
        Dv = v.shape[-1]
        if q.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            raise RuntimeError("decode takes float32, float16 or bfloat16 tokens")
        q, k, v = q.contiguous(), k.to(q.dtype).contiguous(), v.to(q.dtype).contiguous()
        nc = norm_const.detach().reshape(-1).to(device=q.device, dtype=torch.float32).contiguous()
        out = torch.empty(B, H, T, Dv, dtype=q.dtype, device=q.device)
        with torch.cuda.device(q.device):
            st = _lib.lib().cott_decode_steps(
                _lib.ptr(self.state), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(nc), _lib.ptr(out),
                B, H, T, Dk, Dv, _lib.DTYPE_CODE[q.dtype], self.cur_s, None, _lib.stream_ptr(q.device))
        _lib.check(st, "cott_decode_steps")
        self.cur_s += T  # GPTCosAttention.py:269
        return out
