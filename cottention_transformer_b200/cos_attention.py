"""Fused cosine attention operators (the module-level math of the reference, in one op).

``cos_attn_causal(q, k, v, norm_const)`` computes what the training branch of
``GPTCosAttention._cos_attn`` (``GPT_Trainer/GPTCosAttention.py:229-248,282``) computes:
L2-normalise q and k, divide v by ``max(n_s ** sigmoid(norm_const_h), 1)`` where ``n_s`` counts
the un-masked keys up to position s, zero the masked rows, and run the causal scan -- and it is
differentiable w.r.t. q, k, v and ``norm_const``.

Two modes, chosen by dtype (not a fallback chain -- each mode is a CUDA path of this library):

* float16 / bfloat16, head dim 64, no padding mask: ONE fused tensor-core kernel for the forward
  (``cott_cos_attn_fwd``) and two for the backward (``cott_cos_attn_bwd``), fp32 accumulation;
* float16 / bfloat16, head dim 128: the fused head-dim-128 kernels (``cott_cos_attn_wide_fwd`` / ``_bwd``);
* float16 / bfloat16, head dim 192 / 256: the row factors pulled out of the scan, tensor-core scans on
  64-wide slices of the head dimension, closed-form backward (``_WideCausal``);
* float32 / float64 (and any other shape): the reference's own structure --
  elementwise torch ops around ``CustomAttention`` (the exact-mode scan kernel), gradients of
  ``norm_const`` by autograd exactly as in the reference.
"""
from __future__ import annotations

import ctypes

import torch

from . import _binding, _lib
from .custom_kernel import CustomAttention

FUSED_DTYPES = (torch.float16, torch.bfloat16)


def fused_supported(q, k, v, keep=None) -> bool:
    return (
        q.is_cuda and q.dtype in FUSED_DTYPES and k.dtype == q.dtype and v.dtype == q.dtype
        and q.shape[-1] == 64 and v.shape[-1] == 64
        and (keep is None or tuple(keep.shape) == (q.shape[0], q.shape[2]))
    )


class _FusedCausal(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, norm_const, segments=None, keep=None, one_pass=False):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        B, H, N, D = q.shape
        ops = _binding.ops()
        if ops is not None:  # one dispatcher call: validation, allocation and the launch happen in C++
            kp = None if keep is None else keep.to(device=q.device, dtype=torch.uint8).contiguous()
            nseg = 0 if segments is None else int(segments)
            out, ws, saved = ops.causal_fwd(q, k, v, norm_const.detach(), kp, nseg, bool(one_pass))
            ctx.save_for_backward(q, k, v, norm_const.detach())
            ctx.ws, ctx.nseg, ctx.kp, ctx.saved, ctx.compiled = ws, nseg, kp, saved, True
            ctx.nc_shape, ctx.nc_dtype = norm_const.shape, norm_const.dtype
            return out
        ctx.compiled = False
        nc = norm_const.detach().reshape(-1).to(device=q.device, dtype=torch.float32).contiguous()
        if nc.numel() != H:
            raise RuntimeError(f"norm_const must have one entry per head ({H}), got {nc.numel()}")
        out = torch.empty_like(v)
        L = _lib.lib()
        with torch.cuda.device(q.device):
            # few (batch, head) pairs and a long sequence: cut every sequence into segments that run on
            # different SMs (the library says how many for this device; 1 = not worth it)
            nseg = L.cott_cos_attn_seg_count(B, H, N) if segments is None else int(segments)
            kp = None if keep is None else keep.to(device=q.device, dtype=torch.uint8).contiguous()
            saved = None
            if one_pass:  # keep the 16-bit chunk states for the one-pass backward (cott_cos_attn_bwd_train)
                saved = torch.empty(max(L.cott_cos_attn_saved_bytes(B, H, N), 16), dtype=torch.uint8, device=q.device)
                ws = torch.empty(max(L.cott_cos_attn_seg_workspace_bytes(B, H, N, nseg), 16), dtype=torch.uint8, device=q.device)
                st = L.cott_cos_attn_fwd_train(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(kp), _lib.ptr(nc), _lib.ptr(out),
                                               _lib.ptr(saved), _lib.ptr(ws), nseg, None, B, H, N, D, D, _lib.DTYPE_CODE[q.dtype],
                                               _lib.stream_ptr(q.device))
            elif nseg > 1 or kp is not None:  # the general entry point: segments and / or a padding mask
                ws = torch.empty(L.cott_cos_attn_seg_workspace_bytes(B, H, N, nseg), dtype=torch.uint8, device=q.device)
                st = L.cott_cos_attn_fwd_seg(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(kp), _lib.ptr(nc), _lib.ptr(out),
                                             _lib.ptr(ws), nseg, None, B, H, N, D, D, _lib.DTYPE_CODE[q.dtype],
                                             _lib.stream_ptr(q.device))
            else:
                ws = None
                st = L.cott_cos_attn_fwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(nc), _lib.ptr(out), B, H, N, D, D,
                                         _lib.DTYPE_CODE[q.dtype], _lib.stream_ptr(q.device))
        _lib.check(st, "cott_cos_attn_fwd")
        ctx.save_for_backward(q, k, v, nc)
        ctx.ws, ctx.nseg, ctx.kp, ctx.saved = ws, nseg, kp, saved
        ctx.nc_shape, ctx.nc_dtype = norm_const.shape, norm_const.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, nc = ctx.saved_tensors
        if ctx.compiled:
            dq, dk, dv, dnc = _binding.ops().causal_bwd(q, k, v, nc, ctx.kp, dout, ctx.ws, ctx.saved, ctx.nseg)
            return dq, dk, dv, dnc.reshape(ctx.nc_shape).to(ctx.nc_dtype), None, None, None
        dout = dout.contiguous().to(q.dtype)
        B, H, N, D = q.shape
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dnc = torch.empty(H, dtype=torch.float32, device=q.device)
        with torch.cuda.device(q.device):
            if ctx.saved is not None:
                st = _lib.lib().cott_cos_attn_bwd_train(
                    _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(ctx.kp), _lib.ptr(nc), _lib.ptr(dout), _lib.ptr(ctx.saved),
                    _lib.ptr(ctx.ws), ctx.nseg, None, _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(dnc), B, H, N, D, D,
                    _lib.DTYPE_CODE[q.dtype], _lib.stream_ptr(q.device))
            elif ctx.ws is not None:
                st = _lib.lib().cott_cos_attn_bwd_seg(
                    _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(ctx.kp), _lib.ptr(nc), _lib.ptr(dout), _lib.ptr(ctx.ws), ctx.nseg, None,
                    _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(dnc), B, H, N, D, D, _lib.DTYPE_CODE[q.dtype],
                    _lib.stream_ptr(q.device))
            else:
                st = _lib.lib().cott_cos_attn_bwd(
                    _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(nc), _lib.ptr(dout), _lib.ptr(dq), _lib.ptr(dk),
                    _lib.ptr(dv), _lib.ptr(dnc), B, H, N, D, D, _lib.DTYPE_CODE[q.dtype], _lib.stream_ptr(q.device))
        _lib.check(st, "cott_cos_attn_bwd")
        return dq, dk, dv, dnc.reshape(ctx.nc_shape).to(ctx.nc_dtype), None, None, None


class _FusedCausalPacked(torch.autograd.Function):
    """The fused causal op on the packed output of a QKV projection: ``qkv`` is ``[B, N, 3, H, 64]`` and the result
    ``[B, N, H, 64]``; q, k, v, the output and all gradients are read and written in place through strided tensor
    maps, so the head split / merge permutes (GPTCosAttention.py:447-449,478-479,500) cost no copy."""

    @staticmethod
    def forward(ctx, qkv, norm_const, keep=None, sin=None, cos=None):
        qkv = qkv.contiguous()
        B, N, three, H, D = qkv.shape
        nc = norm_const.detach().reshape(-1).to(device=qkv.device, dtype=torch.float32).contiguous()
        out = torch.empty(B, N, H, D, dtype=qkv.dtype, device=qkv.device)
        lay = _lib.CottLayout(N * 3 * H * D, D, 3 * H * D, N * H * D, D, H * D)
        L = _lib.lib()
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        kp = None if keep is None else keep.to(device=qkv.device, dtype=torch.uint8).contiguous()
        rot = None
        if sin is not None:  # the rotary embedding of q, k inside the kernels (one segment per sequence)
            per_batch = sin.dim() == 3 and sin.shape[0] > 1
            rot = _lib.CottRotaryTables(_lib.ptr(sin), _lib.ptr(cos), 2 * sin.shape[-1], N * sin.shape[-1] if per_batch else 0)
        with torch.cuda.device(qkv.device):
            nseg = 1 if rot is not None else L.cott_cos_attn_seg_count(B, H, N)
            ws = torch.empty(L.cott_cos_attn_seg_workspace_bytes(B, H, N, nseg), dtype=torch.uint8, device=qkv.device)
            if rot is not None:
                st = L.cott_cos_attn_fwd_rotary(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(kp), _lib.ptr(nc), _lib.ptr(out),
                                                _lib.ptr(ws), ctypes.byref(lay), ctypes.byref(rot), B, H, N, D, D,
                                                _lib.DTYPE_CODE[qkv.dtype], _lib.stream_ptr(qkv.device))
            else:
                st = L.cott_cos_attn_fwd_seg(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(kp), _lib.ptr(nc), _lib.ptr(out),
                                             _lib.ptr(ws), nseg, ctypes.byref(lay), B, H, N, D, D, _lib.DTYPE_CODE[qkv.dtype],
                                             _lib.stream_ptr(qkv.device))
        _lib.check(st, "cott_cos_attn_fwd_rotary" if rot is not None else "cott_cos_attn_fwd_seg")
        ctx.save_for_backward(qkv, nc, sin, cos)
        ctx.ws, ctx.nseg, ctx.kp, ctx.lay, ctx.rot = ws, nseg, kp, lay, rot
        ctx.nc_shape, ctx.nc_dtype = norm_const.shape, norm_const.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, nc, sin, cos = ctx.saved_tensors
        B, N, three, H, D = qkv.shape
        dout = dout.contiguous().to(qkv.dtype)
        dqkv = torch.empty_like(qkv)
        dnc = torch.empty(H, dtype=torch.float32, device=qkv.device)
        L = _lib.lib()
        with torch.cuda.device(qkv.device):
            if ctx.rot is not None:
                st = L.cott_cos_attn_bwd_rotary(
                    _lib.ptr(qkv[:, :, 0]), _lib.ptr(qkv[:, :, 1]), _lib.ptr(qkv[:, :, 2]), _lib.ptr(ctx.kp), _lib.ptr(nc),
                    _lib.ptr(dout), _lib.ptr(ctx.ws), ctypes.byref(ctx.lay), ctypes.byref(ctx.rot), _lib.ptr(dqkv[:, :, 0]),
                    _lib.ptr(dqkv[:, :, 1]), _lib.ptr(dqkv[:, :, 2]), _lib.ptr(dnc), B, H, N, D, D, _lib.DTYPE_CODE[qkv.dtype],
                    _lib.stream_ptr(qkv.device))
            else:
                st = L.cott_cos_attn_bwd_seg(
                    _lib.ptr(qkv[:, :, 0]), _lib.ptr(qkv[:, :, 1]), _lib.ptr(qkv[:, :, 2]), _lib.ptr(ctx.kp), _lib.ptr(nc),
                    _lib.ptr(dout), _lib.ptr(ctx.ws), ctx.nseg, ctypes.byref(ctx.lay), _lib.ptr(dqkv[:, :, 0]),
                    _lib.ptr(dqkv[:, :, 1]), _lib.ptr(dqkv[:, :, 2]), _lib.ptr(dnc), B, H, N, D, D, _lib.DTYPE_CODE[qkv.dtype],
                    _lib.stream_ptr(qkv.device))
        _lib.check(st, "cott_cos_attn_bwd_rotary" if ctx.rot is not None else "cott_cos_attn_bwd_seg")
        return dqkv, dnc.reshape(ctx.nc_shape).to(ctx.nc_dtype), None, None, None


def cos_attn_causal_packed(qkv, norm_const, keep=None, rotary=None):
    """Causal cosine attention on a packed ``[B, N, 3, H, 64]`` bf16 / fp16 tensor (the reshaped output of one QKV
    projection); returns ``[B, N, H, 64]`` (reshape to ``[B, N, H*64]`` for the output projection).  Same function
    as ``cos_attn_causal`` on the permuted tensors, without the permute copies in either direction.

    ``rotary=(sin, cos)`` -- fp32 ``[N, rot/2]`` or ``[B, N, rot/2]``, the two halves of the module's
    ``embed_positions`` gathered at ``position_ids`` (GPTCosAttention.py:458-476) -- applies the rotary embedding to
    q and k **inside the kernels** (their tiles are rotated in shared memory, dq and dk are rotated back on the way
    out): the same bits as ``rotary_packed_`` followed by this op, without that op's passes over q, k, dq, dk, and
    ``qkv`` itself is left as the projection wrote it.  The rotary dim must be a multiple of 16; sequences that this
    op would cut into segments (few heads, very long N) take the separate rotary pass instead."""
    if not qkv.is_cuda:
        raise RuntimeError("cos_attn_causal_packed needs a CUDA tensor (there is no CPU path)")
    if qkv.dim() != 5 or qkv.shape[2] != 3 or qkv.shape[-1] != 64 or qkv.dtype not in FUSED_DTYPES:
        raise RuntimeError("cos_attn_causal_packed takes a [B, N, 3, H, 64] bfloat16 / float16 tensor")
    if rotary is None:
        return _FusedCausalPacked.apply(qkv, norm_const, keep)
    sin, cos = rotary
    sin = sin.to(device=qkv.device, dtype=torch.float32).contiguous()
    cos = cos.to(device=qkv.device, dtype=torch.float32).contiguous()
    B, N, _, H, _ = qkv.shape
    if sin.shape != cos.shape or sin.shape[-2] != N or (sin.dim() == 3 and sin.shape[0] not in (1, B)):
        raise RuntimeError("sin / cos must be [N, rot/2] or [B, N, rot/2]")
    with torch.cuda.device(qkv.device):
        one_segment = _lib.lib().cott_cos_attn_seg_count(B, H, N) == 1
    if (2 * sin.shape[-1]) % 16 or not one_segment:
        return _FusedCausalPacked.apply(rotary_packed_(qkv.contiguous(), sin, cos), norm_const, keep)
    return _FusedCausalPacked.apply(qkv, norm_const, keep, sin, cos)


class _RotaryPacked(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, sin, cos, H, inverse=False):
        B, N = x.shape[0], x.shape[1]
        D = x.numel() // (B * N * 3 * H)
        qkv = x.view(B, N, 3, H, D)
        rot = 2 * sin.shape[-1]
        lay = _lib.CottLayout(N * 3 * H * D, D, 3 * H * D, 0, 0, 0)
        per_batch = sin.dim() == 3 and sin.shape[0] > 1
        with torch.cuda.device(qkv.device):
            st = _lib.lib().cott_rotary(_lib.ptr(qkv[:, :, 0]), _lib.ptr(qkv[:, :, 1]), _lib.ptr(sin), _lib.ptr(cos),
                                        ctypes.byref(lay), B, H, N, D, rot, N * (rot // 2) if per_batch else 0, int(inverse),
                                        _lib.DTYPE_CODE[qkv.dtype], _lib.stream_ptr(qkv.device))
        _lib.check(st, "cott_rotary")
        ctx.save_for_backward(sin, cos)
        ctx.inverse, ctx.H = inverse, H
        ctx.mark_dirty(x)
        return x

    @staticmethod
    def backward(ctx, g):
        sin, cos = ctx.saved_tensors
        # a private copy: autograd may hand the same gradient tensor to other consumers (both operands of an add,
        # retain_grad, hooks), and the rotation below is in place
        g = g.clone(memory_format=torch.contiguous_format)
        return _RotaryPacked.apply(g, sin, cos, ctx.H, not ctx.inverse), None, None, None, None


def rotary_packed_(qkv, sin, cos, heads=None):
    """GPT-J rotary embedding (GPTCosAttention.py:458-476; transformers ``apply_rotary_pos_emb``) applied IN PLACE
    to the q and k slices of a packed ``[B, N, 3, H, d]`` bf16 / fp16 tensor, one read and one write of q and k.
    The tensor may also be given as the projection output itself, ``[B, N, 3*H*d]`` with ``heads=H`` (an in-place
    op on a view costs autograd extra copies of the gradient; on the projection output it does not).
    ``sin``, ``cos``: fp32 ``[N, rot/2]`` or ``[B, N, rot/2]`` (the two halves of ``embed_positions`` gathered at
    ``position_ids``); the first ``rot`` elements of every head are rotated.  Differentiable (the backward is the
    transposed rotation of the gradient, in place)."""
    ok = qkv.is_cuda and qkv.dtype in FUSED_DTYPES and qkv.is_contiguous()
    if ok and qkv.dim() == 5 and qkv.shape[2] == 3:
        heads = qkv.shape[3]
    elif not (ok and qkv.dim() == 3 and heads and qkv.shape[2] % (3 * heads * 8) == 0):
        raise RuntimeError("rotary_packed_ takes a contiguous [B, N, 3, H, d] (or [B, N, 3*H*d] with heads=H) "
                           "bfloat16 / float16 CUDA tensor")
    sin = sin.to(device=qkv.device, dtype=torch.float32).contiguous()
    cos = cos.to(device=qkv.device, dtype=torch.float32).contiguous()
    if sin.shape != cos.shape or sin.shape[-2] != qkv.shape[1] or (sin.dim() == 3 and sin.shape[0] not in (1, qkv.shape[0])):
        raise RuntimeError("sin / cos must be [N, rot/2] or [B, N, rot/2]")
    return _RotaryPacked.apply(qkv, sin, cos, heads)


class _FusedWide128(torch.autograd.Function):
    """Head dim 128 in bf16 / fp16: ``cott_cos_attn_wide_fwd`` / ``_bwd`` -- one tensor-core pass forward (row norms,
    length factor and output scaling inside the kernel), and a row-dot pass plus three tensor-core passes backward with
    the normalisation terms in their epilogues.  The forward's row factors travel to the backward in ``ws``."""

    @staticmethod
    def forward(ctx, q, k, v, norm_const, keep):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        B, H, N, D = q.shape
        L = _lib.lib()
        nc = norm_const.detach().reshape(-1).to(device=q.device, dtype=torch.float32).contiguous()
        if nc.numel() != H:
            raise RuntimeError(f"norm_const must have one entry per head ({H}), got {nc.numel()}")
        kp = None if keep is None else keep.to(device=q.device, dtype=torch.uint8).contiguous()
        out = torch.empty_like(v)
        with torch.cuda.device(q.device):
            ws = torch.empty(max(L.cott_cos_attn_wide_workspace_bytes(B, H, N), 16), dtype=torch.uint8, device=q.device)
            st = L.cott_cos_attn_wide_fwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(kp), _lib.ptr(nc), _lib.ptr(out),
                                          _lib.ptr(ws), B, H, N, D, D, _lib.DTYPE_CODE[q.dtype], _lib.stream_ptr(q.device))
        _lib.check(st, "cott_cos_attn_wide_fwd")
        ctx.save_for_backward(q, k, v, out, nc, ws)
        ctx.kp = kp
        ctx.nc_shape, ctx.nc_dtype = norm_const.shape, norm_const.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, nc, ws = ctx.saved_tensors
        B, H, N, D = q.shape
        dout = dout.contiguous().to(q.dtype)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dnc = torch.empty(H, dtype=torch.float32, device=q.device)
        with torch.cuda.device(q.device):
            st = _lib.lib().cott_cos_attn_wide_bwd(
                _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(ctx.kp), _lib.ptr(nc), _lib.ptr(out), _lib.ptr(dout), _lib.ptr(ws),
                _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(dnc), B, H, N, D, D, _lib.DTYPE_CODE[q.dtype],
                _lib.stream_ptr(q.device))
        _lib.check(st, "cott_cos_attn_wide_bwd")
        return dq, dk, dv, dnc.reshape(ctx.nc_shape).to(ctx.nc_dtype), None


def wide_supported(q, k, v, keep=None) -> bool:
    return (
        q.is_cuda and q.dtype in FUSED_DTYPES and k.dtype == q.dtype and v.dtype == q.dtype
        and q.shape[-1] in (128, 192, 256) and v.shape[-1] == q.shape[-1]
        and (keep is None or tuple(keep.shape) == (q.shape[0], q.shape[2]))
    )


class _WideCausal(torch.autograd.Function):
    """Head dims 128 / 192 / 256 in bf16 / fp16.  The row factors are pulled out of the scan,

        out_t = r_t * scan(q, k, w v)_t      r_t = keep_t / |q_t|      w_s = keep_s / (|k_s| max(n_s^sigma, 1))

    so q and k go into the tensor-core scans as they are, the factors stay in fp32 ``[B, H, N, 1]`` and the
    backward is three more scans plus the derivatives of r and w in closed form (GPTCosAttention.py:229-248 by
    the chain rule) -- a handful of elementwise passes instead of autograd through normalize / pow / div."""

    @staticmethod
    def forward(ctx, q, k, v, norm_const, keep):
        from .kernel import scan
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        B, H, N, D = q.shape
        f32 = torch.float32
        sig = torch.sigmoid(norm_const.detach().reshape(1, H, 1, 1).to(device=q.device, dtype=f32))
        if keep is None:
            n = torch.arange(1, N + 1, device=q.device, dtype=f32).view(1, 1, N, 1)
            m = None
        else:
            m = keep.to(device=q.device, dtype=f32).view(B, 1, N, 1)
            n = m.cumsum(2).clamp(min=1)
        a = 1.0 / (n ** sig).clamp(min=1)                                                       # [B|1, H, N, 1]
        rq = 1.0 / torch.linalg.vector_norm(q, dim=-1, keepdim=True, dtype=f32).clamp(min=1e-12)  # F.normalize eps
        rk = 1.0 / torch.linalg.vector_norm(k, dim=-1, keepdim=True, dtype=f32).clamp(min=1e-12)
        if m is not None:
            rq, rk = rq * m, rk * m
        w = a * rk
        vw = (v * w).to(q.dtype)
        out = scan(q, k, vw, False)
        out.mul_(rq)
        ctx.save_for_backward(q, k, v, vw, out, rq, rk, w, n, sig)
        ctx.nc_shape, ctx.nc_dtype = norm_const.shape, norm_const.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        from .kernel import scan
        q, k, v, vw, out, rq, rk, w, n, sig = ctx.saved_tensors
        f32 = torch.float32
        dout = dout.contiguous().to(q.dtype)
        d_r = (dout * out).sum(-1, keepdim=True, dtype=f32)        # = r_t (dO_t . scan_t)
        g = (dout * rq).to(q.dtype)
        dq = scan(g, vw, k, False)                                  # Custom_Kernel.py:106
        dk = scan(vw, g, q, True)                                   # :107
        dvw = scan(k, q, g, True)                                   # :108
        dw = (dvw * v).sum(-1, keepdim=True, dtype=f32)
        dq.addcmul_(q, (-(d_r * rq * rq)).to(q.dtype))              # d r / d q = -q r^3, and d_r carries one r
        dk.addcmul_(k, (-(dw * w * rk * rk)).to(q.dtype))           # d w / d k = -k w rk^2
        dv = dvw.mul_(w)
        # d w / d sigma = -ln(n) w where n^sigma > 1
        dsig = -(torch.log(n) * (n > 1) * dw * w).sum(dim=(0, 2, 3))
        s1 = sig.reshape(-1)
        dnc = (dsig * s1 * (1 - s1)).reshape(ctx.nc_shape).to(ctx.nc_dtype)
        return dq, dk, dv, dnc, None


def _exact_causal(q, k, v, norm_const, keep):
    """The reference's structure (GPTCosAttention.py:229-248,282) around the exact-mode scan."""
    B, H, N, _ = q.shape
    qh = torch.nn.functional.normalize(q, dim=-1, p=2)
    kh = torch.nn.functional.normalize(k, dim=-1, p=2)
    if keep is None:
        n = torch.arange(1, N + 1, device=q.device, dtype=q.dtype).view(1, 1, N, 1)
    else:
        n = keep.to(torch.int64).cumsum(-1).to(q.dtype).view(B, 1, N, 1)
    sig = torch.sigmoid(norm_const).reshape(1, H, 1, 1).to(q.dtype)
    vp = v / (n ** sig).clamp(min=1)
    if keep is not None:
        m = keep.view(B, 1, N, 1).to(q.dtype)
        qh, kh, vp = qh * m, kh * m, vp * m
    return CustomAttention.apply(qh, kh, vp)


def cos_attn_causal(q, k, v, norm_const, keep=None, segments=None, one_pass_backward=False):
    """Causal cosine attention with the learned length-norm.

    q, k, v: ``[B, H, N, d]`` CUDA tensors; ``norm_const``: H values (any shape, e.g. the module's
    ``[1, H, 1, 1]`` parameter); ``keep``: optional ``[B, N]`` bool, True = un-masked
    (``attention_mask == 0`` in the reference, ``GPTCosAttention.py:232``).
    ``segments``: how many segments each sequence is cut into on the fused path (they run on different SMs;
    same results); ``None`` lets the library choose -- more than one only for few (batch, head) pairs.
    ``one_pass_backward`` (fused path only): the forward also keeps its 16-bit chunk states (half the size of q) and
    the backward is one kernel that reads every tensor once (``cott_cos_attn_fwd_train`` / ``_bwd_train``) instead
    of two kernels that each read all four: 7.5 instead of 11 tensor passes of HBM traffic at about the same run
    time on an otherwise idle B200.
    """
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise RuntimeError("cos_attn_causal needs CUDA tensors (there is no CPU path)")
    if fused_supported(q, k, v, keep):
        return _FusedCausal.apply(q, k, v, norm_const, segments, keep, bool(one_pass_backward))
    if wide_supported(q, k, v, keep):
        if q.shape[-1] == 128:
            return _FusedWide128.apply(q, k, v, norm_const, keep)
        return _WideCausal.apply(q, k, v, norm_const, keep)
    return _exact_causal(q, k, v, norm_const, keep)


class _Bidirectional(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, norm_const, keep):
        q, k, v = q.contiguous(), k.to(q.dtype).contiguous(), v.to(q.dtype).contiguous()
        B, H, N, Dk = q.shape
        Dv = v.shape[-1]
        ops = _binding.ops()
        ctx.compiled = ops is not None
        if ops is not None:
            kp = None if keep is None else keep.to(device=q.device, dtype=torch.uint8).contiguous()
            out, scratch = ops.bidir_fwd(q, k, v, norm_const.detach(), kp)
            ctx.save_for_backward(q, k, v, norm_const.detach(), scratch)
            ctx.kp = kp
            ctx.nc_shape, ctx.nc_dtype = norm_const.shape, norm_const.dtype
            return out
        L = _lib.lib()
        code = _lib.DTYPE_CODE[q.dtype]
        nc = norm_const.detach().reshape(-1).to(device=q.device, dtype=torch.float32).contiguous()
        kp = None if keep is None else keep.to(device=q.device, dtype=torch.uint8).contiguous()
        nbytes = L.cott_bidir_scratch_bytes(B, H, N, Dk, Dv, code)
        scratch = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=q.device)
        out = torch.empty(B, H, N, Dv, dtype=q.dtype, device=q.device)
        with torch.cuda.device(q.device):
            st = L.cott_bidir_fwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(kp), _lib.ptr(nc), _lib.ptr(out),
                                  _lib.ptr(scratch), B, H, N, Dk, Dv, code, _lib.stream_ptr(q.device))
        _lib.check(st, "cott_bidir_fwd")
        ctx.save_for_backward(q, k, v, nc, scratch)
        ctx.kp = kp
        ctx.nc_shape, ctx.nc_dtype = norm_const.shape, norm_const.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, nc, scratch = ctx.saved_tensors
        kp = ctx.kp
        if ctx.compiled:
            dq, dk, dv, dnc = _binding.ops().bidir_bwd(q, k, v, nc, kp, dout, scratch)
            return dq, dk, dv, dnc.reshape(ctx.nc_shape).to(ctx.nc_dtype), None
        B, H, N, Dk = q.shape
        Dv = v.shape[-1]
        dout = dout.contiguous().to(q.dtype)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dnc = torch.empty(H, dtype=torch.float32, device=q.device)
        scratch2 = torch.empty_like(scratch)
        with torch.cuda.device(q.device):
            st = _lib.lib().cott_bidir_bwd(
                _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(kp), _lib.ptr(nc), _lib.ptr(dout), _lib.ptr(scratch),
                _lib.ptr(scratch2), _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(dnc), B, H, N, Dk, Dv,
                _lib.DTYPE_CODE[q.dtype], _lib.stream_ptr(q.device))
        _lib.check(st, "cott_bidir_bwd")
        return dq, dk, dv, dnc.reshape(ctx.nc_shape).to(ctx.nc_dtype), None


class _BidirectionalPacked(torch.autograd.Function):
    """Bidirectional op on a packed ``[B, N, 3, H, 64]`` tensor; see ``_FusedCausalPacked``."""

    @staticmethod
    def forward(ctx, qkv, norm_const, keep=None):
        qkv = qkv.contiguous()
        B, N, three, H, D = qkv.shape
        nc = norm_const.detach().reshape(-1).to(device=qkv.device, dtype=torch.float32).contiguous()
        out = torch.empty(B, N, H, D, dtype=qkv.dtype, device=qkv.device)
        lay = _lib.CottLayout(N * 3 * H * D, D, 3 * H * D, N * H * D, D, H * D)
        kp = None if keep is None else keep.to(device=qkv.device, dtype=torch.uint8).contiguous()
        with torch.cuda.device(qkv.device):
            st = _lib.lib().cott_bidir_fwd_strided(
                _lib.ptr(qkv[:, :, 0]), _lib.ptr(qkv[:, :, 1]), _lib.ptr(qkv[:, :, 2]), _lib.ptr(kp), _lib.ptr(nc), _lib.ptr(out),
                ctypes.byref(lay), B, H, N, D, D, _lib.DTYPE_CODE[qkv.dtype], _lib.stream_ptr(qkv.device))
        _lib.check(st, "cott_bidir_fwd_strided")
        ctx.save_for_backward(qkv, nc)
        ctx.kp, ctx.lay = kp, lay
        ctx.nc_shape, ctx.nc_dtype = norm_const.shape, norm_const.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, nc = ctx.saved_tensors
        B, N, three, H, D = qkv.shape
        dout = dout.contiguous().to(qkv.dtype)
        dqkv = torch.empty_like(qkv)
        dnc = torch.empty(H, dtype=torch.float32, device=qkv.device)
        with torch.cuda.device(qkv.device):
            st = _lib.lib().cott_bidir_bwd_strided(
                _lib.ptr(qkv[:, :, 0]), _lib.ptr(qkv[:, :, 1]), _lib.ptr(qkv[:, :, 2]), _lib.ptr(ctx.kp), _lib.ptr(nc),
                _lib.ptr(dout), ctypes.byref(ctx.lay), _lib.ptr(dqkv[:, :, 0]), _lib.ptr(dqkv[:, :, 1]), _lib.ptr(dqkv[:, :, 2]),
                _lib.ptr(dnc), B, H, N, D, D, _lib.DTYPE_CODE[qkv.dtype], _lib.stream_ptr(qkv.device))
        _lib.check(st, "cott_bidir_bwd_strided")
        return dqkv, dnc.reshape(ctx.nc_shape).to(ctx.nc_dtype), None


def cos_attn_bidirectional_packed(qkv, norm_const, keep=None):
    """Bidirectional cosine attention on a packed ``[B, N, 3, H, 64]`` bf16 / fp16 tensor; returns ``[B, N, H, 64]``.
    Same function as ``cos_attn_bidirectional`` on the permuted tensors, without the permute copies."""
    if not qkv.is_cuda:
        raise RuntimeError("cos_attn_bidirectional_packed needs a CUDA tensor (there is no CPU path)")
    if qkv.dim() != 5 or qkv.shape[2] != 3 or qkv.shape[-1] != 64 or qkv.dtype not in FUSED_DTYPES:
        raise RuntimeError("cos_attn_bidirectional_packed takes a [B, N, 3, H, 64] bfloat16 / float16 tensor")
    return _BidirectionalPacked.apply(qkv, norm_const, keep)


def cos_attn_bidirectional(q, k, v, norm_const, keep=None):
    """Bidirectional cosine attention with the learned length-norm, the cosine section of the
    reference's ``BertCosAttention.forward`` (``BERT_Trainer/BertCosAttention.py:162-178,249``).

    q, k: ``[B, H, N, d_k]``; v: ``[B, H, N, d_v]``; ``norm_const``: H values (e.g. the module's
    ``[1, H, 1, 1]`` parameter, ``:81``); ``keep``: optional ``[B, N]`` bool, True = un-masked
    (``attention_mask == 0``, ``:163``).  Differentiable w.r.t. q, k, v and ``norm_const``."""
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise RuntimeError("cos_attn_bidirectional needs CUDA tensors (there is no CPU path)")
    if q.dtype not in _lib.DTYPE_CODE:
        raise ValueError("Only float32, float64, float16, and bfloat16 are supported")
    return _Bidirectional.apply(q, k, v, norm_const, keep)
