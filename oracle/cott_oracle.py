"""TEST INFRASTRUCTURE ONLY -- CPU restatement of Cottention's cosine linear attention.

Nothing in the product imports this module.  It is imported by the tests, by the
smoke check and by the CPU-baseline leg of the benchmark, as the checker or as
the timed baseline -- never as the thing that is shipped.

Parity status: pinned.  ``tests/test_oracle.py`` checks every function here against
fixtures produced by executing the reference's own Python modules
(``tests/golden/make_golden.py``) and by running the reference's compiled CUDA kernel
on a B200 (``tests/golden/make_golden_gpu.py``).

All citations are paths inside the reference project.  Tensors are ``[B, H, N, D]``
(the reference's C++ names them ``N, H, S, D``).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libcott_oracle.so")
_lib = None


def build_c_oracle(force: bool = False) -> str:
    """Compile ``cott_oracle.c`` (gcc, OpenMP) next to its source."""
    src = os.path.join(_HERE, "cott_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(
            ["gcc", "-O3", "-fopenmp", "-fPIC", "-shared", "-o", _LIB_PATH, src, "-lm"]
        )
    return _LIB_PATH


def _c():
    global _lib
    if _lib is None:
        build_c_oracle()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


# ------------------------------------------------------------------------------------------------
# The scan itself: what FastAttention2.kernel.<dtype>(Q, K, V, block_size, inplace, reversed) returns
# ------------------------------------------------------------------------------------------------

def scan_recurrent(Q, K, V, reversed: bool = False, acc: str = "f64") -> torch.Tensor:
    """Token-by-token recurrence of ``Cuda_Kernel/combined_kernel_general.cu:96-170``.

    ``acc``: "f64" / "f32" accumulate in that type; "bf16" rounds every intermediate to
    bfloat16 in the reference kernel's order of operations (its bf16 mode keeps the
    state in bf16, ``:121,143``).  Runs in C (``cott_oracle.c``); O(N d^2) per head.
    """
    B, H, N, Dk = Q.shape
    Dv = V.shape[-1]
    lib = _c()
    if acc == "f64":
        q, k, v = (np.ascontiguousarray(t.detach().cpu().double().numpy()) for t in (Q, K, V))
        out = np.empty((B, H, N, Dv), dtype=np.float64)
        lib.cott_oracle_scan_f64(_ptr(q), _ptr(k), _ptr(v), _ptr(out), B, H, N, Dk, Dv, int(reversed))
    else:
        q, k, v = (np.ascontiguousarray(t.detach().cpu().float().numpy()) for t in (Q, K, V))
        out = np.empty((B, H, N, Dv), dtype=np.float32)
        fn = lib.cott_oracle_scan_f32 if acc == "f32" else lib.cott_oracle_scan_bf16_emul
        fn(_ptr(q), _ptr(k), _ptr(v), _ptr(out), B, H, N, Dk, Dv, int(reversed))
    return torch.from_numpy(out)


def scan_cumsum(Q, K, V, reversed: bool = False) -> torch.Tensor:
    """The reference's PyTorch cumsum formulation.

    Forward form ``Cuda_Kernel/speeds.py:67-76`` (``method5`` without its normalize) and the
    three gradient formulas ``Cuda_Kernel/Custom_Kernel.py:63,68,72``: the outer product
    ``V (x) K`` is cumulatively summed along the sequence (flipped for the reverse scans)
    and contracted with Q.  Materialises ``[B,H,N,Dv,Dk]``: small shapes or (b,h) slices only.
    """
    VK = V.unsqueeze(-1) * K.unsqueeze(-2)  # [B,H,N,Dv,Dk]
    if reversed:
        VK = VK.flip(2).cumsum(2).flip(2)
    else:
        VK = VK.cumsum(2)
    return (VK * Q.unsqueeze(-2)).sum(-1)


def scan_quadratic(Q, K, V, reversed: bool = False) -> torch.Tensor:
    """Masked quadratic form, ``Cuda_Kernel/speed_test.py:15-20`` (without its normalize) and the
    commented matrix forms of ``Custom_Kernel.py:61,65-67,70-71``: ``((Q K^T) * M) V`` with M
    lower-triangular (upper-triangular for the reverse scan)."""
    N = Q.shape[2]
    M = torch.tril(torch.ones(N, N, dtype=torch.bool, device=Q.device))
    if reversed:
        M = M.t()
    return (torch.matmul(Q, K.transpose(-1, -2)) * M) @ V


def scan_backward(Q, K, V, dO, scan=scan_quadratic):
    """``CustomAttention.backward``, ``Cuda_Kernel/Custom_Kernel.py:106-108``: three more scans
    with permuted arguments."""
    dQ = scan(dO, V, K, False)
    dK = scan(V, dO, Q, True)
    dV = scan(K, Q, dO, True)
    return dQ, dK, dV


# ------------------------------------------------------------------------------------------------
# Module-level math around the scan
# ------------------------------------------------------------------------------------------------

def causal_counts(keep: torch.Tensor) -> torch.Tensor:
    """``n_s`` = number of un-masked keys at positions <= s:
    ``(causal_mask * attention_mask).sum(-1)`` of ``GPT_Trainer/GPTCosAttention.py:241``.
    ``keep`` is ``[B, N]`` bool; returns ``[B, N]`` int64."""
    return keep.to(torch.int64).cumsum(-1)


def cos_attn_causal(q, k, v, norm_const, keep=None, scan=scan_quadratic):
    """Causal cosine attention as ``GPTCosAttention._cos_attn`` computes it in training
    (``GPT_Trainer/GPTCosAttention.py:229-248,282``):

      q_hat, k_hat = normalize(q), normalize(k)                       (:229-230, eps 1e-12)
      v' = v / clamp(n_s ** sigmoid(norm_const_h), min=1)              (:241)
      q_hat, k_hat, v' zeroed at masked positions                      (:245-248)
      out = scan(q_hat, k_hat, v')                                     (:282)

    ``norm_const`` is ``[H]`` (the module stores ``[1,H,1,1]``, ``:89``); ``keep`` is a
    ``[B, N]`` bool tensor of un-masked positions (``attention_mask == 0``, ``:232``) or None.
    Differentiable with torch autograd when the inputs require grad."""
    B, H, N, _ = q.shape
    qh = torch.nn.functional.normalize(q, dim=-1, p=2)
    kh = torch.nn.functional.normalize(k, dim=-1, p=2)
    if keep is None:
        keep = torch.ones(B, N, dtype=torch.bool, device=q.device)
    n = causal_counts(keep).to(q.dtype).view(B, 1, N, 1)
    sig = torch.sigmoid(norm_const).view(1, H, 1, 1)
    vp = v / (n ** sig).clamp(min=1)
    m = keep.view(B, 1, N, 1).to(q.dtype)
    return scan(qh * m, kh * m, vp * m)


def cos_attn_bidirectional(q, k, v, norm_const, keep=None):
    """Bidirectional cosine attention, ``BERT_Trainer/BertCosAttention.py:162-178,249``:
    mask q,k,v rows (:162-166), normalize (:170-171), ``v' = v / clamp(L ** sigmoid(c_h), 1)``
    with L the un-masked length (:178), ``out = q_hat (k_hat^T v')`` (:249)."""
    B, H, N, _ = q.shape
    if keep is None:
        keep = torch.ones(B, N, dtype=torch.bool, device=q.device)
    m = keep.view(B, 1, N, 1).to(q.dtype)
    q, k, v = q * m, k * m, v * m
    qh = torch.nn.functional.normalize(q, dim=-1, p=2)
    kh = torch.nn.functional.normalize(k, dim=-1, p=2)
    L = keep.sum(-1).to(q.dtype).view(B, 1, 1, 1)
    sig = torch.sigmoid(norm_const).view(1, H, 1, 1)
    vp = v / (L ** sig).clamp(min=1)
    return qh @ (kh.transpose(-1, -2) @ vp)


def decode_step(state, cur_s: int, q, k, v, norm_const):
    """One recurrent step of ``GPT_Trainer/GPTCosAttention.py:236,253-272`` for every (b,h):
    ``state`` is ``[B,H,Dv,Dk]`` float64 and is updated in place; q,k ``[B,H,Dk]``, v ``[B,H,Dv]``;
    ``cur_s`` is the 1-based position (:82).  Returns ``[B,H,Dv]`` float64."""
    B, H, Dv, Dk = state.shape
    st = state.numpy()
    assert st.dtype == np.float64 and st.flags.c_contiguous
    qq, kk, vv = (np.ascontiguousarray(t.detach().cpu().double().numpy()) for t in (q, k, v))
    nc = np.ascontiguousarray(norm_const.detach().cpu().double().numpy().reshape(-1))
    out = np.empty((B, H, Dv), dtype=np.float64)
    _c().cott_oracle_decode_step_f64(
        _ptr(st), _ptr(qq), _ptr(kk), _ptr(vv), _ptr(nc), _ptr(out), B, H, Dk, Dv, ctypes.c_long(cur_s)
    )
    return torch.from_numpy(out)


def decode_step_torch(state, cur_s: int, q, k, v, norm_const):
    """The same step written with torch ops exactly as the reference's loop body
    (``GPTCosAttention.py:229-230,236,264,267``); returns (new_state, out)."""
    qh = torch.nn.functional.normalize(q, dim=-1, p=2)
    kh = torch.nn.functional.normalize(k, dim=-1, p=2)
    H = q.shape[1]
    vp = v / (torch.tensor(float(cur_s), dtype=v.dtype) ** torch.sigmoid(norm_const).view(1, H, 1)).clamp(min=1)
    state = state + (vp.unsqueeze(-1) * kh.unsqueeze(-2)).to(torch.float64)
    out = (qh.unsqueeze(-2) * state).sum(-1)
    return state, out


# ------------------------------------------------------------------------------------------------
# Seeded synthetic inputs shared by tests, smoke and bench
# ------------------------------------------------------------------------------------------------

def make_inputs(B, H, N, Dk, Dv=None, seed=1234, normalize=True, dtype=torch.float32):
    """Q, K, V, dO ~ N(0,1) i.i.d. from a seeded CPU generator; Q and K L2-normalised along d;
    norm_const = 0.5 per head (the module's initial value, ``GPTCosAttention.py:89``)."""
    Dv = Dk if Dv is None else Dv
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, N, Dk, generator=g)
    k = torch.randn(B, H, N, Dk, generator=g)
    v = torch.randn(B, H, N, Dv, generator=g)
    do = torch.randn(B, H, N, Dv, generator=g)
    if normalize:
        q = torch.nn.functional.normalize(q, dim=-1)
        k = torch.nn.functional.normalize(k, dim=-1)
    nc = 0.5 * torch.ones(H)
    return q.to(dtype), k.to(dtype), v.to(dtype), do.to(dtype), nc
