"""Seeded synthetic inputs of the benchmark and of the examples.

The reference trains on tokenised text (the Pile, Wikipedia + BookCorpus); none of that is available offline, so
the measurements run on tensors with the shapes and value distributions its attention op sees:
Q, K, V, dO ~ N(0, 1) i.i.d. from a seeded CPU generator, Q and K L2-normalised along the head dimension
(what ``F.normalize`` leaves, GPT_Trainer/GPTCosAttention.py:229-230), ``norm_const`` = 0.5 per head (the module's
initial value, :89).  The same seed gives the same tensors on every machine and for every GPU count.
"""
from __future__ import annotations

import torch


def make_inputs(B, H, N, Dk, Dv=None, seed=1234, normalize=True, dtype=torch.float32):
    """Returns (q, k, v, dout, norm_const) on the CPU: q, k ``[B,H,N,Dk]``, v, dout ``[B,H,N,Dv]``, norm_const ``[H]``."""
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
