"""Per-rank launch and sharding glue: batch x heads split across the GPUs of one node.

Every (batch, head) pair is an independent scan (the reference launches one block column per
(n, h, d_out), ``Cuda_Kernel/combined_kernel_general.cu:104-106``), so the flattened ``B*H`` units
are cut into contiguous, balanced ranges, one per rank, and no tensor crosses GPUs.  The only
value that is summed across ranks is the gradient of ``norm_const`` (a replicated parameter: under
batch sharding several ranks hold partial sums for the same head), which rides the same
all-reduce that data-parallel training already does for every weight
(``GPT_Trainer/Trainer.py:259``).
"""
from __future__ import annotations

import torch


def shard_range(n_units: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous, balanced range of units of ``rank``: sizes differ by at most one."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad world/rank {world}/{rank}")
    base, extra = divmod(n_units, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_bh(t: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """``[B, H, N, d]`` -> this rank's units as ``[1, n_local, N, d]`` (a view when ``t`` is contiguous)."""
    B, H = t.shape[:2]
    s, e = shard_range(B * H, world, rank)
    return t.reshape(B * H, *t.shape[2:])[s:e].unsqueeze(0)


def local_norm_const(norm_const: torch.Tensor, B: int, H: int, world: int, rank: int) -> torch.Tensor:
    """Per-unit ``norm_const`` of this rank's range: unit u = b*H + h uses entry h.  The result is
    passed to the kernels as if the shard had batch 1 and ``n_local`` heads."""
    s, e = shard_range(B * H, world, rank)
    idx = torch.arange(s, e, device=norm_const.device) % H
    return norm_const.reshape(-1)[idx]


def reduce_dnorm_const(d_local: torch.Tensor, B: int, H: int, world: int, rank: int, group=None) -> torch.Tensor:
    """Per-unit gradients of this rank -> the full ``[H]`` gradient, summed over ranks when a
    process group is initialised."""
    s, e = shard_range(B * H, world, rank)
    idx = torch.arange(s, e, device=d_local.device) % H
    full = torch.zeros(H, dtype=d_local.dtype, device=d_local.device)
    full.index_add_(0, idx, d_local.reshape(-1))
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(full, op=dist.ReduceOp.SUM, group=group)
    return full


def sharded_cos_attn_causal(q, k, v, norm_const, world: int, rank: int, op=None):
    """Run the causal op on this rank's (b,h) range.  ``q, k, v`` are the FULL ``[B,H,N,d]`` tensors
    (or any tensors of that shape whose local range is valid); returns ``[1, n_local, N, d_v]``.
    ``op`` defaults to the fused CUDA operator."""
    if op is None:
        from .cos_attention import cos_attn_causal as op
    B, H = q.shape[:2]
    nc = local_norm_const(norm_const, B, H, world, rank)
    return op(shard_bh(q, world, rank), shard_bh(k, world, rank), shard_bh(v, world, rank), nc)
