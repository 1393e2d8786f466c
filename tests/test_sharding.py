"""CPU tests of the per-rank sharding glue, including a world_size-2 gloo run."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if REPO not in sys.path:
    sys.path.insert(0, REPO)

from cottention_transformer_b200 import sharding  # noqa: E402
from oracle import cott_oracle as O  # noqa: E402


@pytest.mark.parametrize("n,world", [(128, 1), (128, 8), (16, 8), (7, 4), (3, 8), (0, 2)])
def test_shard_ranges_partition_the_units(n, world):
    ranges = [sharding.shard_range(n, world, r) for r in range(world)]
    assert ranges[0][0] == 0 and ranges[-1][1] == n
    assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
    sizes = [e - s for s, e in ranges]
    assert max(sizes) - min(sizes) <= 1


def test_bad_rank_is_an_error():
    with pytest.raises(ValueError):
        sharding.shard_range(8, 2, 2)


def _oracle_op(q, k, v, nc):
    return O.cos_attn_causal(q, k, v, nc)


def _worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, H, N, d = 3, 3, 40, 16   # 9 units over 2 ranks: uneven split, head ranges straddle batches
        q, k, v, do, _ = O.make_inputs(B, H, N, d, seed=5)
        q, k, v, do = (t.double() for t in (q, k, v, do))
        nc = torch.tensor([0.5, -0.2, 1.0], dtype=torch.float64)
        ql, kl, vl = (sharding.shard_bh(t, world, rank).clone().requires_grad_() for t in (q, k, v))
        ncl = sharding.local_norm_const(nc, B, H, world, rank).clone().requires_grad_()
        out = _oracle_op(ql, kl, vl, ncl)
        out.backward(sharding.shard_bh(do, world, rank))
        dnc = sharding.reduce_dnorm_const(ncl.grad, B, H, world, rank)
        gathered = [None] * world
        dist.all_gather_object(gathered, (out.detach(), ql.grad, kl.grad, vl.grad))
        if rank == 0:
            full = [torch.cat([g[i] for g in gathered], 1).reshape(B, H, N, d) for i in range(4)]
            torch.save({"out": full[0], "dq": full[1], "dk": full[2], "dv": full[3], "dnc": dnc}, tmp)
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_run_equals_single_process(tmp_path):
    world, port, tmp = 2, 29500 + os.getpid() % 2000, str(tmp_path / "res.pt")
    mp.spawn(_worker, args=(world, port, tmp), nprocs=world, join=True)
    got = torch.load(tmp)
    B, H, N, d = 3, 3, 40, 16
    q, k, v, do, _ = O.make_inputs(B, H, N, d, seed=5)
    q, k, v, do = (t.double() for t in (q, k, v, do))
    nc = torch.tensor([0.5, -0.2, 1.0], dtype=torch.float64).requires_grad_()
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    out = O.cos_attn_causal(q, k, v, nc)
    out.backward(do)
    assert torch.allclose(got["out"], out.detach(), atol=1e-12)
    assert torch.allclose(got["dq"], q.grad, atol=1e-12)
    assert torch.allclose(got["dk"], k.grad, atol=1e-12)
    assert torch.allclose(got["dv"], v.grad, atol=1e-12)
    assert torch.allclose(got["dnc"], nc.grad, atol=1e-12)


def _failing_worker(rank, world, port):
    """A rank that dies before the collective: the survivor's all_reduce ends with an error
    within the process-group timeout instead of hanging."""
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    if rank == 1:
        os._exit(0)  # leaves between steps, nothing in flight
    entered = []
    real_all_reduce = dist.all_reduce

    def spy(*a, **kw):
        entered.append(True)
        return real_all_reduce(*a, **kw)

    dist.all_reduce = spy
    try:
        sharding.reduce_dnorm_const(torch.ones(4, dtype=torch.float64), 2, 4, world, rank)
    except (RuntimeError, dist.DistBackendError):
        os._exit(0 if entered else 4)  # 0: the collective was entered and ended with a distributed error
    except Exception:
        os._exit(5)  # anything else (argument, shape, import errors) is a bug, not the lost rank
    os._exit(3)  # the collective must not succeed without its peer


def test_lost_rank_surfaces_as_an_error_not_a_hang():
    ctx = mp.get_context("spawn")
    port = 31500 + os.getpid() % 2000
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, port)) for r in range(2)]
    [p.start() for p in procs]
    [p.join(timeout=60) for p in procs]
    assert all(not p.is_alive() for p in procs), "a rank hung"
    assert procs[0].exitcode == 0, f"exit code {procs[0].exitcode}: 3 = the collective succeeded, 4 = error before it, 5 = other error"
