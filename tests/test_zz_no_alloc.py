"""GPU test of cott_bidir_fwd_static, the entry point for hosts that may not allocate device memory
once they are running (frozen memory pools, loops that cannot take cudaMalloc's device-wide stall).

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.  It calls the entry point straight through the C ABI and checks it against
cott_bidir_fwd (which gets its scratch from the caller) on two calls in a row -- the second with
different data and a smaller problem, so leftovers of the first call in the shared built-in scratch
would show.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

STATIC_BYTES = 8 << 20  # COTT_BIDIR_STATIC_SCRATCH_BYTES in include/cottention_b200.h


def _both(L, _lib, q, k, v, keep, nc):
    B, H, N, Dk = q.shape
    Dv = v.shape[-1]
    code = _lib.DTYPE_CODE[q.dtype]
    kp = None if keep is None else keep.to(torch.uint8).contiguous()
    stream = _lib.stream_ptr(q.device)
    want = torch.empty(B, H, N, Dv, dtype=q.dtype, device=q.device)
    scratch = torch.empty(max(L.cott_bidir_scratch_bytes(B, H, N, Dk, Dv, code), 1), dtype=torch.uint8, device=q.device)
    _lib.check(L.cott_bidir_fwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(kp), _lib.ptr(nc), _lib.ptr(want),
                                _lib.ptr(scratch), B, H, N, Dk, Dv, code, stream), "cott_bidir_fwd")
    got = torch.full_like(want, float("nan"))
    _lib.check(L.cott_bidir_fwd_static(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(kp), _lib.ptr(nc),
                                       _lib.ptr(got), B, H, N, Dk, Dv, code, stream), "cott_bidir_fwd_static")
    torch.cuda.synchronize()
    return got, want


def test_static_scratch_entry_point_matches_the_allocating_one_twice_in_a_row():
    from cottention_transformer_b200 import _lib
    L = _lib.lib()
    g = torch.Generator(device="cuda").manual_seed(77)
    cases = [((4, 12, 512, 64), torch.float32, 2e-4, True), ((2, 3, 200, 32), torch.bfloat16, 2e-2, True),
             ((2, 2, 150, 48), torch.float64, 1e-10, False),      # 8-byte accumulators, no padding mask
             ((3, 4, 300, 64), torch.bfloat16, 2e-2, True)]       # 16-bit, head dim 64: the on-chip (tensor-core) kernel
    for (B, H, N, d), dt, tol, masked in cases:
        q = torch.randn(B, H, N, d, device="cuda", generator=g).to(dt)
        k = torch.randn(B, H, N, d, device="cuda", generator=g).to(dt)
        v = torch.randn(B, H, N, d, device="cuda", generator=g).to(dt)
        keep = None
        if masked:
            keep = torch.ones(B, N, dtype=torch.bool, device="cuda")
            keep[0, N // 2:] = False
        nc = torch.linspace(-0.5, 1.0, H, device="cuda")
        got, want = _both(L, _lib, q, k, v, keep, nc)
        assert torch.isfinite(got).all()
        err = (got.double() - want.double()).abs().max().item()
        assert err <= tol * max(want.abs().max().item(), 1.0), err


def test_problem_larger_than_the_built_in_scratch_is_refused_with_both_sizes_named():
    from cottention_transformer_b200 import _lib
    L = _lib.lib()
    B, H, N, d = 64, 16, 512, 64   # 1024 (b,h) states of 16 KiB = 16 MiB > 8 MiB
    assert L.cott_bidir_scratch_bytes(B, H, N, d, d, 0) > STATIC_BYTES
    x = torch.zeros(1, device="cuda")
    st = L.cott_bidir_fwd_static(x.data_ptr(), x.data_ptr(), x.data_ptr(), None, x.data_ptr(), x.data_ptr(),
                                 B, H, N, d, d, 0, None)
    assert st == 2
    msg = L.cott_last_error().decode()
    assert str(STATIC_BYTES) in msg and "cott_bidir_fwd" in msg


@pytest.mark.parametrize("dt,d", [(torch.float32, 64), (torch.bfloat16, 64)])
def test_the_call_leaves_device_memory_in_use_unchanged(dt, d):
    """The property the entry point exists for: after one warm-up call (which looks up the built-in array's
    address and loads the kernels) a further call changes neither the free memory the driver reports nor the
    number of allocations torch's caching allocator has made."""
    from cottention_transformer_b200 import _lib
    L = _lib.lib()
    B, H, N = 4, 12, 512
    g = torch.Generator(device="cuda").manual_seed(3)
    q, k, v = (torch.randn(B, H, N, d, device="cuda", generator=g).to(dt) for _ in range(3))
    nc = torch.zeros(H, device="cuda")
    out = torch.empty_like(v)
    code, stream = _lib.DTYPE_CODE[dt], _lib.stream_ptr(q.device)

    def call():
        _lib.check(L.cott_bidir_fwd_static(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), None, _lib.ptr(nc), _lib.ptr(out),
                                           B, H, N, d, d, code, stream), "cott_bidir_fwd_static")
        torch.cuda.synchronize()

    call()
    free0 = torch.cuda.mem_get_info()[0]
    stats0 = torch.cuda.memory_stats()
    for _ in range(3):
        call()
    stats1 = torch.cuda.memory_stats()
    assert torch.cuda.mem_get_info()[0] == free0
    assert stats1["allocation.all.allocated"] == stats0["allocation.all.allocated"]
    assert stats1["segment.all.allocated"] == stats0["segment.all.allocated"]
