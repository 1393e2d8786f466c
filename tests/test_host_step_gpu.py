"""GPU test of the host-buffer pipelined step: same results as the fused op on device tensors."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("slices,graph", [(None, False), (1, False), (2, False), (12, False), (4, True), (12, True)])
def test_host_step_matches_the_device_op(slices, graph):
    from cottention_transformer_b200 import cos_attn_causal
    from cottention_transformer_b200.host_step import CausalHostStep
    B, H, N, D = 4, 3, 700, 64
    g = torch.Generator().manual_seed(5)
    host = [torch.randn(B, H, N, D, generator=g).to(torch.bfloat16).pin_memory() for _ in range(4)]
    nc = torch.linspace(-0.3, 0.9, H)
    step = CausalHostStep(B, H, N, D, torch.bfloat16, "cuda:0", slices=slices, graph=graph)
    outs = [torch.empty(B, H, N, D, dtype=torch.bfloat16).pin_memory() for _ in range(4)]
    for rep in range(3 if graph else 2):  # the second call reuses the device buffers while nothing of the first is in flight
        for o in outs:
            o.fill_(float("nan"))
        dnc = step(*host, nc, *outs)
        torch.cuda.synchronize()
        q, k, v, do = (t.cuda() for t in host)
        q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
        ncd = nc.cuda().requires_grad_()
        ref = cos_attn_causal(q, k, v, ncd, segments=1)  # the step runs every sequence in one CTA
        ref.backward(do)
        for got, want in zip(outs, (ref.detach(), q.grad, k.grad, v.grad)):
            assert torch.equal(got, want.cpu()), rep
        assert torch.allclose(dnc.cpu(), ncd.grad.cpu(), rtol=1e-4, atol=1e-5)
    assert step.launches == (4 if graph else 2) * 3 * step.slices  # graph: one eager call before the capture


def test_host_step_rejects_pageable_and_device_tensors():
    from cottention_transformer_b200.host_step import CausalHostStep
    step = CausalHostStep(1, 1, 128, 64, torch.bfloat16, "cuda:0")
    pin = [torch.zeros(1, 1, 128, 64, dtype=torch.bfloat16).pin_memory() for _ in range(8)]
    nc = torch.zeros(1)
    bad = list(pin)
    bad[2] = torch.zeros(1, 1, 128, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="pinned"):
        step(*bad[:4], nc, *bad[4:])
    bad[2] = pin[2].cuda()
    with pytest.raises(RuntimeError, match="host tensors"):
        step(*bad[:4], nc, *bad[4:])
