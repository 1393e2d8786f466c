"""CPU tests: the oracle against the fixtures produced by executing the reference."""
import os

import numpy as np
import pytest
import torch

from oracle import cott_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _load(name):
    path = os.path.join(GOLDEN, name)
    if not os.path.exists(path):
        pytest.skip(f"fixture {name} not generated yet")
    return {k: v for k, v in np.load(path).items()}


def _t(a):
    return torch.from_numpy(np.asarray(a)).double()


def test_scan_forms_agree():
    q, k, v, do, _ = O.make_inputs(2, 2, 77, 32, 48, seed=7)
    q, k, v = q.double(), k.double(), v.double()
    for rev in (False, True):
        a = O.scan_cumsum(q, k, v, rev)
        b = O.scan_quadratic(q, k, v, rev)
        c = O.scan_recurrent(q, k, v, rev, "f64")
        d = O.scan_recurrent(q, k, v, rev, "f32").double()
        assert torch.allclose(a, b, atol=1e-12)
        assert torch.allclose(a, c, atol=1e-12)
        assert torch.allclose(a, d, atol=1e-4)


def test_scan_backward_is_autograd_of_forward():
    q, k, v, do, _ = O.make_inputs(1, 2, 40, 32, 32, seed=8)
    q, k, v, do = (t.double() for t in (q, k, v, do))
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    (O.scan_quadratic(q, k, v) * do).sum().backward()
    dq, dk, dv = O.scan_backward(q.detach(), k.detach(), v.detach(), do)
    assert torch.allclose(dq, q.grad, atol=1e-12)
    assert torch.allclose(dk, k.grad, atol=1e-12)
    assert torch.allclose(dv, v.grad, atol=1e-12)
    dq2, dk2, dv2 = O.scan_backward(q.detach(), k.detach(), v.detach(), do,
                                    scan=lambda a, b, c, r: O.scan_recurrent(a, b, c, r, "f64"))
    assert torch.allclose(dq2, q.grad, atol=1e-11)
    assert torch.allclose(dk2, k.grad, atol=1e-11)
    assert torch.allclose(dv2, v.grad, atol=1e-11)


def test_bf16_emulation_is_close_to_truth_but_not_equal():
    q, k, v, _, _ = O.make_inputs(1, 1, 256, 64, 64, seed=9, dtype=torch.bfloat16)
    truth = O.scan_recurrent(q, k, v, False, "f64")
    emu = O.scan_recurrent(q.float(), k.float(), v.float(), False, "bf16").double()
    rel = (emu - truth).norm() / truth.norm()
    assert 1e-4 < rel < 0.2


@pytest.mark.parametrize("scan", ["quadratic", "recurrent"])
def test_gpt_train_branch_golden(scan):
    g = _load("gpt_cos_attn_train_branch.npz")
    q, k, v, do = (_t(g[n]) for n in ("q", "k", "v", "dout"))
    nc = _t(g["norm_const"]).requires_grad_()
    keep = torch.from_numpy(g["keep"])
    if scan == "quadratic":
        q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
        out = O.cos_attn_causal(q, k, v, nc, keep)
        (out * do).sum().backward()
        assert torch.allclose(q.grad, _t(g["dq"]), atol=1e-10)
        assert torch.allclose(k.grad, _t(g["dk"]), atol=1e-10)
        assert torch.allclose(v.grad, _t(g["dv"]), atol=1e-10)
        assert torch.allclose(nc.grad, _t(g["dnorm_const"]), atol=1e-10)
    else:
        out = O.cos_attn_causal(q, k, v, nc, keep, scan=lambda a, b, c: O.scan_recurrent(a, b, c, False, "f64"))
    assert torch.allclose(out.detach(), _t(g["out"]), atol=1e-10)


def test_gpt_recurrent_golden_matches_causal_op_and_decode_step():
    g = _load("gpt_cos_attn_recurrent.npz")
    q, k, v, do = (_t(g[n]) for n in ("q", "k", "v", "dout"))
    nc = _t(g["norm_const"]).requires_grad_()
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    # prompt + single-token steps of the recurrent branch == one causal pass over all tokens
    out = O.cos_attn_causal(q, k, v, nc)
    (out * do).sum().backward()
    assert torch.allclose(out.detach(), _t(g["out"]), atol=1e-10)
    assert torch.allclose(q.grad, _t(g["dq"]), atol=1e-10)
    assert torch.allclose(k.grad, _t(g["dk"]), atol=1e-10)
    assert torch.allclose(v.grad, _t(g["dv"]), atol=1e-10)
    assert torch.allclose(nc.grad, _t(g["dnorm_const"]), atol=1e-10)
    # decode-step restatement, token by token from an empty state
    B, H, T, d = q.shape
    S = int(g["prompt_len"])
    state = torch.zeros(B, H, d, d, dtype=torch.float64)
    state_t = torch.zeros(B, H, d, d, dtype=torch.float64)
    outs = []
    for t in range(T):
        qq, kk, vv = q[:, :, t].detach(), k[:, :, t].detach(), v[:, :, t].detach()
        outs.append(O.decode_step(state, t + 1, qq, kk, vv, nc.detach()))
        state_t, o_t = O.decode_step_torch(state_t, t + 1, qq, kk, vv, nc.detach())
        assert torch.allclose(outs[-1], o_t, atol=1e-12)
        if t == S - 1:
            assert torch.allclose(state, _t(g["state_after_prompt"]), atol=1e-10)
    assert torch.allclose(torch.stack(outs, 2), _t(g["out"]), atol=1e-10)
    assert torch.allclose(state, _t(g["state_final"]), atol=1e-10)
    assert int(g["cur_s_final"]) == T + 1


@pytest.mark.parametrize("name", ["bert_cos_attn_s40.npz", "bert_cos_attn_s12.npz"])
def test_bert_golden(name):
    g = _load(name)
    H = int(g["num_heads"])
    hs = _t(g["hidden"]).requires_grad_()
    nc = _t(g["norm_const"]).requires_grad_()
    keep = torch.from_numpy(g["keep"])
    B, S, E = hs.shape
    d = E // H

    def proj(w, b):
        return (hs @ _t(g[w]).t() + _t(g[b])).view(B, S, H, d).permute(0, 2, 1, 3)

    out = O.cos_attn_bidirectional(proj("wq", "bq"), proj("wk", "bk"), proj("wv", "bv"), nc, keep)
    ctx = out.permute(0, 2, 1, 3).reshape(B, S, E)
    (ctx * _t(g["dctx"])).sum().backward()
    assert torch.allclose(ctx.detach(), _t(g["ctx"]), atol=1e-10)
    assert torch.allclose(hs.grad, _t(g["dhidden"]), atol=1e-10)
    assert torch.allclose(nc.grad, _t(g["dnorm_const"]), atol=1e-10)


GPU_FIXTURES = ["f64_gradcheck_shape", "f32_d64", "f32_d32_halfwarp", "f32_dv_ne_dk", "bf16_d64", "f16_d128"]


@pytest.mark.parametrize("name", GPU_FIXTURES)
def test_reference_cuda_kernel_fixture(name):
    """The oracle against outputs recorded from the reference's compiled CUDA kernel on a B200."""
    g = _load(f"kernel_ref_{name}.npz")
    q, k, v, do = (_t(g[n]) for n in ("q", "k", "v", "dout"))
    low = name.startswith(("bf16", "f16"))
    tol = dict(f64=1e-10, f32=2e-5).get(name[:3], None)
    for rev, key in ((False, "out"), (True, "out_rev")):
        truth = O.scan_recurrent(q, k, v, rev, "f64")
        ref = _t(g[key])
        if low:
            # the reference keeps its state in the storage type: only loosely equal to the truth
            rel = (ref - truth).norm() / truth.norm()
            assert rel < 0.1, rel
        else:
            assert torch.allclose(truth, ref, atol=tol), (truth - ref).abs().max()
    if "dq" in g and not low:
        dq, dk, dv = O.scan_backward(q, k, v, do)
        assert torch.allclose(dq, _t(g["dq"]), atol=tol * 10)
        assert torch.allclose(dk, _t(g["dk"]), atol=tol * 10)
        assert torch.allclose(dv, _t(g["dv"]), atol=tol * 10)
    if name == "bf16_d64":
        emu = O.scan_recurrent(q.float(), k.float(), v.float(), False, "bf16").double()
        ref = _t(g["out"])
        # the bf16 emulation follows the reference kernel's order of operations
        assert (emu - ref).norm() / ref.norm() < 0.02
