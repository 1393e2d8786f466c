"""The zero-edit drop-in claim, tested: the reference's own ``GPTCosAttention`` module -- the file as it is in the
reference checkout, copied byte for byte into git-ignored ``oracle/_ref/reference_modules`` by ``oracle/build_ref.py``
-- is imported with this package's ``dropin/`` directory first on ``sys.path``, so that its
``from Custom_Kernel import CustomAttention`` (GPTCosAttention.py:17-18) and, behind it, ``FastAttention2.kernel``
resolve to this library.  Its training branch ``_cos_attn`` (:229-248,282) then runs on the GPU with a padding mask
and must reproduce the fixture recorded from the reference itself (``tests/golden/make_golden.py``)."""
import importlib
import os
import sys

import numpy as np
import pytest
import torch
import types

pytestmark = pytest.mark.gpu
REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(REPO, "tests", "golden")
MODS = os.path.join(REPO, "oracle", "_ref", "reference_modules")


@pytest.fixture()
def reference_gpt_module(monkeypatch):
    if not os.path.exists(os.path.join(MODS, "GPTCosAttention.py")):
        pytest.skip("oracle/_ref/reference_modules not present (built by oracle/build_ref.py from a reference checkout)")
    monkeypatch.setenv("WANDB_MODE", "disabled")
    dropin = os.path.join(REPO, "cottention_transformer_b200", "dropin")
    monkeypatch.syspath_prepend(MODS)
    monkeypatch.syspath_prepend(dropin)
    for name in ("GPTCosAttention", "Custom_Kernel", "FastAttention2", "FastAttention2.kernel"):
        sys.modules.pop(name, None)
    G = importlib.import_module("GPTCosAttention")
    yield G
    for name in ("GPTCosAttention", "Custom_Kernel", "FastAttention2", "FastAttention2.kernel"):
        sys.modules.pop(name, None)


@pytest.mark.parametrize("dt,tol", [(torch.float64, 1e-10), (torch.float32, 1e-4)])
def test_unmodified_reference_module_runs_on_this_library(reference_gpt_module, dt, tol):
    G = reference_gpt_module
    import cottention_transformer_b200 as pkg
    assert G.CustomAttention is pkg.CustomAttention          # the module picked up this library's autograd Function
    g = np.load(os.path.join(GOLDEN, "gpt_cos_attn_train_branch.npz"))
    B, H, S, d = g["q"].shape
    cfg = types.SimpleNamespace(max_position_embeddings=128, attn_pdrop=0.0, resid_pdrop=0.0, hidden_size=H * d,
                                num_attention_heads=H, rotary_dim=None)
    mod = G.GPTCosAttention(cfg).to(dt).cuda()
    with torch.no_grad():
        mod.norm_const.copy_(torch.from_numpy(g["norm_const"]).to(dt).view(1, H, 1, 1))
    q, k, v, do = (torch.from_numpy(g[n]).to(dt).cuda() for n in ("q", "k", "v", "dout"))
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    keep = torch.from_numpy(g["keep"]).cuda()
    add_mask = torch.zeros(B, 1, 1, S, dtype=dt, device="cuda")
    add_mask[~keep.view(B, 1, 1, S)] = torch.finfo(torch.float32).min    # HF's additive padding mask
    out, _ = mod._cos_attn(q, k, v, add_mask)
    (out * do).sum().backward()
    for a, name in ((out, "out"), (q.grad, "dq"), (k.grad, "dk"), (v.grad, "dv"), (mod.norm_const.grad.view(-1), "dnorm_const")):
        err = (a.detach().double().cpu() - torch.from_numpy(g[name])).abs().max().item()
        assert err <= tol, (name, err)


@pytest.mark.parametrize("rotary_in_kernel", [False, True])
@pytest.mark.parametrize("name", ["rot32", "rot64"])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_packed_pipeline_matches_the_reference_module_forward(name, dt, rotary_in_kernel):
    """``GPTCosAttention.forward`` (:427-511) recorded from the reference in float64 -- projections, rotary embedding by
    ``transformers``' ``apply_rotary_pos_emb`` with per-batch positions, head split / merge permutes, ``_cos_attn`` with a
    padding mask, output projection -- against this library's pipeline for the same module: ONE QKV projection,
    ``rotary_packed_`` in place on it, ``cos_attn_causal_packed`` on the packed tensor (strided tensor maps, no
    permute copies), output projection.  16-bit tolerance on the output and on the gradients.
    ``rotary_in_kernel``: the rotary embedding is applied by the attention kernels themselves
    (``cos_attn_causal_packed(..., rotary=(sin, cos))``) instead of by a pass of its own."""
    from cottention_transformer_b200 import cos_attn_causal_packed, rotary_packed_
    g = np.load(os.path.join(GOLDEN, f"gpt_module_forward_{name}.npz"))
    H = int(g["num_heads"])
    hidden = torch.from_numpy(g["hidden"]).cuda().requires_grad_()
    B, S, E = hidden.shape
    d = E // H
    wqkv = torch.cat([torch.from_numpy(g[n]) for n in ("wq", "wk", "wv")], 0).cuda().requires_grad_()   # [3E, E]
    wo = torch.from_numpy(g["wo"]).cuda()
    nc = torch.from_numpy(g["norm_const"]).float().cuda().requires_grad_()
    keep = torch.from_numpy(g["keep"]).cuda()
    sin, cos = torch.from_numpy(g["sin"]).float().cuda(), torch.from_numpy(g["cos"]).float().cuda()   # [B, S, rot/2]
    # (the projections stay in fp32 so that the 16-bit error measured below is the attention path's, not the GEMMs')
    qkv = torch.nn.functional.linear(hidden, wqkv).to(dt)                    # [B, S, 3*H*d], q | k | v blocks of H*d
    if rotary_in_kernel:
        ctx = cos_attn_causal_packed(qkv.view(B, S, 3, H, d), nc, keep, rotary=(sin, cos))
    else:
        qkv = rotary_packed_(qkv, sin, cos, heads=H)
        ctx = cos_attn_causal_packed(qkv.view(B, S, 3, H, d), nc, keep)      # [B, S, H, d]
    out = torch.nn.functional.linear(ctx.reshape(B, S, E).float(), wo)
    do = torch.from_numpy(g["dout"]).cuda()
    (out.float() * do).sum().backward()

    def close(a, ref, what):
        ref = torch.from_numpy(ref).double()
        a = a.detach().double().cpu()
        e_max, e_fro = ((a - ref).abs().max() / ref.abs().max()).item(), ((a - ref).norm() / ref.norm()).item()
        # (dnorm_const: two numbers, each a nearly cancelling sum over 96 positions -- see test_cos_attn_gpu.py)
        tol = 8e-2 if what == "dnorm_const" else 2e-2
        assert e_max <= 1.5 * tol and e_fro <= tol, (what, e_max, e_fro)

    close(out, g["out"], "out")
    close(hidden.grad, g["dhidden"], "dhidden")
    close(wqkv.grad[:E], g["dwq"], "dWq")
    close(wqkv.grad[2 * E:], g["dwv"], "dWv")
    close(nc.grad, g["dnorm_const"], "dnorm_const")


def test_compiled_binding_and_ctypes_routes_give_the_same_results(monkeypatch):
    """Both routes into the library -- the compiled torch binding and ctypes -- end in the same C entry points:
    bit-identical outputs and gradients for the causal op (with a mask, with the one-pass backward), the
    bidirectional op and the reference's kernel functions."""
    from cottention_transformer_b200 import _binding, cos_attn_bidirectional, cos_attn_causal, kernel
    if _binding.module() is None:
        pytest.skip("cott_torch_binding.so not built")
    g = torch.Generator(device="cuda").manual_seed(21)
    B, H, N = 2, 3, 700
    q, k, v, do = (torch.randn(B, H, N, 64, device="cuda", generator=g).bfloat16() for _ in range(4))
    nc = torch.linspace(-0.5, 1.0, H, device="cuda")
    keep = torch.ones(B, N, dtype=torch.bool, device="cuda")
    keep[0, 500:] = False

    def run(fn):
        a, b, c = (t.clone().requires_grad_() for t in (q, k, v))
        n = nc.clone().requires_grad_()
        out = fn(a, b, c, n)
        out.backward(do)
        return [out.detach(), a.grad, b.grad, c.grad, n.grad]

    cases = [lambda a, b, c, n: cos_attn_causal(a, b, c, n), lambda a, b, c, n: cos_attn_causal(a, b, c, n, keep, segments=3),
             lambda a, b, c, n: cos_attn_causal(a, b, c, n, one_pass_backward=True), lambda a, b, c, n: cos_attn_bidirectional(a, b, c, n, keep)]
    compiled = [run(f) for f in cases]
    scan_c = kernel.bfloat16(q, k, v, 1, False, True)
    monkeypatch.setattr(_binding, "ops", lambda: None)
    monkeypatch.setattr(_binding, "module", lambda: None)
    plain = [run(f) for f in cases]
    for x, y in zip(compiled, plain):
        for a, b in zip(x[:4], y[:4]):
            assert torch.equal(a, b)
        assert torch.allclose(x[4], y[4], rtol=1e-5, atol=1e-6)   # (atomics: the order of the fp32 sum may differ)
    assert torch.equal(scan_c, kernel.bfloat16(q, k, v, 1, False, True))
