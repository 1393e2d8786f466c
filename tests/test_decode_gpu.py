"""GPU parity tests of the recurrent decode step through the C ABI."""
import os

import numpy as np
import pytest
import torch

from oracle import cott_oracle as O

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_decode_matches_reference_recurrent_fixture():
    """Prompt then single tokens, against outputs and states recorded from the reference's own
    (unmodified) fast_inference branch."""
    from cottention_transformer_b200 import CosAttnDecodeState
    g = np.load(os.path.join(GOLDEN, "gpt_cos_attn_recurrent.npz"))
    q, k, v = (torch.from_numpy(g[n]).float().cuda() for n in ("q", "k", "v"))
    nc = torch.from_numpy(g["norm_const"]).float().cuda()
    S = int(g["prompt_len"])
    B, H, T, d = q.shape
    st = CosAttnDecodeState(B, H, d)
    outs = [st.step(q[:, :, :S], k[:, :, :S], v[:, :, :S], nc)]
    assert (st.state.double().cpu() - torch.from_numpy(g["state_after_prompt"])).abs().max() < 1e-5
    for t in range(S, T):
        outs.append(st.step(q[:, :, t:t + 1], k[:, :, t:t + 1], v[:, :, t:t + 1], nc))
    out = torch.cat(outs, 2)
    assert (out.double().cpu() - torch.from_numpy(g["out"])).abs().max() < 1e-4   # fp32 mode tolerance
    assert (st.state.double().cpu() - torch.from_numpy(g["state_final"])).abs().max() < 1e-5
    assert st.cur_s == int(g["cur_s_final"])


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(3, 2, 64, 64), (2, 3, 128, 128), (1, 2, 32, 48), (2, 1, 16, 7)])
def test_decode_steps_match_oracle(dt, shape):
    from cottention_transformer_b200 import CosAttnDecodeState
    B, H, Dk, Dv = shape
    T = 9
    g = torch.Generator().manual_seed(Dk + Dv)
    q = torch.randn(B, H, T, Dk, generator=g).to(dt)
    k = torch.randn(B, H, T, Dk, generator=g).to(dt)
    v = torch.randn(B, H, T, Dv, generator=g).to(dt)
    nc = torch.linspace(-0.5, 1.0, H)
    state = torch.zeros(B, H, Dv, Dk, dtype=torch.float64)
    want = torch.stack([O.decode_step(state, t + 1, q[:, :, t], k[:, :, t], v[:, :, t], nc) for t in range(T)], 2)
    # (a) token by token, (b) all T tokens in one launch: same results
    sa, sb = CosAttnDecodeState(B, H, Dk, Dv), CosAttnDecodeState(B, H, Dk, Dv)
    qa, ka, va, nca = q.cuda(), k.cuda(), v.cuda(), nc.cuda()
    got_a = torch.cat([sa.step(qa[:, :, t:t + 1], ka[:, :, t:t + 1], va[:, :, t:t + 1], nca) for t in range(T)], 2)
    got_b = sb.step(qa, ka, va, nca)
    tol = 1e-4 if dt == torch.float32 else 2e-2 * want.abs().max().item()
    assert (got_a.double().cpu() - want).abs().max().item() <= tol
    assert (got_b.double().cpu() - want).abs().max().item() <= tol
    assert (sa.state.double().cpu() - state).abs().max().item() <= 1e-4
    assert torch.allclose(sa.state, sb.state, atol=1e-6)
    assert sa.cur_s == sb.cur_s == T + 1


def test_decode_equals_causal_prefill():
    """The recurrent form and the chunked tensor-core prefill are the same function."""
    from cottention_transformer_b200 import CosAttnDecodeState, cos_attn_causal
    q, k, v, _, _ = O.make_inputs(2, 2, 200, 64, 64, seed=21, dtype=torch.bfloat16)
    nc = torch.tensor([0.5, -0.3])
    q, k, v, nc = q.cuda(), k.cuda(), v.cuda(), nc.cuda()
    a = cos_attn_causal(q, k, v, nc).float()
    b = CosAttnDecodeState(2, 2, 64).step(q, k, v, nc).float()
    assert ((a - b).norm() / b.norm()).item() < 1e-2


def test_decode_rejects_bad_arguments():
    from cottention_transformer_b200 import _lib
    L = _lib.lib()
    z = torch.zeros(1, 1, 64, 64, device="cuda")
    x = torch.zeros(1, 1, 1, 64, device="cuda")
    nc = torch.zeros(1, device="cuda")
    args = (z.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), nc.data_ptr(), x.data_ptr())
    assert L.cott_decode_step(*args, 1, 1, 48, 64, 0, 1, None, None) == 2     # Dk not supported
    assert L.cott_decode_step(*args, 1, 1, 64, 64, 1, 1, None, None) == 3     # float64 tokens
    assert L.cott_decode_step(*args, 1, 1, 64, 64, 0, 0, None, None) == 2     # positions are 1-based


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("shape", [(2, 3, 300), (1, 16, 4096)])
def test_prefill_hands_the_state_to_decode(dt, shape, d):
    """A prompt absorbed by ``prefill`` (fused causal kernels + segment-state kernels; head dim 128: the 128-wide
    kernels and a state-only pass of them) followed by single-token steps gives what the recurrent kernel gives for the
    whole stream (state and outputs)."""
    from cottention_transformer_b200 import CosAttnDecodeState
    B, H, N = shape
    T = 5
    q, k, v, _, _ = O.make_inputs(B, H, N + T, d, d, seed=N, normalize=False, dtype=dt)
    q, k, v = q.cuda(), k.cuda(), v.cuda()
    nc = torch.linspace(-0.5, 1.0, H).cuda()
    ref = CosAttnDecodeState(B, H, d)
    out_ref = ref.step(q, k, v, nc)                      # every token through the recurrent kernel (fp32 state)
    fast = CosAttnDecodeState(B, H, d)
    out_p = fast.prefill(q[:, :, :N], k[:, :, :N], v[:, :, :N], nc)
    assert fast.cur_s == N + 1
    outs = [fast.step(q[:, :, N + t:N + t + 1], k[:, :, N + t:N + t + 1], v[:, :, N + t:N + t + 1], nc) for t in range(T)]
    out_fast = torch.cat([out_p] + outs, dim=2)
    scale = out_ref.float().abs().max().item()
    assert (out_fast.float() - out_ref.float()).abs().max().item() <= 2e-2 * scale
    # the decode tokens only see the state: they isolate the hand-off
    assert (out_fast[:, :, N:].float() - out_ref[:, :, N:].float()).abs().max().item() <= 2e-2 * scale
    s_scale = ref.state.abs().max().item()
    assert (fast.state - ref.state).abs().max().item() <= 1e-2 * s_scale
