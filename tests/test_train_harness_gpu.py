"""GPU tests of the whole-model training-step harnesses: two layers of the GPT-style decoder and of the BERT-style
encoder, one bf16-autocast step each, against the SAME model (same weights, same inputs) whose attention is the
oracle's fp32 statement of the reference module math (GPTCosAttention.py:229-248,282 / BertCosAttention.py:162-178,249)
behind the reference's layout handling (permute + contiguous copies).  Compared: the loss, the gradient of
``norm_const`` of every layer, and the gradients of the QKV projection weights."""
import copy

import pytest
import torch
import torch.nn.functional as F

from oracle import cott_oracle as O

pytestmark = pytest.mark.gpu


def _oracle_op(fn):
    def op(q, k, v, norm_const):
        with torch.autocast("cuda", enabled=False):
            return fn(q.float(), k.float(), v.float(), norm_const.float().reshape(-1)).to(q.dtype)
    return op


@pytest.mark.parametrize("name", ["gpt", "bert"])
@pytest.mark.parametrize("rotary", [False, True])
def test_two_layer_step_matches_the_same_model_with_the_oracle_attention(name, rotary, monkeypatch):
    from cottention_transformer_b200 import bench_train as T
    if rotary and name == "bert":
        pytest.skip("rotary belongs to the GPT module")
    causal = name == "gpt"
    cfg = dict(vocab=1000, seq=384, d_model=256, n_layers=2, n_heads=4, d_ff=512, causal=causal)
    dev = torch.device("cuda")
    torch.manual_seed(7)
    model = T.Model(**cfg).to(dev)
    with torch.no_grad():  # distinct per-head exponents, so that a head mix-up would show
        for b in model.blocks:
            b.attn.norm_const.copy_(torch.linspace(-0.5, 1.0, cfg["n_heads"]).view(1, -1, 1, 1))
    ref_model = copy.deepcopy(model)
    g = torch.Generator(device=dev).manual_seed(11)
    ids = torch.randint(0, cfg["vocab"], (3, cfg["seq"]), device=dev, generator=g)
    labels = torch.roll(ids, -1, 1)
    sincos = None
    if rotary:
        ang = torch.arange(cfg["seq"], device=dev).float()[:, None] / (10000 ** (torch.arange(0, 64, 2, device=dev).float() / 64))
        sincos = (torch.sin(ang), torch.cos(ang))

    def run(m):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits = m(ids)
        loss = F.cross_entropy(logits.float().view(-1, cfg["vocab"]), labels.view(-1))
        loss.backward()
        return loss.detach()

    # ours: packed QKV layout, fused kernels (and the rotary kernel on the packed projection)
    monkeypatch.setattr(T.CosSelfAttention, "permute", False)
    monkeypatch.setattr(T.CosSelfAttention, "rotary", sincos)
    loss = run(model)
    # the checker: the reference's layout handling around the oracle op (rotary applied by plain torch ops)
    monkeypatch.setattr(T.CosSelfAttention, "permute", True)
    monkeypatch.setattr(T.CosSelfAttention, "rotary", None)
    if causal:
        base = _oracle_op(O.cos_attn_causal)
        if rotary:
            def op(q, k, v, nc):  # q, k: [B, H, S, d]; rotate-every-two, as transformers' apply_rotary_pos_emb for GPT-J
                def rot(x):
                    s = torch.repeat_interleave(sincos[0], 2, -1)[None, None].to(torch.float32)
                    c = torch.repeat_interleave(sincos[1], 2, -1)[None, None].to(torch.float32)
                    xf = x.float()
                    x2 = torch.stack((-xf[..., 1::2], xf[..., ::2]), -1).flatten(-2)
                    return (xf * c + x2 * s).to(x.dtype)
                return base(rot(q), rot(k), v, nc)
        else:
            op = base
        monkeypatch.setattr(T, "cos_attn_causal", op)
    else:
        monkeypatch.setattr(T, "cos_attn_bidirectional", _oracle_op(O.cos_attn_bidirectional))
    ref_loss = run(ref_model)

    assert abs(loss.item() - ref_loss.item()) <= 1e-2 * abs(ref_loss.item()), (loss, ref_loss)
    for b, rb in zip(model.blocks, ref_model.blocks):
        gn, rn = b.attn.norm_const.grad.double().flatten(), rb.attn.norm_const.grad.double().flatten()
        assert (gn - rn).abs().max() <= 5e-2 * rn.abs().max() + 1e-6, (gn, rn)
        gw, rw = b.attn.qkv.weight.grad.double(), rb.attn.qkv.weight.grad.double()
        assert ((gw - rw).norm() / rw.norm()).item() <= 5e-2
