"""Generate golden fixtures by EXECUTING the reference's own Python modules on CPU.

Run where the reference checkout and the compiled reference extension exist:

    python oracle/build_ref.py                      # builds oracle/_ref/FastAttention2 (import-time dependency)
    python tests/golden/make_golden.py [--reference /path/to/Cottention_Transformer]

Writes small ``.npz`` files next to this script.  Nothing here is imported by the product.

What is executed, unmodified, from the reference:

* ``GPT_Trainer/GPTCosAttention.py``: ``GPTCosAttention._cos_attn`` -- its training branch
  (``:229-248,282``) and its recurrent ``fast_inference`` branch (``:235-272``);
* ``BERT_Trainer/BertCosAttention.py``: ``BertCosAttention.forward`` (``:111-334``).

The one substitution: the training branch calls ``CustomAttention.apply`` (``:282``), whose
kernel only runs on a GPU.  For the CPU fixtures that name is bound to the masked quadratic
form the reference itself states for the kernel (``Cuda_Kernel/Custom_Kernel.py:61`` /
``Cuda_Kernel/speed_test.py:15-20``); the kernel itself is pinned separately by
``make_golden_gpu.py``, which runs the compiled reference kernel on a B200.
"""
import argparse
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))


def _import_reference(root):
    os.environ.setdefault("WANDB_MODE", "disabled")
    sys.path.insert(0, os.path.join(REPO, "oracle", "_ref"))  # FastAttention2 (import-time only)
    sys.path.insert(0, os.path.join(root, "Cuda_Kernel"))
    sys.path.insert(0, os.path.join(root, "GPT_Trainer"))
    sys.path.insert(0, os.path.join(root, "BERT_Trainer"))
    cwd = os.getcwd()
    os.chdir(root)  # GPTCosAttention.py:17 appends the relative path "Cuda_Kernel"
    try:
        import GPTCosAttention as G
        import BertCosAttention as Bm
    finally:
        os.chdir(cwd)
    return G, Bm


class _QuadraticScan(torch.autograd.Function):
    """CPU stand-in bound to the name ``CustomAttention`` for the training-branch fixture:
    ``((Q K^T) * tril) V``, differentiated by torch autograd."""

    @staticmethod
    def apply(Q, K, V):  # plain function, autograd handles the rest
        S = Q.shape[-2]
        M = torch.tril(torch.ones(S, S, dtype=torch.bool))
        return ((Q @ K.transpose(-1, -2)) * M) @ V


def _f32(t):
    a = t.detach().numpy()
    b = a.astype(np.float32)
    assert (b.astype(np.float64) == a).all()
    return b


def _gpt_module(G, H, d, max_pos, fast):
    cfg = types.SimpleNamespace(
        max_position_embeddings=max_pos, attn_pdrop=0.0, resid_pdrop=0.0, hidden_size=H * d,
        num_attention_heads=H, rotary_dim=None,
    )
    if fast:
        cfg.fast_inference = True
    return G.GPTCosAttention(cfg).double()


def gpt_train_branch(G, out):
    torch.manual_seed(101)
    B, H, S, d = 2, 2, 50, 32
    mod = _gpt_module(G, H, d, 128, fast=False)
    with torch.no_grad():
        mod.norm_const.copy_(torch.tensor([0.5, -0.7], dtype=torch.float64).view(1, H, 1, 1))
    q = torch.randn(B, H, S, d).double().requires_grad_()
    k = torch.randn(B, H, S, d).double().requires_grad_()
    v = torch.randn(B, H, S, d).double().requires_grad_()
    keep = torch.ones(B, S, dtype=torch.bool)
    keep[0, :9] = False       # left padding
    keep[1, 41:] = False      # right padding
    keep[1, 17] = False       # a hole
    add_mask = torch.zeros(B, 1, 1, S, dtype=torch.float64)
    add_mask[~keep.view(B, 1, 1, S)] = torch.finfo(torch.float32).min
    saved = G.CustomAttention
    G.CustomAttention = _QuadraticScan
    try:
        o, _ = mod._cos_attn(q, k, v, add_mask)
    finally:
        G.CustomAttention = saved
    do = torch.randn(o.shape).double()
    (o * do).sum().backward()
    np.savez_compressed(
        out, q=_f32(q), k=_f32(k), v=_f32(v), keep=keep.numpy(),
        norm_const=mod.norm_const.detach().view(-1).numpy(), out=o.detach().numpy(), dout=_f32(do),
        dq=q.grad.numpy(), dk=k.grad.numpy(), dv=v.grad.numpy(),
        dnorm_const=mod.norm_const.grad.view(-1).numpy(),
    )


def gpt_module_forward(G, out, rotary_dim):
    """``GPTCosAttention.forward`` end to end (:427-511): projections, head split, rotary embedding through the
    ``transformers`` helpers the module imports (:7, :458-476), permutes, ``_cos_attn`` with a padding mask, head
    merge, output projection.  The kernel call is bound to the masked quadratic form as in ``gpt_train_branch``."""
    torch.manual_seed(404 + (rotary_dim or 0))
    B, H, S, d = 2, 2, 48, 64
    cfg = types.SimpleNamespace(max_position_embeddings=128, attn_pdrop=0.0, resid_pdrop=0.0, hidden_size=H * d,
                                num_attention_heads=H, rotary_dim=rotary_dim)
    mod = G.GPTCosAttention(cfg).double()
    with torch.no_grad():
        mod.norm_const.copy_(torch.tensor([0.5, -0.4], dtype=torch.float64).view(1, H, 1, 1))
    hs = torch.randn(B, S, H * d).double().requires_grad_()
    keep = torch.ones(B, S, dtype=torch.bool)
    keep[1, 37:] = False
    add_mask = torch.zeros(B, 1, 1, S, dtype=torch.float64)
    add_mask[~keep.view(B, 1, 1, S)] = torch.finfo(torch.float32).min
    position_ids = torch.arange(S).unsqueeze(0).repeat(B, 1)
    position_ids[1] += 5                                    # per-batch positions
    # what the module gathers for these positions (:454-456), recorded so that the test needs no transformers
    emb = mod._get_embed_positions(position_ids)
    sincos = torch.gather(emb, 1, position_ids.unsqueeze(-1).repeat(1, 1, emb.shape[-1]))
    sin, cos = torch.split(sincos, sincos.shape[-1] // 2, dim=-1)
    saved = G.CustomAttention
    G.CustomAttention = _QuadraticScan
    try:
        o = mod(hs, attention_mask=add_mask, position_ids=position_ids)[0]
    finally:
        G.CustomAttention = saved
    do = torch.randn(o.shape).double()
    (o * do).sum().backward()
    np.savez_compressed(
        out, hidden=_f32(hs), keep=keep.numpy(), position_ids=position_ids.numpy(), sin=sin.double().numpy(), cos=cos.double().numpy(),
        wq=_f32(mod.q_proj.weight), wk=_f32(mod.k_proj.weight), wv=_f32(mod.v_proj.weight),
        wo=_f32(mod.out_proj.weight), norm_const=mod.norm_const.detach().view(-1).numpy(),
        out=o.detach().numpy(), dout=_f32(do), dhidden=hs.grad.numpy(), dnorm_const=mod.norm_const.grad.view(-1).numpy(),
        dwq=mod.q_proj.weight.grad.numpy(), dwv=mod.v_proj.weight.grad.numpy(),
        num_heads=np.int64(H), rotary_dim=np.int64(rotary_dim or 0),
    )


def gpt_recurrent_branch(G, out):
    """Unmodified reference code end to end: prompt of S tokens, then single-token steps."""
    torch.manual_seed(202)
    B, H, S, d, extra = 1, 2, 45, 32, 3
    mod = _gpt_module(G, H, d, 128, fast=True)
    with torch.no_grad():
        mod.norm_const.copy_(torch.tensor([0.5, 0.9], dtype=torch.float64).view(1, H, 1, 1))
    T = S + extra
    q = torch.randn(B, H, T, d).double().requires_grad_()
    k = torch.randn(B, H, T, d).double().requires_grad_()
    v = torch.randn(B, H, T, d).double().requires_grad_()
    outs = []
    o, _ = mod._cos_attn(q[:, :, :S], k[:, :, :S], v[:, :, :S], torch.zeros(B, 1, 1, S, dtype=torch.float64))
    outs.append(o)
    state_after_prompt = mod.past_KV.detach().clone()
    for t in range(S, T):
        o, _ = mod._cos_attn(q[:, :, t:t + 1], k[:, :, t:t + 1], v[:, :, t:t + 1],
                             torch.zeros(B, 1, 1, 1, dtype=torch.float64))
        outs.append(o)
    o = torch.cat(outs, dim=2)
    do = torch.randn(o.shape).double()
    (o * do).sum().backward()
    np.savez_compressed(
        out, q=_f32(q), k=_f32(k), v=_f32(v), prompt_len=np.int64(S),
        norm_const=mod.norm_const.detach().view(-1).numpy(), out=o.detach().numpy(), dout=_f32(do),
        dq=q.grad.numpy(), dk=k.grad.numpy(), dv=v.grad.numpy(),
        dnorm_const=mod.norm_const.grad.view(-1).numpy(),
        state_after_prompt=state_after_prompt.numpy(), state_final=mod.past_KV.detach().numpy(),
        cur_s_final=np.int64(mod.cur_s),
    )


def bert_forward(Bm, out, S, name_suffix=""):
    torch.manual_seed(303 + S)
    B, H, d = 2, 2, 16
    cfg = types.SimpleNamespace(
        hidden_size=H * d, num_attention_heads=H, attention_probs_dropout_prob=0.0,
        position_embedding_type="absolute", max_position_embeddings=64, is_decoder=False,
    )
    mod = Bm.BertCosAttention(cfg).double()
    with torch.no_grad():
        mod.norm_const.copy_(torch.tensor([0.5, -1.1], dtype=torch.float64).view(1, H, 1, 1))
    hs = torch.randn(B, S, H * d).double().requires_grad_()
    keep = torch.ones(B, S, dtype=torch.bool)
    keep[1, S - S // 3:] = False
    add_mask = torch.zeros(B, 1, 1, S, dtype=torch.float64)
    add_mask[~keep.view(B, 1, 1, S)] = -10000.0
    (ctx,) = mod(hs, attention_mask=add_mask)
    dctx = torch.randn_like(ctx)
    (ctx * dctx).sum().backward()
    np.savez_compressed(
        out, hidden=hs.detach().numpy(), keep=keep.numpy(),
        wq=mod.query.weight.detach().numpy(), bq=mod.query.bias.detach().numpy(),
        wk=mod.key.weight.detach().numpy(), bk=mod.key.bias.detach().numpy(),
        wv=mod.value.weight.detach().numpy(), bv=mod.value.bias.detach().numpy(),
        norm_const=mod.norm_const.detach().view(-1).numpy(), ctx=ctx.detach().numpy(), dctx=dctx.numpy(),
        dhidden=hs.grad.numpy(), dnorm_const=mod.norm_const.grad.view(-1).numpy(),
        num_heads=np.int64(H),
    )


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("COTT_REFERENCE_ROOT"), required="COTT_REFERENCE_ROOT" not in os.environ,
                    help="path of the reference checkout (or set COTT_REFERENCE_ROOT)")
    a = ap.parse_args()
    G, Bm = _import_reference(a.reference)
    gpt_train_branch(G, os.path.join(HERE, "gpt_cos_attn_train_branch.npz"))
    gpt_recurrent_branch(G, os.path.join(HERE, "gpt_cos_attn_recurrent.npz"))
    gpt_module_forward(G, os.path.join(HERE, "gpt_module_forward_rot32.npz"), rotary_dim=32)
    gpt_module_forward(G, os.path.join(HERE, "gpt_module_forward_rot64.npz"), rotary_dim=64)   # the trainer's setting (rotary_dim = head dim)
    bert_forward(Bm, os.path.join(HERE, "bert_cos_attn_s40.npz"), S=40)   # d <= S: Q (K^T V) order
    bert_forward(Bm, os.path.join(HERE, "bert_cos_attn_s12.npz"), S=12)   # d  > S: (Q K^T) V order
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))
