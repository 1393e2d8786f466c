"""Whole-model training-step harnesses around the cosine-attention op (synthetic data, random weights).

    python -m cottention_transformer_b200.bench_train --model gpt  [--steps 10 --warmup 3]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m cottention_transformer_b200.bench_train --model bert

gpt:  24 layers, d_model 1024, 16 heads of 64, MLP 4096 (GELU), pre-LayerNorm, vocab 50304, sequence 1024,
      batch 8 per GPU, causal cosine attention (``cos_attn_causal``), next-token loss.
bert: 12 layers, hidden 768, 12 heads of 64, intermediate 3072, vocab 30522, sequence 512, batch 32 per GPU,
      bidirectional cosine attention (``cos_attn_bidirectional``), masked-LM loss on 15 % of the positions.
bf16 autocast, fused AdamW, DDP over NCCL when launched with more than one rank.  These are minimal models
with the reference trainers' attention call sites (GPT_Trainer/GPTCosAttention.py:282,
BERT_Trainer/BertCosAttention.py:249), not the reference's HuggingFace model classes; token ids are uniform
random, so the loss value means nothing -- the harness measures tokens/s of a full step.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.nn as nn
import torch.nn.functional as F

from .cos_attention import (cos_attn_bidirectional, cos_attn_bidirectional_packed, cos_attn_causal,
                            cos_attn_causal_packed, rotary_packed_)


class CosSelfAttention(nn.Module):
    permute = False  # True: the reference's layout handling (permute + contiguous copies around the op)
    rotary = None    # (sin, cos) fp32 [S, 32]: GPT-J rotary on q and k (GPTCosAttention.py:458-476), packed path only
    rotary_separate = False  # True: a pass of its own over q, k (rotary_packed_) instead of inside the attention kernels

    def __init__(self, d_model, n_heads, causal):
        super().__init__()
        self.h, self.causal = n_heads, causal
        self.qkv = nn.Linear(d_model, 3 * d_model, bias=not causal)
        self.proj = nn.Linear(d_model, d_model, bias=not causal)
        self.norm_const = nn.Parameter(0.5 * torch.ones(1, n_heads, 1, 1))  # GPTCosAttention.py:89

    def forward(self, x):
        B, S, D = x.shape
        qkv = self.qkv(x)
        rot = None
        if self.rotary is not None and self.causal and not self.permute:
            rot = (self.rotary[0][:S], self.rotary[1][:S])
            if self.rotary_separate:
                qkv, rot = rotary_packed_(qkv, rot[0], rot[1], heads=self.h), None
        qkv = qkv.view(B, S, 3, self.h, D // self.h)
        if not self.permute:  # strided tensor maps: no head split / merge copies
            if self.causal:
                return self.proj(cos_attn_causal_packed(qkv, self.norm_const, rotary=rot).reshape(B, S, D))
            return self.proj(cos_attn_bidirectional_packed(qkv, self.norm_const).reshape(B, S, D))
        qkv = qkv.permute(2, 0, 3, 1, 4).contiguous()  # [3,B,H,S,d]
        op = cos_attn_causal if self.causal else cos_attn_bidirectional
        o = op(qkv[0], qkv[1], qkv[2], self.norm_const)
        return self.proj(o.transpose(1, 2).reshape(B, S, D))


class Block(nn.Module):
    def __init__(self, d_model, n_heads, d_ff, causal, pre_ln):
        super().__init__()
        self.pre_ln = pre_ln
        self.attn = CosSelfAttention(d_model, n_heads, causal)
        self.ln1, self.ln2 = nn.LayerNorm(d_model), nn.LayerNorm(d_model)
        self.fc1, self.fc2 = nn.Linear(d_model, d_ff), nn.Linear(d_ff, d_model)

    def forward(self, x):
        if self.pre_ln:
            x = x + self.attn(self.ln1(x))
            return x + self.fc2(F.gelu(self.fc1(self.ln2(x))))
        x = self.ln1(x + self.attn(x))
        return self.ln2(x + self.fc2(F.gelu(self.fc1(x))))


class Model(nn.Module):
    def __init__(self, vocab, seq, d_model, n_layers, n_heads, d_ff, causal):
        super().__init__()
        self.tok, self.pos = nn.Embedding(vocab, d_model), nn.Embedding(seq, d_model)
        self.blocks = nn.ModuleList(Block(d_model, n_heads, d_ff, causal, pre_ln=causal) for _ in range(n_layers))
        self.ln_f = nn.LayerNorm(d_model)
        self.head = nn.Linear(d_model, vocab, bias=False)
        self.head.weight = self.tok.weight  # tied

    def forward(self, ids):
        x = self.tok(ids) + self.pos(torch.arange(ids.shape[1], device=ids.device))
        for b in self.blocks:
            x = b(x)
        return self.head(self.ln_f(x))


CONFIGS = {
    "gpt": dict(vocab=50304, seq=1024, d_model=1024, n_layers=24, n_heads=16, d_ff=4096, causal=True, batch=8),
    "bert": dict(vocab=30522, seq=512, d_model=768, n_layers=12, n_heads=12, d_ff=3072, causal=False, batch=32),
}


def run_model(name, steps=10, warmup=3, layers=0, permute=False, rotary=False, ddp_bf16_grads=False, rotary_separate=False):
    """One harness, on this rank's current CUDA device; under more than one rank the default process group must be
    initialised (NCCL).  Returns the result dict on rank 0, None elsewhere.

    DDP settings: gradients live in the reduction buckets (``gradient_as_bucket_view``: no copy into them) and the
    buckets are 128 MB (the step is short -- 36 ms for 355 M parameters -- so a few large all-reduces that start as
    soon as the last layers' gradients exist overlap the rest of the backward better than ~60 small ones): GPT on two
    B200s 39.5 ms per step against 40.7 ms with DDP's defaults and 36.5 ms on one GPU.  What remains is the tail: the
    tied 50304 x 1024 embedding gradient (206 MB in fp32) only exists when the backward ends, so its all-reduce
    overlaps nothing.  ``ddp_bf16_grads`` moves bf16 over NVLink instead (``bf16_compress_hook``); measured slower
    (40.6 ms): the two extra cast passes over every gradient cost more than the halved transfer saves."""
    import torch.distributed as dist
    world, rank = (dist.get_world_size(), dist.get_rank()) if dist.is_available() and dist.is_initialized() else (1, 0)
    dev = torch.device("cuda", torch.cuda.current_device())
    CosSelfAttention.permute = permute
    cfg = dict(CONFIGS[name])
    batch = cfg.pop("batch")
    if layers:
        cfg["n_layers"] = layers
    CosSelfAttention.rotary = None
    CosSelfAttention.rotary_separate = rotary_separate
    if rotary:
        ang = torch.arange(cfg["seq"], device=dev).float()[:, None] / (10000 ** (torch.arange(0, 64, 2, device=dev).float() / 64))
        CosSelfAttention.rotary = (torch.sin(ang), torch.cos(ang))
    torch.manual_seed(1234)
    model = Model(**cfg).to(dev)
    n_params = sum(p.numel() for p in model.parameters())
    net = model
    if world > 1:
        net = nn.parallel.DistributedDataParallel(model, device_ids=[dev.index], gradient_as_bucket_view=True, bucket_cap_mb=128)
        if ddp_bf16_grads:
            from torch.distributed.algorithms.ddp_comm_hooks import default_hooks
            net.register_comm_hook(None, default_hooks.bf16_compress_hook)
    opt = torch.optim.AdamW(net.parameters(), lr=1e-4, fused=True)
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    ids = torch.randint(0, cfg["vocab"], (batch, cfg["seq"]), device=dev, generator=g)
    if cfg["causal"]:
        inp, labels = ids, torch.roll(ids, -1, 1)
    else:  # 15 % of the positions are replaced by a mask id and carry the label
        pick = torch.rand(ids.shape, device=dev, generator=g) < 0.15
        inp, labels = torch.where(pick, torch.full_like(ids, 103), ids), torch.where(pick, ids, torch.full_like(ids, -100))

    def step():
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits = net(inp)
        loss = F.cross_entropy(logits.float().view(-1, cfg["vocab"]), labels.view(-1), ignore_index=-100)
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    res = None
    if rank == 0:
        ms = t.item()
        res = {"what": f"{name} training step, {cfg['n_layers']} layers, bf16 autocast, AdamW"
                       + (f", DDP ({'bf16' if ddp_bf16_grads else 'fp32'} gradient all-reduce, 128 MB buckets)" if world > 1 else ""),
               "params_M": n_params / 1e6, "n_gpus": world, "batch_per_gpu": batch, "seq_len": cfg["seq"], "ms_per_step": ms,
               "tokens_per_s": world * batch * cfg["seq"] / ms * 1e3, "loss": float(loss.detach()), "data": "synthetic"}
    del net, model, opt
    torch.cuda.empty_cache()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", choices=list(CONFIGS), default="gpt")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (smoke runs)")
    ap.add_argument("--permute", action="store_true", help="permute + copy around the op instead of the packed layout")
    ap.add_argument("--rotary", action="store_true", help="gpt: rotary embedding on q and k, inside the attention kernels")
    ap.add_argument("--rotary-separate", action="store_true", help="with --rotary: as a pass of its own, in place on the packed projection")
    ap.add_argument("--bf16-allreduce", action="store_true", help="DDP: all-reduce bf16 copies of the gradients")
    a = ap.parse_args()
    world, rank, local = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", 1), ("RANK", 0), ("LOCAL_RANK", 0)))
    torch.cuda.set_device(local)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local))
    res = run_model(a.model, a.steps, a.warmup, a.layers, a.permute, a.rotary, ddp_bf16_grads=a.bf16_allreduce,
                    rotary_separate=a.rotary_separate)
    if rank == 0:
        print(json.dumps(res))
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
