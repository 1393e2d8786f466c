"""Secondary measurements of the hot path (not the headline bench line): recurrent decode and the
bidirectional (encoder) form, each against the HBM roofline.

    python -m cottention_transformer_b200.bench_extra [--decode-steps 256] [--json out.json]

Decode: batch 64, H=16, d in {64, 128}, bf16 tokens, fp32 state in HBM, one launch per token
(``cott_decode_step``), plus the multi-token launch (``cott_decode_steps``) that keeps the state in
registers.  Algorithmic bytes per (b,h) per step: 2*d*d*4 (state read + write) + 4*d*2 (q, k, v, out).
Bidirectional: B=32, H=12, N=512, d=64, bf16 (BERT-base attention shapes), forward + backward.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from . import _lib


def _peak_gbs():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def _time(fn, iters, warmup=5):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e-3  # seconds per call


def bench_decode(d, steps, B=64, H=16):
    L = _lib.lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(1234)
    nstates = 8  # rotate over several state buffers so that the state does not sit in L2 (8 x 16.8/67 MB)
    states = [torch.zeros(B, H, d, d, device=dev) for _ in range(nstates)]
    q = torch.randn(B, H, 1, d, device=dev, generator=g).bfloat16()
    k = torch.randn(B, H, 1, d, device=dev, generator=g).bfloat16()
    v = torch.randn(B, H, 1, d, device=dev, generator=g).bfloat16()
    out = torch.empty_like(v)
    nc = 0.5 * torch.ones(H, device=dev)
    stream = _lib.stream_ptr(dev)
    it = [0]

    def one():
        s = states[it[0] % nstates]
        it[0] += 1
        _lib.check(L.cott_decode_step(s.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), nc.data_ptr(), out.data_ptr(),
                                      B, H, d, d, 3, it[0], None, stream), "cott_decode_step")

    t_eager = _time(one, steps)
    # the per-token launch is host-bound when driven from Python: replay the same launches from a CUDA graph
    t = t_eager
    graphed = False
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            stream_side = _lib.stream_ptr(dev)
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=side):
                for i in range(64):
                    s_ = states[i % nstates]
                    _lib.check(L.cott_decode_step(s_.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), nc.data_ptr(),
                                                  out.data_ptr(), B, H, d, d, 3, i + 1, None, _lib.stream_ptr(dev)),
                               "cott_decode_step")
        torch.cuda.current_stream().wait_stream(side)
        t = _time(gr.replay, max(4, steps // 64), warmup=2) / 64
        graphed = True
    except Exception as e:  # report the eager figure and say why
        graphed = f"graph capture failed: {type(e).__name__}: {str(e)[:80]}"
    bytes_step = B * H * (2 * d * d * 4 + 4 * d * 2)
    t2 = _decode_groups(L, dev, d, B, H, nstates, groups=2) if graphed is True else None
    # multi-token launch: state resident in registers
    T = 512
    qs = torch.randn(B, H, T, d, device=dev, generator=g).bfloat16()
    ks = torch.randn(B, H, T, d, device=dev, generator=g).bfloat16()
    vs = torch.randn(B, H, T, d, device=dev, generator=g).bfloat16()
    outs = torch.empty_like(vs)

    def many():
        _lib.check(L.cott_decode_steps(states[0].data_ptr(), qs.data_ptr(), ks.data_ptr(), vs.data_ptr(), nc.data_ptr(),
                                       outs.data_ptr(), B, H, T, d, d, 3, 1, None, stream), "cott_decode_steps")

    tm = _time(many, 5, warmup=2)
    peak, kind = _peak_gbs()
    return {
        "what": f"decode step, batch {B}, H={H}, d={d}, bf16 tokens, fp32 state",
        "us_per_step": t * 1e6, "us_per_step_python_launch": t_eager * 1e6, "cuda_graph": graphed,
        "tokens_per_s": B / t, "algorithmic_bytes_per_step": bytes_step,
        "achieved_gbs": bytes_step / t / 1e9, "peak_gbs": peak, "peak_source": kind, "frac": bytes_step / t / 1e9 / peak,
        "multi_token_launch": {"T": T, "us_per_token": tm / T * 1e6, "tokens_per_s": B * T / tm},
        "two_groups": None if t2 is None else {
            "what": "the batch as two independent half-batches, each its own chain of per-token launches on its own stream",
            "us_per_step": t2 * 1e6, "tokens_per_s": B / t2, "frac": bytes_step / t2 / 1e9 / peak},
    }


def _decode_groups(L, dev, d, B, H, nstates, groups=2, steps=64, reps=16):
    """The same decode work as ``groups`` independent chains (different batch entries never depend on each other): one
    CUDA graph of per-token launches per group, replayed on a stream of its own, so that one chain's launch gap and
    first-byte latency fall into the other's streaming.  Seconds per step of the whole batch."""
    Bc = B // groups
    g = torch.Generator(device=dev).manual_seed(4321)
    nc = 0.5 * torch.ones(H, device=dev)
    cur = torch.cuda.current_stream()
    streams, graphs, keep = [torch.cuda.Stream() for _ in range(groups)], [], []
    for c in range(groups):
        states = [torch.zeros(Bc, H, d, d, device=dev) for _ in range(nstates)]
        q, k, v = (torch.randn(Bc, H, 1, d, device=dev, generator=g).bfloat16() for _ in range(3))
        out = torch.empty_like(v)
        keep.append((states, q, k, v, out))
        s = streams[c]
        s.wait_stream(cur)
        with torch.cuda.stream(s):
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=s):
                for i in range(steps):
                    _lib.check(L.cott_decode_step(states[i % nstates].data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                                  nc.data_ptr(), out.data_ptr(), Bc, H, d, d, 3, i + 1, None,
                                                  _lib.stream_ptr(dev)), "cott_decode_step")
        graphs.append(gr)
    torch.cuda.synchronize()

    def once():
        for c in range(groups):
            streams[c].wait_stream(cur)
            with torch.cuda.stream(streams[c]):
                graphs[c].replay()
        for c in range(groups):
            cur.wait_stream(streams[c])

    return _time(once, reps, warmup=3) / steps


def bench_bidir(B=32, H=12, N=512, d=64):
    from .cos_attention import cos_attn_bidirectional
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(1234)
    q, k, v, do = (torch.randn(B, H, N, d, device=dev, generator=g).bfloat16() for _ in range(4))
    nc = (0.5 * torch.ones(H, device=dev)).requires_grad_()
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()

    def step():
        out = cos_attn_bidirectional(q, k, v, nc)
        out.backward(do)
        q.grad = k.grad = v.grad = nc.grad = None

    t = _time(step, 20)
    # the two kernels on their own, through the C ABI (no autograd bookkeeping)
    L = _lib.lib()
    st = _lib.stream_ptr(dev)
    scr = torch.empty(L.cott_bidir_scratch_bytes(B, H, N, d, d, 3) // 4 + 1, device=dev)
    scr2 = torch.empty_like(scr)
    out, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
    dnc = torch.empty(H, device=dev)
    P = lambda x: x.data_ptr()  # noqa: E731
    ncd = nc.detach()
    t_f = _time(lambda: _lib.check(L.cott_bidir_fwd(P(q), P(k), P(v), None, P(ncd), P(out), P(scr), B, H, N, d, d, 3, st),
                                   "bidir fwd"), 20)
    t_b = _time(lambda: _lib.check(L.cott_bidir_bwd(P(q), P(k), P(v), None, P(ncd), P(do), P(scr), P(scr2), P(dq), P(dk),
                                                    P(dv), P(dnc), B, H, N, d, d, 3, st), "bidir bwd"), 20)
    _lib.check_device_status()
    nbytes = 11 * B * H * N * d * 2
    peak, kind = _peak_gbs()
    return {"what": f"bidirectional fwd+bwd, B={B} H={H} N={N} d={d} bf16", "us_per_step": t * 1e6,
            "fwd_kernel_us": t_f * 1e6, "bwd_kernel_us": t_b * 1e6,
            "kernels_frac": nbytes / (t_f + t_b) / 1e9 / _peak_gbs()[0],
            "tokens_per_s": B * N / t, "algorithmic_bytes": nbytes, "achieved_gbs": nbytes / t / 1e9,
            "peak_gbs": peak, "peak_source": kind, "frac": nbytes / t / 1e9 / peak}


def bench_scan_d128(B=1, H=16, N=16384, d=128):
    """Head dim 128: one scan per dtype (bf16: 64-wide tensor-core launches on strided slices; fp32: exact kernel)."""
    L = _lib.lib()
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(1234)
    res = {"what": f"bare scan, B={B} H={H} N={N} d={d}"}
    st = _lib.stream_ptr(dev)
    for name, dt in (("bf16", torch.bfloat16), ("f32", torch.float32)):
        q, k, v = (torch.nn.functional.normalize(torch.randn(B, H, N, d, device=dev, generator=g), dim=-1).to(dt) for _ in range(3))
        out = torch.empty_like(q)
        fn = lambda: _lib.check(L.cott_scan(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, H, N, d, d,  # noqa: E731
                                            _lib.DTYPE_CODE[dt], 0, st), "cott_scan")
        res[name + "_scan_us"] = _time(fn, 3, 1) * 1e6
    return res


def bench_scan(B=8, H=16, N=4096, d=64):
    """The reference's own operator (``FastAttention2.kernel.*`` = ``cott_scan``; ``CustomAttention`` backward =
    ``cott_scan_bwd``, three scans) at the headline shape, per dtype.  bf16 / fp16 run on the tensor cores, fp32 /
    fp64 on the exact CUDA-core kernel.  Algorithmic bytes: 4 tensor passes per scan."""
    L = _lib.lib()
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(1234)
    peak, kind = _peak_gbs()
    res = {"what": f"bare scan (reference kernel API), B={B} H={H} N={N} d={d}", "peak_source": kind}
    st = _lib.stream_ptr(dev)
    P = lambda t: t.data_ptr()  # noqa: E731
    for name, dt, iters in (("bf16", torch.bfloat16, 20), ("f16", torch.float16, 20), ("f32", torch.float32, 5),
                            ("f64", torch.float64, 2)):
        q, k, v, do = (torch.nn.functional.normalize(torch.randn(B, H, N, d, device=dev, generator=g), dim=-1).to(dt)
                       for _ in range(4))
        out, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
        code = _lib.DTYPE_CODE[dt]
        fwd = lambda r: _lib.check(L.cott_scan(P(q), P(k), P(v), P(out), B, H, N, d, d, code, r, st), "cott_scan")  # noqa: E731
        bwd = lambda: _lib.check(L.cott_scan_bwd(P(q), P(k), P(v), P(do), P(dq), P(dk), P(dv), B, H, N, d, d, code, st),  # noqa: E731
                                 "cott_scan_bwd")
        t_f, t_r, t_b = _time(lambda: fwd(0), iters, 2), _time(lambda: fwd(1), iters, 2), _time(bwd, iters, 2)
        nbytes = 4 * q.numel() * q.element_size()
        res[name] = {"scan_us": t_f * 1e6, "scan_reversed_us": t_r * 1e6, "scan_bwd_us": t_b * 1e6,
                     "scan_frac_of_hbm_peak": nbytes / t_f / 1e9 / peak,
                     "fwd_bwd_tokens_per_s": B * N / (t_f + t_b)}
    _lib.check_device_status()
    return res


def bench_long_context(N, B=1, H=16, d=64, iters=5):
    """Prefill forward + backward at B=1 (few sequences, long): segment-parallel against one CTA per head."""
    L = _lib.lib()
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(1234)
    q, k, v, do = (torch.randn(B, H, N, d, device=dev, generator=g).bfloat16() for _ in range(4))
    out, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
    nc, dnc = 0.5 * torch.ones(H, device=dev), torch.empty(H, device=dev)
    st = _lib.stream_ptr(dev)
    P = lambda t: t.data_ptr()  # noqa: E731
    nseg = L.cott_cos_attn_seg_count(B, H, N)
    ws = torch.empty(max(L.cott_cos_attn_seg_workspace_bytes(B, H, N, nseg), 16), dtype=torch.uint8, device=dev)

    def step(n):
        _lib.check(L.cott_cos_attn_fwd_seg(P(q), P(k), P(v), None, P(nc), P(out), P(ws), n, None, B, H, N, d, d, 3, st), "fwd_seg")
        _lib.check(L.cott_cos_attn_bwd_seg(P(q), P(k), P(v), None, P(nc), P(do), P(ws), n, None, P(dq), P(dk), P(dv), P(dnc), B, H, N, d, d,
                                           3, st), "bwd_seg")

    t_seg = _time(lambda: step(nseg), iters, warmup=2)
    t_one = _time(lambda: step(1), iters, warmup=2)
    _lib.check_device_status()
    nbytes = 11 * B * H * N * d * 2
    peak, kind = _peak_gbs()
    return {"what": f"causal fwd+bwd prefill, B={B} H={H} N={N} d={d} bf16", "segments": nseg, "us_per_step": t_seg * 1e6,
            "tokens_per_s": B * N / t_seg, "one_cta_per_head_us": t_one * 1e6, "speedup_vs_one_cta_per_head": t_one / t_seg,
            "algorithmic_bytes": nbytes, "achieved_gbs": nbytes / t_seg / 1e9, "peak_gbs": peak, "peak_source": kind,
            "frac": nbytes / t_seg / 1e9 / peak}


def bench_long_context_d128(N, B=1, H=16, d=128, iters=5):
    """Head dim 128 has no fused kernel: ``cos_attn_causal`` keeps the row factors in fp32 outside four tensor-core
    scans that run as 64-wide launches (``_WideCausal``)."""
    from .cos_attention import cos_attn_causal
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(1234)
    q, k, v = (torch.randn(B, H, N, d, device=dev, generator=g).bfloat16().requires_grad_() for _ in range(3))
    do = torch.randn(B, H, N, d, device=dev, generator=g).bfloat16()
    nc = (0.5 * torch.ones(1, H, 1, 1, device=dev)).requires_grad_()

    def step():
        q.grad = k.grad = v.grad = nc.grad = None
        cos_attn_causal(q, k, v, nc).backward(do)

    t = _time(step, iters, warmup=2)
    _lib.check_device_status()
    nbytes = 11 * B * H * N * d * 2
    peak, kind = _peak_gbs()
    return {"what": f"causal fwd+bwd prefill, B={B} H={H} N={N} d={d} bf16, the fused 128-wide tensor-core kernels",
            "us_per_step": t * 1e6, "tokens_per_s": B * N / t, "algorithmic_bytes": nbytes, "frac": nbytes / t / 1e9 / peak,
            "peak_source": kind}


def bench_prefill_sharded(N, d, world=1, rank=0, iters=3, H=16):
    """Long-context prefill, forward + backward, B = 1, the H heads split over `world` GPUs (no tensor crosses GPUs:
    every head is an independent sequence).  The full tensors are generated from one seed and sliced, so every GPU
    count works on the same data.  Through the public op ``cos_attn_causal`` (head dim 64: fused tensor-core kernels,
    segment-parallel; head dim 128: the fused 128-wide kernels, one scan per output).  Returns this rank's seconds per step."""
    from .cos_attention import cos_attn_causal
    from .sharding import shard_range
    dev = torch.device("cuda", torch.cuda.current_device())
    h0, h1 = shard_range(H, world, rank)
    g = torch.Generator(device=dev).manual_seed(1234 + d)
    loc = []
    for i in range(4):  # q, k, v, dout: one full tensor at a time
        full = torch.randn(1, H, N, d, device=dev, generator=g)
        if i < 2:
            full = torch.nn.functional.normalize(full, dim=-1)
        loc.append(full[:, h0:h1].to(torch.bfloat16).contiguous())
        del full
    q, k, v, do = loc
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    nc = (0.5 * torch.ones(h1 - h0, device=dev)).requires_grad_()

    def step():
        q.grad = k.grad = v.grad = nc.grad = None
        cos_attn_causal(q, k, v, nc).backward(do)

    t = _time(step, iters, warmup=2)
    _lib.check_device_status()
    return t


def bench_one_pass(B=8, H=16, N=4096, d=64, iters=20):
    """The two backward routes at the headline shape, kernels only through the C ABI: forward / forward that also keeps
    its chunk states, and the two-kernel backward / the one-pass backward that reads those states."""
    L = _lib.lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(1234)
    q, k, v, do = (torch.randn(B, H, N, d, device=dev, generator=g).bfloat16() for _ in range(4))
    out, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
    nc, dnc = 0.5 * torch.ones(H, device=dev), torch.empty(H, device=dev)
    saved = torch.empty(L.cott_cos_attn_saved_bytes(B, H, N), dtype=torch.uint8, device=dev)
    st = _lib.stream_ptr(dev)
    P = lambda t: t.data_ptr()  # noqa: E731
    fns = {
        "fwd_us": lambda: L.cott_cos_attn_fwd(P(q), P(k), P(v), P(nc), P(out), B, H, N, d, d, 3, st),
        "fwd_keeping_states_us": lambda: L.cott_cos_attn_fwd_train(P(q), P(k), P(v), None, P(nc), P(out), P(saved), None, 1, None, B, H, N,
                                                                   d, d, 3, st),
        "bwd_two_kernels_us": lambda: L.cott_cos_attn_bwd(P(q), P(k), P(v), P(nc), P(do), P(dq), P(dk), P(dv), P(dnc), B, H, N, d, d, 3, st),
        "bwd_one_pass_us": lambda: L.cott_cos_attn_bwd_train(P(q), P(k), P(v), None, P(nc), P(do), P(saved), None, 1, None, P(dq), P(dk),
                                                             P(dv), P(dnc), B, H, N, d, d, 3, st),
    }
    res = {"what": f"causal backward routes, B={B} H={H} N={N} d={d} bf16, kernels only"}
    for name, fn in fns.items():
        res[name] = _time(lambda: _lib.check(fn(), name), iters, warmup=3) * 1e6
    _lib.check_device_status()
    res["hbm_passes"] = {"two_kernels": 11, "one_pass": 7.5, "forward_extra_for_one_pass": 0.5}
    return res


def bench_rotary(B=8, H=16, N=1024, d=64, iters=20):
    """The rotary embedding of q, k: inside the causal kernels against a pass of its own, on a packed [B, N, 3, H, 64]
    tensor, kernels only through the C ABI (forward and backward timed separately)."""
    import ctypes
    L = _lib.lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(1234)
    qkv = torch.randn(B, N, 3, H, d, device=dev, generator=g).bfloat16()
    dqkv = torch.empty_like(qkv)
    do = torch.randn(B, N, H, d, device=dev, generator=g).bfloat16()
    out = torch.empty_like(do)
    nc, dnc = 0.5 * torch.ones(H, device=dev), torch.empty(H, device=dev)
    ang = torch.arange(N, device=dev).float()[:, None] / (10000 ** (torch.arange(0, d, 2, device=dev).float() / d))
    sin, cos = torch.sin(ang).contiguous(), torch.cos(ang).contiguous()
    lay = _lib.CottLayout(N * 3 * H * d, d, 3 * H * d, N * H * d, d, H * d)
    rlay = _lib.CottLayout(N * 3 * H * d, d, 3 * H * d, 0, 0, 0)
    rot = _lib.CottRotaryTables(sin.data_ptr(), cos.data_ptr(), d, 0)
    ws = torch.empty(L.cott_cos_attn_seg_workspace_bytes(B, H, N, 1), dtype=torch.uint8, device=dev)
    st = _lib.stream_ptr(dev)
    P = lambda t: t.data_ptr()  # noqa: E731
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    gq, gk, gv = dqkv[:, :, 0], dqkv[:, :, 1], dqkv[:, :, 2]
    LB, RB = ctypes.byref(lay), ctypes.byref(rot)
    fns = {
        "fwd_us": lambda: L.cott_cos_attn_fwd_seg(P(q), P(k), P(v), None, P(nc), P(out), P(ws), 1, LB, B, H, N, d, d, 3, st),
        "fwd_rotary_inside_us": lambda: L.cott_cos_attn_fwd_rotary(P(q), P(k), P(v), None, P(nc), P(out), P(ws), LB, RB, B, H, N, d, d, 3, st),
        "bwd_us": lambda: L.cott_cos_attn_bwd_seg(P(q), P(k), P(v), None, P(nc), P(do), P(ws), 1, LB, P(gq), P(gk), P(gv), P(dnc), B, H,
                                                  N, d, d, 3, st),
        "bwd_rotary_inside_us": lambda: L.cott_cos_attn_bwd_rotary(P(q), P(k), P(v), None, P(nc), P(do), P(ws), LB, RB, P(gq), P(gk), P(gv),
                                                                   P(dnc), B, H, N, d, d, 3, st),
        "rotary_pass_us": lambda: L.cott_rotary(P(q), P(k), P(sin), P(cos), ctypes.byref(rlay), B, H, N, d, d, 0, 0, 3, st),
    }
    res = {"what": f"rotary embedding inside the causal kernels vs a pass of its own, packed QKV, B={B} H={H} N={N} d={d} bf16, kernels only"}
    for name, fn in fns.items():
        res[name] = _time(lambda: _lib.check(fn(), name), iters, warmup=3) * 1e6
    _lib.check_device_status()
    return res


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--decode-steps", type=int, default=256)
    ap.add_argument("--json", default=None)
    ap.add_argument("--long-context", action="store_true", help="only the B=1 long-sequence prefill sweep")
    ap.add_argument("--scan", action="store_true", help="only the bare scan of the reference's kernel API, per dtype")
    ap.add_argument("--bidir-only", action="store_true", help="only the bidirectional benchmark")
    ap.add_argument("--one-pass", action="store_true", help="only the two backward routes at the headline shape")
    ap.add_argument("--prefill", nargs=2, type=int, metavar=("N", "D"), help="only one long-context prefill step (B=1, H=16)")
    ap.add_argument("--rotary", nargs="?", type=int, const=1024, metavar="N", help="only the rotary routes, B=8 H=16 at sequence length N")
    a = ap.parse_args()
    if a.rotary:
        print(json.dumps(bench_rotary(N=a.rotary)))
        raise SystemExit(0)
    if a.long_context:
        for n in (16384, 65536, 262144):
            print(json.dumps(bench_long_context(n)))
        for n in (16384, 65536, 262144):
            print(json.dumps(bench_long_context_d128(n)))
        raise SystemExit(0)
    if a.scan:
        print(json.dumps(bench_scan()))
        print(json.dumps(bench_scan_d128()))
        raise SystemExit(0)
    if a.one_pass:
        print(json.dumps(bench_one_pass()))
        raise SystemExit(0)
    if a.prefill:
        n, d = a.prefill
        t = bench_prefill_sharded(n, d)
        print(json.dumps({"what": f"causal fwd+bwd prefill, B=1 H=16 N={n} d={d} bf16", "us_per_step": t * 1e6,
                          "frac": 11 * 16 * n * d * 2 / t / 1e9 / _peak_gbs()[0]}))
        raise SystemExit(0)
    if a.bidir_only:
        print(json.dumps(bench_bidir()))
        raise SystemExit(0)
    res = [bench_decode(64, a.decode_steps), bench_decode(128, a.decode_steps),
           bench_bidir()]
    for r in res:
        print(json.dumps(r))
    if a.json:
        json.dump(res, open(a.json, "w"), indent=1)
