"""Causal cosine attention forward + backward on HOST buffers, pipelined over the batch.

A caller whose activations live in pinned host memory (offloaded activations, a data-loader process) pays the
PCIe copies either side of the kernels.  The kernels take ~0.2 ms for the headline shape and the copies ~10 ms
when run back to back, so the end-to-end figure is a copy-scheduling question: the link is full duplex, and every
(batch, head) sequence is independent, so the batch is cut into slices and three streams run

    host->device copy of slice i+1   |   kernels on slice i   |   device->host copy of slice i-1

at the same time (the kernels of consecutive slices on a few streams in turn: a slice of a few sequences
fills only a few SMs).  The step then costs about max(H2D, D2H) instead of H2D + kernels + D2H.

    step = CausalHostStep(B, H, N, 64, torch.bfloat16, device)
    step(q, k, v, dout, norm_const, out, dq, dk, dv)   # pinned host tensors [B,H,N,64]; returns d norm_const [H]

The arithmetic is the fused op's (``cott_cos_attn_fwd`` / ``_bwd_dq`` / ``_bwd_dkdv`` per slice through the C
ABI, GPTCosAttention.py:229-248,282 + Custom_Kernel.py:36-141), so the results are bit-identical to
``cos_attn_causal`` on device tensors; only the order of the fp32 sum over the batch of the norm-parameter
gradient differs.
"""
from __future__ import annotations

import torch

from . import _lib


class CausalHostStep:
    def __init__(self, B, H, N, D, dtype, device, slices=None, compute_streams=4, graph=False):
        if D != 64 or dtype not in (torch.bfloat16, torch.float16):
            raise RuntimeError("CausalHostStep takes head dim 64 and bfloat16 / float16 (the tensor-core kernels)")
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("CausalHostStep needs a CUDA device (there is no CPU path)")
        self.shape, self.dtype = (B, H, N, D), dtype
        # a slice is `per` consecutive (batch, head) sequences: whole batch entries, or a run of heads of one entry
        self.slices = B if slices is None else slices
        self.per = B * H // max(self.slices, 1)
        if self.slices < 1 or B * H % self.slices or (self.per % H and H % self.per):
            raise RuntimeError(f"slices={self.slices} must cut B*H={B * H} sequences into whole batch entries or equal runs of heads")
        self.sub_b, self.sub_h = (self.per // H, H) if self.per >= H else (1, self.per)
        self.code = _lib.DTYPE_CODE[dtype]
        with torch.cuda.device(self.device):
            self.dev = [torch.empty(B, H, N, D, dtype=dtype, device=self.device) for _ in range(8)]
            self.dnc = torch.empty(self.slices, self.sub_h, dtype=torch.float32, device=self.device)
            self.s_in, self.s_out = torch.cuda.Stream(self.device), torch.cuda.Stream(self.device)
            # a slice of a few sequences fills a few SMs only: slices on different streams run side by side
            self.s_run = [torch.cuda.Stream(self.device) for _ in range(max(1, compute_streams))]
            self.ev_in = [torch.cuda.Event() for _ in range(self.slices)]
            self.ev_run = [torch.cuda.Event() for _ in range(self.slices)]
        self.launches = 0
        # graph=True: the copies and launches of a step are captured once per set of host buffers and replayed
        # (a step of many small slices is otherwise bound by the host issuing ~15 calls per slice)
        self.use_graph, self.graphs = graph, {}
        with torch.cuda.device(self.device):
            self.nc_buf = torch.empty(H, dtype=torch.float32, device=self.device)
            self.dnc_sum = torch.empty(H, dtype=torch.float32, device=self.device)

    def __call__(self, q, k, v, dout, norm_const, out, dq, dk, dv):
        B, H, N, D = self.shape
        host_in, host_out = (q, k, v, dout), (out, dq, dk, dv)
        for t in host_in + host_out:
            if t.is_cuda or tuple(t.shape) != self.shape or t.dtype != self.dtype or not t.is_contiguous():
                raise RuntimeError("CausalHostStep takes contiguous host tensors of the shape and dtype it was built for")
            if not t.is_pinned():
                raise RuntimeError("CausalHostStep needs pinned host memory (pageable copies cannot overlap)")
        self.nc_buf.copy_(norm_const.detach().reshape(-1), non_blocking=True)
        self.launches += 3 * self.slices
        if not self.use_graph:
            self._issue(host_in, host_out)
        else:
            key = tuple(t.data_ptr() for t in host_in + host_out)
            g = self.graphs.get(key)
            if g is None:
                self._issue(host_in, host_out)  # once eagerly: lazy CUDA initialisation stays out of the capture
                torch.cuda.synchronize(self.device)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=torch.cuda.Stream(self.device), capture_error_mode="relaxed"):
                    self._issue(host_in, host_out)
                self.graphs[key] = g
                self.launches += 3 * self.slices
            g.replay()
        return self.dnc_sum

    def copy_only(self, host_in, host_out):
        """The copies of a step without its kernels: the four inputs host -> device on one stream and four
        tensors of the same size device -> host on another, at the same time, as whole-tensor copies.  What this
        takes is the floor of ``__call__`` on this host: the step can at best hide its kernels behind it."""
        cur = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(cur)
        with torch.cuda.stream(self.s_in):
            self.s_in.wait_event(start)
            for d, h in zip(self.dev[:4], host_in):
                d.copy_(h, non_blocking=True)
            e_in = torch.cuda.Event()
            e_in.record(self.s_in)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(start)
            for h, d in zip(host_out, self.dev[4:]):
                h.copy_(d, non_blocking=True)
            e_out = torch.cuda.Event()
            e_out.record(self.s_out)
        cur.wait_event(e_in)
        cur.wait_event(e_out)

    def _issue(self, host_in, host_out):
        B, H, N, D = self.shape
        L, P = _lib.lib(), _lib.ptr
        cur = torch.cuda.current_stream(self.device)
        nc = self.nc_buf
        start = torch.cuda.Event()
        start.record(cur)
        for s in (self.s_in, self.s_out, *self.s_run):
            s.wait_event(start)  # the previous step's readers of the device buffers are done
        dev = [d.view(B * H, N, D) for d in self.dev]
        host_in, host_out = [t.view(B * H, N, D) for t in host_in], [t.view(B * H, N, D) for t in host_out]
        dq_d, dk_d, dv_d, out_d = dev[4:]
        sb, sh = self.sub_b, self.sub_h
        for i in range(self.slices):
            sl = slice(i * self.per, (i + 1) * self.per)
            nc_i = P(nc) + 4 * ((i * self.per) % H)  # first head of the slice
            with torch.cuda.stream(self.s_in):
                for d, h in zip(dev[:4], host_in):
                    d[sl].copy_(h[sl], non_blocking=True)
                self.ev_in[i].record(self.s_in)
            run = self.s_run[i % len(self.s_run)]
            with torch.cuda.stream(run):
                run.wait_event(self.ev_in[i])
                a = [P(d[sl]) for d in dev]
                st = run.cuda_stream
                _lib.check(L.cott_cos_attn_fwd(a[0], a[1], a[2], nc_i, a[7], sb, sh, N, D, D, self.code, st), "fwd")
                _lib.check(L.cott_cos_attn_bwd_dq(a[0], a[1], a[2], nc_i, a[3], a[4], sb, sh, N, D, D, self.code, st), "bwd_dq")
                _lib.check(L.cott_cos_attn_bwd_dkdv(a[0], a[1], a[2], nc_i, a[3], a[5], a[6], P(self.dnc[i]), sb, sh, N, D, D,
                                                    self.code, st), "bwd_dkdv")
                self.ev_run[i].record(run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_run[i])
                for h, d in zip(host_out, (out_d, dq_d, dk_d, dv_d)):
                    h[sl].copy_(d[sl], non_blocking=True)
        done = torch.cuda.Event()
        done.record(self.s_out)
        cur.wait_event(done)
        torch.sum(self.dnc.view(-1, H), 0, out=self.dnc_sum)
