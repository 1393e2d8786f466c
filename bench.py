"""Benchmark of the hot path: causal cosine attention forward + backward (tokens/s).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" = one forward + one backward of the fused causal cosine-attention op over one batch
of synthetic input of the headline shape (B=8 per GPU, H=16, N=4096, d=64, bfloat16).  Under
torchrun each rank (one per GPU) processes its own batch shard; there is no data-path collective
(weak scaling).  Rank 0 prints ONE JSON line.

Keys beyond the basic contract:
  value      whole-job tokens/s with inputs resident in HBM, device-timed (CUDA events), max over ranks
  e2e        the same through the public host-buffer call (``CausalHostStep``) with pinned HOST buffers: every
             step copies q, k, v, dO host->device and out, dq, dk, dv, dnorm device->host inside the timed
             region, pipelined over the batch on three streams (the PCIe link is full duplex)
  roofline   the dominant kernel (reverse-direction dK/dV pass): algorithmic bytes per launch /
             average launch duration (CUDA events on the launching stream, inside the timed region)
             against the measured HBM copy bandwidth
  cpu_baseline  the reference's PyTorch CPU formulation (cumsum form + autograd) restated in oracle/,
             timed on this host on a bounded sample of the same workload
  extra      secondary workloads, each with its own algorithmic bytes, device time and fraction of the HBM peak:
             ``prefill_long`` (B=1, H=16 heads split over the ranks, N in {16k, 64k, 256k}, d in {64, 128}, fwd+bwd)
             and ``decode`` (batch 64 per GPU, 4096 single-token steps, fp32 state, d in {64, 128}) with the
             reference's CPU recurrent loop timed beside it, ``bidirectional`` (fwd+bwd at BERT-base attention
             shapes) and ``train`` (whole-model bf16 training steps of a
             GPT-style decoder and a BERT-base encoder with the op inside, DDP when there are several ranks);
             ``--no-extra`` skips them

``--impl reference`` times that CPU formulation alone, with all host threads, as the reference arm; when the
reference's CUDA extension has been built into oracle/_ref it also reports, under ``reference_cuda_kernel``, what that
extension does on the GPU for the same shape (context only: the arm's ``value`` is the CPU figure).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

B_PER_GPU, H, N, D = 8, 16, 4096, 64
WORKLOAD = "causal cosine attention fwd+bwd, B=8/GPU H=16 N=4096 d=64 bf16 (Q,K L2-normalised N(0,1), norm_const=0.5)"
ELEM = 2  # bf16
# dram__bytes_read.sum + dram__bytes_write.sum per launch of causal_bwd_kv_kernel at the bench shape, RECORDED from an
# ncu capture of this kernel (268.5 MB read + 98.2 MB write): a run of this file does not measure it.
RECORDED_TRAFFIC_BYTES_PER_LAUNCH = 366_749_952


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._halt = threading.Event()
        self.ready = threading.Event()   # set once NVML is initialised (or has failed)
        self.armed = False               # samples are recorded only while armed (the timed region)

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {
                nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
                nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
                nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
                nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
            }
            self.ready.set()
            while not self._halt.is_set():
                if self.armed:
                    self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                    for bit, name in names.items():
                        if r & bit:
                            self.reasons.add(name)
                time.sleep(0.001)
        except Exception as e:  # NVML missing: report nothing rather than fail the bench
            self.reasons.add(f"nvml_unavailable:{type(e).__name__}")
            self.ready.set()

    def stop(self):
        self._halt.set()
        self.join(timeout=2)
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
        }


def _bind_to_gpu_numa_node(index):
    """Restrict this process to the CPUs next to GPU `index` (sysfs: the PCI device's local_cpulist), so that the
    pinned host buffers it allocates afterwards are first touched on that NUMA node.  Read-only with respect to
    the GPU; returns what was found, or None when the topology is not exposed."""
    try:
        bus = torch.cuda.get_device_properties(index).pci_bus_id
        domain = torch.cuda.get_device_properties(index).pci_domain_id
        dev_id = torch.cuda.get_device_properties(index).pci_device_id
        path = f"/sys/bus/pci/devices/{domain:04x}:{bus:02x}:{dev_id:02x}.0"
        with open(os.path.join(path, "numa_node")) as f:
            node = int(f.read().strip())
        with open(os.path.join(path, "local_cpulist")) as f:
            cpulist = f.read().strip()
        cpus = set()
        for part in cpulist.split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if allowed:
            os.sched_setaffinity(0, allowed)
        return {"node": node, "cpus": cpulist, "bound": bool(allowed)}
    except Exception:
        return None


def _host_inputs(rank):
    """Seeded synthetic shard of this rank in pinned host memory (seed 1234 + rank)."""
    from cottention_transformer_b200.synthetic import make_inputs
    q, k, v, do, nc = make_inputs(B_PER_GPU, H, N, D, seed=1234 + rank, dtype=torch.bfloat16)
    return [t.pin_memory() for t in (q, k, v, do)], nc


def cpu_reference_sample(threads, budget_s=12.0, max_slices=64):
    """The reference's PyTorch formulation on CPU (cumsum form, Custom_Kernel.py:63, with the module
    math of GPTCosAttention.py:229-248 around it, gradients by autograd), fp32, on (b,h) slices of
    the bench workload.  Returns (tokens_per_s, slices_done, seconds)."""
    from oracle import cott_oracle as O
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(1234)
    done, t_total = -1, 0.0  # the first slice is a warm-up (thread pool, allocator) and is not counted
    while done < max_slices and t_total < budget_s:
        q = torch.nn.functional.normalize(torch.randn(1, 1, N, D, generator=g), dim=-1).requires_grad_()
        k = torch.nn.functional.normalize(torch.randn(1, 1, N, D, generator=g), dim=-1).requires_grad_()
        v = torch.randn(1, 1, N, D, generator=g).requires_grad_()
        do = torch.randn(1, 1, N, D, generator=g)
        nc = (0.5 * torch.ones(1)).requires_grad_()
        t0 = time.perf_counter()
        out = O.cos_attn_causal(q, k, v, nc, scan=lambda a, b, c: O.scan_cumsum(a, b, c, False))
        out.backward(do)
        if done >= 0:
            t_total += time.perf_counter() - t0
        done += 1
    tokens = done * N / H  # one token = one position across all H heads
    return tokens / t_total, done, t_total


def cpu_decode_sample(d, threads, steps=200, heads=16):
    """The reference's recurrent decode loop on the CPU (GPTCosAttention.py:253-272 as restated in oracle/: batch 1,
    float64 [1, H, d, d] state, torch ops per token).  Returns tokens/s."""
    from oracle import cott_oracle as O
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(d)
    q, k, v = (torch.randn(1, heads, steps + 8, d, generator=g) for _ in range(3))
    nc = 0.5 * torch.ones(heads)
    state = torch.zeros(1, heads, d, d, dtype=torch.float64)
    for t in range(8):
        state, _ = O.decode_step_torch(state, t + 1, q[:, :, t], k[:, :, t], v[:, :, t], nc)
    t0 = time.perf_counter()
    for t in range(8, steps + 8):
        state, _ = O.decode_step_torch(state, t + 1, q[:, :, t], k[:, :, t], v[:, :, t], nc)
    return steps / (time.perf_counter() - t0)


def cpu_config1_forward(threads):
    """The reference's CPU-runnable case whole: forward only, fp32, B=2, H=8, N=1024, d=64, PyTorch cumsum
    formulation with the module math around it.  Returns seconds."""
    from oracle import cott_oracle as O
    torch.set_num_threads(threads)
    q, k, v, _, nc = O.make_inputs(2, 8, 1024, 64, seed=1234)
    best = None
    for _ in range(2):
        t0 = time.perf_counter()
        with torch.no_grad():
            O.cos_attn_causal(q, k, v, nc, scan=lambda a, b, c: O.scan_cumsum(a, b, c, False))
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return best


def run_extras(world, rank, dev, with_cpu):
    """Secondary workloads (every rank takes part; figures are the max over ranks of device-timed seconds)."""
    import torch.distributed as dist
    from cottention_transformer_b200 import bench_extra as X
    from cottention_transformer_b200.sharding import shard_range
    peak, kind = _peaks()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    heads = 16
    h0, h1 = shard_range(heads, world, rank)
    prefill = []
    for d in (64, 128):
        for n in (16384, 65536, 262144):
            t = max_over_ranks(X.bench_prefill_sharded(n, d, world, rank, H=heads))
            nbytes = 11 * heads * n * d * ELEM  # 4 (fwd) + 7 (bwd) tensor passes over all heads
            prefill.append({"N": n, "d": d, "heads_on_rank0": h1 - h0, "us_per_step": t * 1e6, "tokens_per_s": n / t,
                            "algorithmic_bytes": nbytes, "achieved_gbs": nbytes / t / 1e9,
                            "frac": nbytes / t / 1e9 / (world * peak)})
            torch.cuda.empty_cache()
    decode = []
    for d in (64, 128):
        r = X.bench_decode(d, 4096)
        t = max_over_ranks(r["us_per_step"] * 1e-6)
        row = {"d": d, "batch_per_gpu": 64, "heads": heads, "steps": 4096, "us_per_step": t * 1e6,
               "tokens_per_s": world * 64 / t, "algorithmic_bytes_per_step_per_gpu": r["algorithmic_bytes_per_step"],
               "achieved_gbs_per_gpu": r["algorithmic_bytes_per_step"] / t / 1e9,
               "frac": r["algorithmic_bytes_per_step"] / t / 1e9 / peak, "cuda_graph": r["cuda_graph"],
               "us_per_step_python_launch": r["us_per_step_python_launch"]}
        if r.get("two_groups"):  # the batch as two independent chains of launches on two streams
            t2 = max_over_ranks(r["two_groups"]["us_per_step"] * 1e-6)
            row["two_groups"] = {"what": r["two_groups"]["what"], "us_per_step": t2 * 1e6, "tokens_per_s": world * 64 / t2,
                                 "frac": r["algorithmic_bytes_per_step"] / t2 / 1e9 / peak}
        if with_cpu and rank == 0:
            threads = os.cpu_count() or 1
            row["cpu_baseline"] = {"value": cpu_decode_sample(d, threads), "unit": "tokens/s", "cores": threads, "kind": "port",
                                   "sample": "200 tokens at batch 1, float64 state, the reference's per-token torch loop"}
        decode.append(row)
    # the bidirectional form at BERT-base attention shapes (B=32 per GPU, H=12, N=512, d=64): every rank its own batch
    rb = X.bench_bidir()
    tb = max_over_ranks((rb["fwd_kernel_us"] + rb["bwd_kernel_us"]) * 1e-6)
    ts = max_over_ranks(rb["us_per_step"] * 1e-6)
    bidir = {"what": "bidirectional cosine attention fwd+bwd, B=32 per GPU, H=12, N=512, d=64, bf16 (BERT-base attention shapes)",
             "scaling": "weak", "kernels_us": tb * 1e6, "fwd_kernel_us": rb["fwd_kernel_us"], "bwd_kernel_us": rb["bwd_kernel_us"],
             "kernels_frac": rb["algorithmic_bytes"] / tb / 1e9 / peak, "us_per_step_through_the_op": ts * 1e6,
             "tokens_per_s": world * 32 * 512 / ts, "algorithmic_bytes_per_gpu": rb["algorithmic_bytes"]}
    # whole-model training steps around the op (synthetic token ids, random weights; DDP over NCCL when world > 1)
    from cottention_transformer_b200 import bench_train as T
    train = [T.run_model(name, steps=4, warmup=2) for name in ("gpt", "bert")]
    return {"peak_gbs": peak, "peak_source": kind,
            "train": {"what": "whole-model bf16 training step with the op inside (GPT-style decoder 24 x 1024, 16 heads, seq 1024, "
                              "batch 8 per GPU; BERT-base encoder, seq 512, batch 32 per GPU), DDP gradient all-reduce over NCCL",
                      "scaling": "weak", "rows": train},
            "prefill_long": {"what": "causal fwd+bwd, B=1, H=16 heads split evenly over the GPUs (no collective), bf16; "
                                     "frac = algorithmic bytes / time / (GPUs x HBM peak)", "scaling": "strong",
                             "rows": prefill},
            "decode": {"what": "recurrent decode, one launch per token replayed from a CUDA graph, batch 64 per GPU, "
                               "bf16 tokens, fp32 state in HBM (8 state buffers in rotation: larger than L2 at d=128)",
                       "scaling": "weak", "rows": decode},
            "bidirectional": bidir}


def reference_cuda_kernel_sample(iters=3):
    """The reference's own CUDA extension (built unmodified into oracle/_ref by oracle/build_ref.py), when it is
    present and a GPU is visible: forward + the three backward scans of ``CustomAttention`` (Custom_Kernel.py:24,
    106-108) at the bench shape in bf16, kernel calls only (the module's elementwise PyTorch ops are not counted).
    Context for the CPU figure of this arm, which stays the arm's ``value``.  Returns a dict or None."""
    so = os.path.join(ROOT, "oracle", "_ref", "FastAttention2", "kernel.so")
    if not (os.path.exists(so) and torch.cuda.is_available()):
        return None
    import importlib.util
    spec = importlib.util.spec_from_file_location("kernel", so)  # the extension's init symbol is PyInit_kernel
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    g = torch.Generator(device=dev).manual_seed(1234)
    q, k, v, do = (torch.nn.functional.normalize(torch.randn(B_PER_GPU, H, N, D, device=dev, generator=g), dim=-1).bfloat16()
                   for _ in range(4))

    def step():
        ref.bfloat16(q, k, v, 1, False, False), ref.bfloat16(do, v, k, 1, False, False)
        ref.bfloat16(v, do, q, 1, False, True), ref.bfloat16(k, q, do, 1, False, True)

    step()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        step()
    e1.record()
    torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1) / iters
    return {"value": B_PER_GPU * N / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms,
            "what": "reference CUDA extension (oracle/_ref), CustomAttention forward + backward = four kernel calls, "
                    f"B={B_PER_GPU} H={H} N={N} d={D} bf16, one GPU, CUDA events"}


def run_reference_arm(args, rank, world):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    vals = []
    for i in range(args.warmup + args.steps):
        tps, slices, secs = cpu_reference_sample(threads, budget_s=4.0, max_slices=8)
        if i >= args.warmup:
            vals.append((tps, slices, secs))
    tps = sum(v[0] for v in vals) / len(vals)
    slices = vals[-1][1]
    ms = 1e3 * sum(v[2] for v in vals) / len(vals)
    line = {
        "impl": "reference", "metric": "causal cosine-attention fwd+bwd tokens/s", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_batch": B_PER_GPU * args.gpus, "seq_len": N, "heads": H, "head_dim": D},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": f"{slices} (batch,head) slices of N={N}, d={D} per step (after one untimed warm-up "
                                   "slice), fp32, PyTorch cumsum formulation + autograd"},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    gpu_ref = reference_cuda_kernel_sample()
    if gpu_ref is not None:
        line["reference_cuda_kernel"] = gpu_ref
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline leg (profiling runs)")
    ap.add_argument("--e2e-slices", type=int, default=8, help="batch slices of the pipelined host-buffer step")
    ap.add_argument("--e2e-no-graph", action="store_true", help="issue the host-buffer step call by call instead of replaying a CUDA graph")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary workloads (long prefill, decode)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch.distributed as dist
    from cottention_transformer_b200 import _lib
    from cottention_transformer_b200.host_step import CausalHostStep

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L = _lib.lib()
    numa = _bind_to_gpu_numa_node(local_rank)  # before any pinned allocation: first touch lands on the GPU's node
    host, nc_host = _host_inputs(rank)
    q, k, v, do = (t.to(dev) for t in host)
    nc = nc_host.to(dev)
    out, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
    dnc = torch.empty(H, dtype=torch.float32, device=dev)
    stream = _lib.stream_ptr(dev)
    P = lambda t: t.data_ptr()  # noqa: E731
    code = _lib.DTYPE_CODE[torch.bfloat16]

    def fwd():
        _lib.check(L.cott_cos_attn_fwd(P(q), P(k), P(v), P(nc), P(out), B_PER_GPU, H, N, D, D, code, stream), "fwd")

    def bwd_dq():
        _lib.check(L.cott_cos_attn_bwd_dq(P(q), P(k), P(v), P(nc), P(do), P(dq), B_PER_GPU, H, N, D, D, code, stream), "dq")

    def bwd_dkdv():
        _lib.check(L.cott_cos_attn_bwd_dkdv(P(q), P(k), P(v), P(nc), P(do), P(dk), P(dv), P(dnc), B_PER_GPU, H, N, D, D,
                                            code, stream), "dkdv")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing --------------------------------------------------------------------
    for _ in range(args.warmup):
        fwd(), bwd_dq(), bwd_dkdv()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(args.steps)]
    sampler = ClockSampler(local_rank)
    sampler.start()
    sampler.ready.wait(timeout=10)
    barrier()
    sampler.armed = True
    for i in range(args.steps):
        ev[i][0].record()
        fwd()
        ev[i][1].record()
        bwd_dq()
        ev[i][2].record()
        bwd_dkdv()
        ev[i][3].record()
    barrier()
    sampler.armed = False
    clocks = sampler.stop()
    _lib.check_device_status()
    total_ms = ev[0][0].elapsed_time(ev[-1][3])
    t_fwd = sum(e[0].elapsed_time(e[1]) for e in ev) / args.steps
    t_dq = sum(e[1].elapsed_time(e[2]) for e in ev) / args.steps
    t_kv = sum(e[2].elapsed_time(e[3]) for e in ev) / args.steps
    if world > 1:
        t = torch.tensor([total_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = t.item()
    ms_per_step = total_ms / args.steps
    tokens_per_step = B_PER_GPU * N * world
    value = tokens_per_step / (ms_per_step * 1e-3)

    # ---- end to end: pinned host buffers in, host buffers out ------------------------------------------
    host_out = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in (out, dq, dk, dv)]
    host_dnc = torch.empty(H, dtype=torch.float32).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host)
    d2h = sum(t.numel() * t.element_size() for t in host_out) + H * 4

    host_step = CausalHostStep(B_PER_GPU, H, N, D, torch.bfloat16, dev, slices=args.e2e_slices, graph=not args.e2e_no_graph)

    def e2e_step():
        host_dnc.copy_(host_step(*host, nc, *host_out), non_blocking=True)

    e2e_steps = max(3, min(args.steps, 10))
    e2e_value = None
    copy_ceiling = None
    if not args.no_e2e:
        # the floor of the host-buffer step on this host: the same bytes both ways at once, no kernels
        for _ in range(2):
            host_step.copy_only(host, host_out)
        barrier()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for _ in range(e2e_steps):
            host_step.copy_only(host, host_out)
        c1.record()
        barrier()
        copy_ms = c0.elapsed_time(c1)
        if world > 1:
            t = torch.tensor([copy_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            copy_ms = t.item()
        copy_s = copy_ms * 1e-3 / e2e_steps
        copy_ceiling = {"value": B_PER_GPU * N * world / copy_s, "unit": "tokens/s",
                        "h2d_gbs_per_gpu": h2d / copy_s / 1e9, "d2h_gbs_per_gpu": (d2h - H * 4) / copy_s / 1e9,
                        "what": "pinned cudaMemcpyAsync of the step's inputs and outputs, both directions at once, no kernels",
                        "numa": numa}
    if not args.no_e2e:
        for _ in range(2):
            e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e2e_steps):
            e2e_step()
        e1.record()
        barrier()
        e2e_ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([e2e_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = t.item()
        e2e_value = tokens_per_step * e2e_steps / (e2e_ms * 1e-3)

    extra = None if args.no_extra else run_extras(world, rank, dev, with_cpu=(world == 1 and not args.no_cpu_baseline))

    if rank == 0:
        peak, peak_kind = _peaks()
        per_launch = lambda passes: passes * B_PER_GPU * H * N * D * ELEM  # noqa: E731
        kv_bytes = per_launch(6)  # read q, k, v, dO; write dk, dv
        achieved = kv_bytes / (t_kv * 1e-3) / 1e9
        step_bytes = per_launch(11)  # 4 (fwd) + 7 (bwd) tensor passes
        step_gbs = step_bytes / ((t_fwd + t_dq + t_kv) * 1e-3) / 1e9
        line = {
            "metric": "causal cosine-attention fwd+bwd tokens/s", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "global_batch": B_PER_GPU * world, "seq_len": N, "heads": H,
                       "head_dim": D, "sharding": f"batch x heads, {B_PER_GPU * H} (b,h) sequences per GPU, no collective",
                       "l2": "inputs 268 MB + outputs 268 MB per step exceed the 126 MB L2"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "copy_ceiling": copy_ceiling},
            "gpu_launches": 3 * args.steps,
            "roofline": {"bound": "hbm", "kernel": "causal_bwd_kv_kernel", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "traffic": RECORDED_TRAFFIC_BYTES_PER_LAUNCH,
                         "traffic_source": "recorded: one ncu capture of this kernel at this shape (dram bytes read + "
                                           "written per launch), not measured by this run",
                         "peak_source": peak_kind, "algorithmic_bytes_per_launch": kv_bytes,
                         "kernel_us": {"causal_tc_kernel<fwd>": t_fwd * 1e3, "causal_tc_kernel<dq>": t_dq * 1e3,
                                       "causal_bwd_kv_kernel": t_kv * 1e3},
                         "step": {"algorithmic_bytes": step_bytes, "achieved": step_gbs, "frac": step_gbs / peak}},
        }
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            tps, slices, secs = cpu_reference_sample(threads, budget_s=12.0)
            line["cpu_baseline"] = {
                "value": tps, "unit": "tokens/s", "cores": threads, "kind": "port",
                "sample": f"{slices} of {B_PER_GPU * H} (batch,head) slices at N={N}, d={D}, fp32, PyTorch cumsum "
                          f"formulation + autograd, {secs:.1f} s (after one untimed warm-up slice)",
                "config1_forward_s": cpu_config1_forward(threads),
                "config1_forward_s_one_thread": cpu_config1_forward(1),
                "config1": "forward only, fp32, B=2 H=8 N=1024 d=64, the same formulation, whole"}
            torch.set_num_threads(threads)
        if extra is not None:
            line["extra"] = extra
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
