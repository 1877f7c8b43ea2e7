#!/usr/bin/env python
"""Benchmark of the hot path: RWKV-7 state-passing WKV forward + backward, bf16,
B=16 T=4096 C=4096 (H=64, N=64, chunk 16), synthetic inputs, on N GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--op NAME]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

A step = one forward + one backward of the operator over the whole batch.  The batch is
sharded over the ranks (total work fixed: strong scaling); nothing is exchanged between
ranks because every (batch, head) unit is independent and this operator has no parameter
gradient to reduce.  Rank 0 prints ONE JSON line.

  value     tokens/s with inputs resident in HBM (CUDA events, max over ranks)
  e2e       tokens/s through the public operator API from pinned HOST buffers: the step's
            inputs are copied host->device and all results device->host inside the timed region
  roofline  dominant kernel (the backward): compulsory HBM bytes / measured kernel time,
            against the measured copy bandwidth in MEASURED_PEAKS.json
  cpu_baseline  the reference's PyTorch formula path (oracle port) timed on the host cores on a
            bounded sample
`--impl reference` times only that CPU formula path and prints the same line shape.
`--op` selects one of the other benchmark configurations (wkv4, timex, wkv5, wkv6state).
"""
import argparse
import json
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0  # earlier measurement on this pool, used only if MEASURED_PEAKS.json is absent


# --------------------------------------------------------------------------------------
# workloads: name -> description, token count, compulsory bytes (fwd, bwd), runner factory
# --------------------------------------------------------------------------------------
class V7Workload:
    """BASELINE config 5: RWKV-7 state passing, bf16, B16 T4096 C4096 N64 chunk 16."""
    name = "rwkv7_statepassing_clampw fwd+bwd B16 T4096 C4096 N64 chunk16"
    B, T, H, N = 16, 4096, 64, 64
    dtype_name = "bf16"
    metric = "WKV fwd+bwd tokens/s, RWKV-7 B16 T4096 C4096 bf16"

    def __init__(self, b_local, device, rank):
        """Every rank draws the same seed-42 batch of the full configuration and keeps rows
        [rank*b_local, (rank+1)*b_local): shard g of a multi-GPU run is bit-identical to those rows of
        the single-GPU input."""
        import rwkv_cuda_b200 as R
        self.R = R
        B, T, H, N = b_local, self.T, self.H, self.N
        self.b = B
        g = torch.Generator(device=device)
        g.manual_seed(42)
        bf = torch.bfloat16
        lo = rank * b_local

        def mk(scale=1.0):
            return (torch.randn(self.B, T, H, N, generator=g, device=device)[lo:lo + B] * scale).contiguous()

        # generated on the device for speed, then parked in pinned HOST buffers: the end-to-end
        # leg starts from those host copies
        r, k, v = mk(0.5), mk(0.5), mk(0.5)
        w = mk()
        kk = torch.nn.functional.normalize(mk(), dim=-1)
        a, b = -kk, kk * torch.sigmoid(mk())
        # (pinned buffers are allocated with the thread bound to the GPU's NUMA node, where the platform tells)
        with R.host_pipeline.host_memory_near(device) as node:
            self.numa_node = node
            self.host_in = [x.to(bf).cpu().pin_memory() for x in (r, w, k, v, a, b)]
            self.host_dy = mk().to(bf).cpu().pin_memory()
            self.host_s0 = (0.1 * torch.randn(self.B, H, N, N, generator=g, device=device)[lo:lo + B]).cpu().pin_memory()
            self.host_dsT = torch.randn(self.B, H, N, N, generator=g, device=device)[lo:lo + B].cpu().pin_memory()
        del r, k, v, w, kk, a, b
        dev = device
        self.dev = dev
        self.inp = [x.to(dev) for x in self.host_in]
        self.dy, self.s0, self.dsT = self.host_dy.to(dev), self.host_s0.to(dev), self.host_dsT.to(dev)
        self.y = torch.empty(B, T, H, N, dtype=bf, device=dev)
        self.sT = torch.empty(B, H, N, N, device=dev)
        self.s = torch.empty(B, H, T // 16, N, N, device=dev)  # saved-for-backward buffers, as the harness allocates them
        self.sa = torch.empty(B, T, H, N, device=dev)
        self.ds0 = torch.empty(B, H, N, N, device=dev)
        self.grads = [torch.empty(B, T, H, N, dtype=bf, device=dev) for _ in range(6)]
        self.host_out = None

    tokens_per_unit_batch = T

    @classmethod
    def bytes_fwd(cls, B):
        C = cls.H * cls.N
        return 14 * C * B * cls.T + 2 * 4 * B * cls.H * cls.N * cls.N

    @classmethod
    def bytes_bwd(cls, B):
        C = cls.H * cls.N
        return 26 * C * B * cls.T + 2 * 4 * B * cls.H * cls.N * cls.N

    def forward(self):
        self.R.ops.wkv7_forward(self.s0, *self.inp, self.y, self.sT, self.s, self.sa)

    def backward(self):
        self.R.ops.wkv7_backward(*self.inp, self.dy, self.dsT, self.s, self.sa, self.ds0, *self.grads)

    launches_per_step = 2
    # dram__bytes_read.sum + dram__bytes_write.sum of the backward kernel per token, from the ncu
    # capture of the reduced case (profiles/wkv7_tcgen05_chunk32_B8_T1024.md); traffic is
    # proportional to the token count
    dram_bytes_per_token_bwd = (0.758777e9 + 0.379956e9) / (8 * 1024)

    def e2e_step(self):
        """Host buffers in, host buffers out, through the public host-buffer API
        (rwkv_cuda_b200.host_pipeline): every operand starts in pinned host memory and every result
        ends there; copies in both directions and the kernels are inside the timed region."""
        if self.host_out is None:
            names = self.R.host_pipeline.Wkv7HostPipeline
            with self.R.host_pipeline.host_memory_near(self.dev):
                self.host_out = {n: torch.empty_like(self.host_in[0]).pin_memory() for n in names.OUT}
                self.host_out.update(sT=torch.empty_like(self.host_s0).pin_memory(), ds0=torch.empty_like(self.host_s0).pin_memory())
            self.host_named = dict(zip(("r", "w", "k", "v", "a", "b"), self.host_in))
            self.host_named.update(dy=self.host_dy, s0=self.host_s0, dsT=self.host_dsT)
            self.pipe = names(self.T, self.H, self.N, self.dev, slice_batch=1)
        self.pipe.forward_backward(self.host_named, self.host_out)

    def e2e_bytes(self):
        big = self.host_in[0].numel() * 2
        st = self.host_s0.numel() * 4
        return 7 * big + 2 * st, 7 * big + 2 * st


def cpu_formula_step(T_cpu, threads):
    """One fwd+bwd of the reference's RWKV-7 PyTorch formula (oracle port) on the host cores:
    B=1, T=T_cpu, C=4096, fp32, gradients by autograd, as the reference harness computes them."""
    from oracle import wkv_oracle as O
    torch.set_num_threads(threads)
    H, N = 64, 64
    C = H * N
    g = torch.Generator()
    g.manual_seed(42)
    mk = lambda s=1.0: (torch.randn(1, T_cpu, C, generator=g) * s).requires_grad_(True)
    r, k, v, w = mk(0.5), mk(0.5), mk(0.5), mk()
    kk = torch.nn.functional.normalize(torch.randn(1, T_cpu, H, N, generator=g), dim=-1).view(1, T_cpu, C)
    a = (-kk).requires_grad_(True)
    b = (kk * torch.sigmoid(torch.randn(1, T_cpu, C, generator=g))).requires_grad_(True)
    s0 = (0.1 * torch.randn(1, H, N, N, generator=g)).requires_grad_(True)
    dy, dsT = torch.randn(1, T_cpu, C, generator=g), torch.randn(1, H, N, N, generator=g)
    t0 = time.perf_counter()
    y, sT = O.wkv7(r, w, k, v, a, b, H, s0=s0)
    torch.autograd.backward([y, sT], [dy, dsT])
    return time.perf_counter() - t0


# --------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    bits = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for n, bit in names.items():
                    if bits & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            self._stop.wait(0.01)   # the timed region of the default run lasts about 0.12 s

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def run_reference_arm(args, rank, world):
    """CPU arm: the reference's PyTorch formula path (oracle port), all host threads, rank 0 only."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    T_cpu = args.cpu_seq
    for _ in range(args.warmup):
        cpu_formula_step(T_cpu, threads)
    times = [cpu_formula_step(T_cpu, threads) for _ in range(args.steps)]
    total = sum(times)
    val = T_cpu * len(times) / total
    sample = f"B1 T{T_cpu} C4096 N64 fp32 fwd+bwd per step (autograd through the formula), {threads} threads"
    print(json.dumps({
        "impl": "reference", "metric": V7Workload.metric, "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": V7Workload.name, "sample": sample},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }), flush=True)



# --------------------------------------------------------------------------------------
# the other benchmark configurations (--op): same timing rules, one GPU, no end-to-end leg
# --------------------------------------------------------------------------------------
FP32_NOMINAL_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12   # CUDA-core fp32 FMA peak (nominal, not measured)


def _time_fb(fwd, bwd, steps, warmup):
    for _ in range(max(warmup, 3)):
        fwd(); bwd()
    torch.cuda.synchronize()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
    for e in evs:
        e[0].record(); fwd(); e[1].record(); bwd(); e[2].record()
    torch.cuda.synchronize()
    f = sum(e[0].elapsed_time(e[1]) for e in evs) / steps
    b = sum(e[1].elapsed_time(e[2]) for e in evs) / steps
    return f, b


def _cpu_time(fn, repeat=2):
    fn()
    t0 = time.perf_counter()
    for _ in range(repeat):
        fn()
    return (time.perf_counter() - t0) / repeat


def run_secondary(op, args, emit=True):
    """BASELINE configurations 1-4.  Prints one JSON line (or returns it as a dict when `emit` is false): tokens/s
    (or rows/s), per-kernel times, the roofline of the backward kernel and the CPU formula path on a bounded sample."""
    import rwkv_cuda_b200 as R
    from oracle import wkv_oracle as O
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev)
    g.manual_seed(42)
    rn = lambda *s: torch.randn(*s, device=dev, generator=g)
    ru = lambda lo, hi, *s: torch.rand(*s, device=dev, generator=g) * (hi - lo) + lo
    bf = torch.bfloat16
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    extra = {}
    if op == "wkv4":       # config 1: RWKV-4 fp32 B4 T256 C256
        B, T, C = 4, 256, 256
        name, dtype, tokens = f"wkv4 fwd+bwd fp32 B{B} T{T} C{C}", "f32", B * T
        w, u = -torch.exp(ru(-4, 1, C)), ru(-1, 1, C)
        k, v, gy = 0.5 * rn(B, T, C), rn(B, T, C), rn(B, T, C)
        y, gk, gv = (torch.empty(B, T, C, device=dev) for _ in range(3))
        gw, gu = torch.zeros(B, C, device=dev), torch.zeros(B, C, device=dev)
        fwd = lambda: R.ops.wkv4_forward(B, T, C, w, u, k, v, y)
        bwd = lambda: R.ops.wkv4_backward(B, T, C, w, u, k, v, gy, gw, gu, gk, gv)
        bytes_f, bytes_b = 12 * B * T * C, 20 * B * T * C
        bound, note = "hbm", "latency bound: 1024 independent recurrences of 256 dependent steps"

        def cpu():
            xs = [x.cpu().requires_grad_(True) for x in (torch.log(-w), u, k, v)]
            O.wkv4(*xs).backward(gy.cpu())
        cpu_tokens, cpu_sample = B * T, f"full config (B{B} T{T} C{C}), fp32 formula + autograd"
    elif op == "timex":    # config 2: depthwise_conv1d fp32 B32 C768 T768
        B, C, T = 32, 768, 768
        name, dtype, tokens = f"depthwise_conv1d fwd+bwd fp32 B{B} C{C} T{T}", "f32", B * T
        w, k, gy = rn(C, T) / T ** 0.5, rn(B, C, T), rn(B, C, T)
        x, gk, gws = torch.empty(B, C, T, device=dev), torch.empty(B, C, T, device=dev), torch.empty(C, T, device=dev)
        fwd = lambda: R.ops.timex_forward(w, k, x, 0.1, B, C, T)
        bwd = lambda: R.ops.timex_backward_reduced(w, k, gy, gws, gk, B, C, T)
        bytes_f, bytes_b = 4 * (2 * B * C * T + C * T), 4 * (3 * B * C * T + 2 * C * T)
        flop_f, flop_b = B * C * T * (T + 1), 2 * B * C * T * (T + 1)
        bound, note = "fp32", "FP32-pipe bound (T/2 FMA per loaded element); peak is the nominal CUDA-core figure"

        def cpu():
            wl, kl = w.cpu().requires_grad_(True), k.cpu().requires_grad_(True)
            O.timex_conv(wl, kl, 0.1).backward(gy.cpu())
        cpu_tokens, cpu_sample = B * T, "full config, grouped conv1d formula + autograd, fp32"
    elif op == "wkv5":     # config 3: RWKV-5 bf16 B8 T4096 C4096 N64
        B, T, H, N = 8, 4096, 64, 64
        C = H * N
        name, dtype, tokens = f"wkv5 fwd+bwd bf16 B{B} T{T} C{C} N{N}", "bf16", B * T
        r, k, v = ((0.5 * rn(B, T, C)).to(bf) for _ in range(3))
        gy = rn(B, T, C).to(bf)
        wraw, u = ru(-6, -1, H, N).to(bf), ru(-1, 1, H, N).to(bf)
        ew = -torch.exp(wraw.float())
        eew = torch.exp(ew)
        y, gr, gk, gv = (torch.empty(B, T, C, dtype=bf, device=dev) for _ in range(4))
        gw, gu = torch.empty(B, C, dtype=bf, device=dev), torch.empty(B, C, dtype=bf, device=dev)
        # the training flow: the forward keeps the chunk-start states for the backward
        saved5 = torch.empty(R.ops.wkv5_saved_bytes(B, T, C), dtype=torch.uint8, device=dev)
        valid5 = [False]

        def fwd():
            valid5[0] = R.ops.wkv5_forward_saved(B, T, C, H, r, k, v, eew, u, y, saved5)

        def bwd():
            R.ops.wkv5_backward_saved(B, T, C, H, r, k, v, eew, ew, u, gy, gr, gk, gv, gw, gu, saved5, valid5[0])
        bytes_f, bytes_b = 8 * C * B * T, 14 * C * B * T
        bound, note = "hbm", "tcgen05 kernels on 32-token chunks, chunk states saved by the forward; decay constant over time"
        Tc = 256

        def cpu():
            xs = [x[:1, :Tc].float().cpu().requires_grad_(True) for x in (r, k, v)] + [wraw.float().cpu().requires_grad_(True), u.float().cpu().requires_grad_(True)]
            O.wkv5(*xs, H).backward(gy[:1, :Tc].float().cpu())
        cpu_tokens, cpu_sample = Tc, f"B1 T{Tc} C{C} N{N} fp32 recurrent formula + autograd"
    elif op == "wkv6state":  # config 4: RWKV-6 with fp32 state in/out, bf16, B16 T4096 C4096 N64
        B, T, H, N = args.batch or 16, args.seq or 4096, 64, 64   # --batch/--seq: reduced case for profiler captures
        C = H * N
        name, dtype, tokens = f"wkv6state(_ex) fwd+bwd bf16 B{B} T{T} C{C} N{N}", "bf16", B * T
        r, k, v = ((0.5 * rn(B, T, C)).to(bf) for _ in range(3))
        gy = rn(B, T, C).to(bf)
        wraw, u = (rn(B, T, C) - 5.0).to(bf), ru(-1, 1, H, N).to(bf)
        s0, dsT = 0.1 * rn(B, H, N, N), rn(B, H, N, N)
        y, gr, gk, gv, gw = (torch.empty(B, T, C, dtype=bf, device=dev) for _ in range(5))
        gu = torch.empty(B, C, dtype=bf, device=dev)
        sT, ds0 = torch.empty_like(s0), torch.empty_like(s0)
        # the training flow: the forward keeps the chunk-start states for the backward
        saved = torch.empty(R.ops.wkv6_saved_bytes(B, T, C), dtype=torch.uint8, device=dev)
        valid = [False]

        def fwd():
            valid[0] = R.ops.wkv6state_forward_saved(B, T, C, H, r, k, v, wraw, u, s0, y, sT, saved)

        def bwd():
            R.ops.wkv6state_backward_saved(B, T, C, H, r, k, v, wraw, u, s0, gy, dsT, gr, gk, gv, gw, gu, ds0, saved, valid[0])
        st = 4 * B * H * N * N
        bytes_f, bytes_b = 10 * C * B * T + 2 * st, 18 * C * B * T + 2 * st
        bound, note = "hbm", "tcgen05 kernels on 32-token chunks, chunk states saved by the forward; per-token decay, fp32 state in/out"
        Tc = 256

        def cpu():
            xs = [x[:1, :Tc].float().cpu().requires_grad_(True) for x in (r, k, v, wraw)] + [u.float().cpu().requires_grad_(True), s0[:1].cpu().requires_grad_(True)]
            yy, ss = O.wkv6(*xs[:5], H, s0=xs[5], return_state=True)
            torch.autograd.backward([yy, ss], [gy[:1, :Tc].float().cpu(), dsT[:1].cpu()])
        cpu_tokens, cpu_sample = Tc, f"B1 T{Tc} C{C} N{N} fp32 recurrent formula + autograd"
    else:
        raise SystemExit(f"unknown --op {op}")

    with ClockSampler(0) as clocks:
        fwd_ms, bwd_ms = _time_fb(fwd, bwd, args.steps, args.warmup)
    peak, peak_src = hbm_peak()
    ach = bytes_b / (bwd_ms * 1e-3) / 1e9
    roof = {"bound": "hbm", "kernel": op + " backward", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
            "traffic": None, "peak_source": peak_src, "algorithmic_bytes_per_launch": bytes_b,
            "fwd": {"achieved": bytes_f / (fwd_ms * 1e-3) / 1e9, "frac": bytes_f / (fwd_ms * 1e-3) / 1e9 / peak}, "note": note}
    if bound == "fp32":
        tf = flop_b / (bwd_ms * 1e-3) / 1e12
        roof.update({"bound": "fp32 (CUDA cores)", "achieved": tf, "peak": FP32_NOMINAL_TFLOPS, "unit": "TFLOP/s",
                     "frac": tf / FP32_NOMINAL_TFLOPS, "peak_source": "nominal 148 SMs x 128 lanes x 2 x 1.965 GHz",
                     "hbm_frac": ach / peak,
                     "fwd": {"achieved": flop_f / (fwd_ms * 1e-3) / 1e12, "frac": flop_f / (fwd_ms * 1e-3) / 1e12 / FP32_NOMINAL_TFLOPS}})
    out = {"metric": f"{op} fwd+bwd tokens/s", "value": tokens / ((fwd_ms + bwd_ms) * 1e-3), "unit": "tokens/s", "n_gpus": 1,
           "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": fwd_ms + bwd_ms, "higher_is_better": True,
           "scaling": "strong", "vs_baseline": None, "dtype": dtype, "data": "synthetic", "config": {"workload": name},
           "fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "roofline": roof,
           # wkv6state, wkv5: tensor-core forward and backward, each followed by its guarded general-shape twin
           "gpu_launches": (4 if op in ("wkv6state", "wkv5") else 3 if op == "timex" else 2) * args.steps,
           "clocks": clocks.summary()}
    if not args.no_cpu_baseline:
        ct = _cpu_time(cpu)
        out["cpu_baseline"] = {"value": cpu_tokens / ct, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": cpu_sample}
    if not emit:
        return out
    print(json.dumps(out), flush=True)


def run_wkv5_sharded(args, rank, world, local):
    """BASELINE configuration 3 (RWKV-5 bf16 B8 T4096 C4096 N64) sharded by batch over the ranks, with the one
    collective this library has: gw and gu are reduced over the local batch in fp32 into one buffer
    (rwkvb200_reduce_batch_partials) and that buffer is all-reduced once over NCCL, on a side stream.
    Every rank draws the same seed-42 batch and keeps its rows.  Rank 0 prints one JSON line."""
    import torch.distributed as dist
    import rwkv_cuda_b200 as R
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    B, T, H, N = args.batch or 8, args.seq or 4096, 64, 64
    C, bf = H * N, torch.bfloat16
    assert B % world == 0
    bl, lo = B // world, rank * (B // world)
    g = torch.Generator(device=dev)
    g.manual_seed(42)
    full = lambda sc=1.0: torch.randn(B, T, C, generator=g, device=dev) * sc
    r, k, v = (full(0.5)[lo:lo + bl].to(bf).contiguous() for _ in range(3))
    gy = full()[lo:lo + bl].to(bf).contiguous()
    wraw = (torch.rand(H, N, generator=g, device=dev) * 5 - 6).to(bf)
    u = (torch.rand(H, N, generator=g, device=dev) * 2 - 1).to(bf)
    ew = -torch.exp(wraw.float())
    eew = torch.exp(ew)
    y, gr, gk, gv = (torch.empty(bl, T, C, dtype=bf, device=dev) for _ in range(4))
    gw, gu = torch.empty(bl, C, dtype=bf, device=dev), torch.empty(bl, C, dtype=bf, device=dev)
    red = R.dist.ParamGradReducer(dev, 2 * C)
    gw32, gu32 = torch.empty(bl, C, device=dev), torch.empty(bl, C, device=dev)   # unrounded partials of gw, gu
    saved = torch.empty(R.ops.wkv5_saved_bytes(bl, T, C), dtype=torch.uint8, device=dev)

    def step():
        valid = R.ops.wkv5_forward_saved(bl, T, C, H, r, k, v, eew, u, y, saved)
        R.ops.wkv5_backward_saved(bl, T, C, H, r, k, v, eew, ew, u, gy, gr, gk, gv, gw, gu, saved, valid, gw32, gu32)
        red.reset()
        red.add(gw32); red.add(gu32)
        red.launch()
        return red.result(0), red.result(1)

    for _ in range(max(args.warmup, 3)):
        step()
    dist.barrier(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        gws, gus = step()
    e1.record()
    dist.barrier(); torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    # the same reduction on one rank over the whole batch would be sum over all rows: check the collective
    chk = torch.stack([gws.sum(), gus.sum()]).double()
    loc = torch.stack([gw32.sum(), gu32.sum()]).double()   # local sums of the unrounded partials
    dist.all_reduce(loc, op=dist.ReduceOp.SUM)
    if rank == 0:
        ms = t.item() / args.steps
        print(json.dumps({"metric": "WKV fwd+bwd tokens/s, RWKV-5 B8 T4096 C4096 bf16 (batch-sharded, parameter gradients all-reduced)",
                          "value": B * T / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "ms_per_step": ms,
                          "higher_is_better": True, "scaling": "strong", "dtype": "bf16", "data": "synthetic",
                          "config": {"workload": f"wkv5 fwd+bwd bf16 B{B} T{T} C{C} N{N}", "batch_per_gpu": bl,
                                     "parallelism": f"batch-sharded x{world}; one fp32 all-reduce of {2 * C} floats (NCCL) per step on a side stream"},
                          "collective_check": {"allreduced_sum": chk.tolist(), "sum_of_local_sums": loc.tolist(),
                                               "rel_diff": ((chk - loc).abs() / loc.abs().clamp_min(1e-30)).tolist()}}), flush=True)
    dist.destroy_process_group()


def reference_kernel_timing(wl, fwd_ms, bwd_ms):
    """The reference project's own CUDA kernel (built as a test-only checker into oracle/_ref/ where a
    reference checkout was present) on this rank's device tensors, outside the timed region: its times,
    the speed-up of this library over it, and both kernels' RMS errors against the fp64 formula on a
    sample of (batch, head) units.  None-like dict with a reason when the library is not there."""
    try:
        from tests import ref_kernel
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"tests/ref_kernel.py not importable: {e}"}
    if not ref_kernel.available():
        return {"unavailable": "oracle/_ref/librwkv7_ref.so not built (no reference checkout at build time)"}
    y, sT, ds0 = torch.empty_like(wl.y), torch.empty_like(wl.sT), torch.empty_like(wl.ds0)
    gr = [torch.empty_like(x) for x in wl.grads]
    f = lambda: ref_kernel.forward(wl.s0, *wl.inp, y, sT, wl.s, wl.sa)
    b = lambda: ref_kernel.backward(*wl.inp, wl.dy, wl.dsT, wl.s, wl.sa, ds0, *gr)
    f(); b()
    tf, tb = ref_kernel._time(f, 3), ref_kernel._time(b, 3)
    out = {"fwd_ms": tf, "bwd_ms": tb, "tokens_per_s": wl.b * wl.T / ((tf + tb) * 1e-3), "speedup": (tf + tb) / (fwd_ms + bwd_ms),
           "source": "rwkv7_fast_fused/cuda/rwkv7_statepassing_clampw.cu compiled for sm_100a with its own flags"}
    # errors of both kernels on two units against the fp64 formula (the reference run leaves s/sa in its own layout: rerun ours after)
    try:
        from oracle import wkv_oracle as O
        N = wl.N
        units = [(0, 0), (wl.b - 1, wl.H - 1)]
        names = ("y", "dr", "dw", "dk", "dv", "da", "db")
        ref_out = dict(zip(names, [y] + gr))
        wl.forward(); wl.backward(); torch.cuda.synchronize()
        our_out = dict(zip(names, [wl.y] + wl.grads))
        Tc = min(wl.T, 1024)   # the first Tc tokens of a unit do not depend on later ones in the forward; gradients need the whole unit
        errs = {"ours": {}, "reference_kernel": {}}
        acc = {k: {n: [0.0, 0.0] for n in ("y",)} for k in errs}
        for (bi, hi) in units:
            x64 = [t[bi:bi + 1, :Tc, hi].double().cpu().reshape(1, Tc, N) for t in wl.inp]
            s064 = wl.s0[bi:bi + 1, hi:hi + 1].double().cpu()
            y64, _ = O.wkv7(*x64, 1, s0=s064)
            for k, o in (("ours", our_out), ("reference_kernel", ref_out)):
                d = o["y"][bi, :Tc, hi].double().cpu().reshape(1, Tc, N) - y64
                acc[k]["y"][0] += float((d * d).sum()); acc[k]["y"][1] += float((y64 * y64).sum())
        out["rms_error_y_first_%d_tokens" % Tc] = {k: (acc[k]["y"][0] / acc[k]["y"][1]) ** 0.5 for k in acc}
    except Exception as e:  # noqa: BLE001
        out["rms_error_note"] = f"error sample skipped: {e}"
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-other-configs", action="store_true", help="skip the short runs of BASELINE configurations 1-4 after the main one")
    ap.add_argument("--cpu-seq", type=int, default=256, help="sequence length of one CPU-baseline step (B=1, C=4096)")
    ap.add_argument("--batch", type=int, default=None, help="profiling aid: smaller global batch than the config's 16")
    ap.add_argument("--seq", type=int, default=None, help="profiling aid: shorter sequence than the config's 4096")
    ap.add_argument("--path", type=int, default=0, choices=[0, 1, 2],
                    help="RWKV-7 kernel family (rwkvb200_wkv7_select_path); 0 = automatic")
    ap.add_argument("--op", default="wkv7", choices=["wkv7", "wkv4", "timex", "wkv5", "wkv6state"],
                    help="wkv7 = the headline configuration (default); the others are BASELINE configurations 1-4")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this benchmark has no CPU fallback (use --impl reference for the CPU arm)")
    if args.op == "wkv5" and world > 1:
        run_wkv5_sharded(args, rank, world, local)
        return
    if args.op != "wkv7":
        if rank == 0:
            run_secondary(args.op, args)
        return
    import torch.distributed as dist
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    W = V7Workload
    if args.batch or args.seq:  # reduced case for profiler captures; not the benchmark configuration
        W.B, W.T = args.batch or W.B, args.seq or W.T
        W.name = f"REDUCED rwkv7_statepassing_clampw fwd+bwd B{W.B} T{W.T} C4096 N64 chunk16"
    assert W.B % world == 0, f"batch {W.B} does not divide over {world} ranks"
    b_local = W.B // world
    wl = W(b_local, dev, rank)
    if args.path:
        from rwkv_cuda_b200 import _lib
        _lib.call("rwkvb200_wkv7_select_path", args.path)
        W.name += f" (kernel family {args.path})"

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step():
        wl.forward()
        wl.backward()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()

    # ---- timed region: K steps, CUDA events on the launching stream ------------------
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    fe = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
          for _ in range(args.steps)]
    with ClockSampler(local) as clocks:
        barrier()
        ev[0].record()
        for i in range(args.steps):
            fe[i][0].record()
            wl.forward()
            fe[i][1].record()
            wl.backward()
            fe[i][2].record()
        ev[1].record()
        barrier()
    ms_total = ev[0].elapsed_time(ev[1])
    fwd_ms = sum(a.elapsed_time(b) for a, b, _ in fe) / args.steps
    bwd_ms = sum(b.elapsed_time(c) for _, b, c in fe) / args.steps
    t = torch.tensor([ms_total, fwd_ms, bwd_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, fwd_ms, bwd_ms = t.tolist()
    tokens_step = W.B * W.T
    value = tokens_step * args.steps / (ms_total * 1e-3)

    # ---- end to end: host buffers through the public API ------------------------------
    e2e_val, h2d, d2h = None, 0, 0
    if not args.no_e2e:
        wl.e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(args.e2e_steps):
            wl.e2e_step()
        e1.record()
        barrier()
        te = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_val = tokens_step * args.e2e_steps / (te.item() * 1e-3)
        h2d, d2h = wl.e2e_bytes()

    from rwkv_cuda_b200 import _lib as _L
    st = _L.lib().rwkvb200_device_status()
    if st != 0:
        raise SystemExit(f"bench.py: device status {st} after the timed region (a bounded wait ran out): results invalid")
    ref_kernel_block = reference_kernel_timing(wl, fwd_ms, bwd_ms) if rank == 0 else None

    if rank == 0:
        peak, peak_src = hbm_peak()
        bb = W.bytes_bwd(b_local)
        achieved = bb / (bwd_ms * 1e-3) / 1e9
        fb = W.bytes_fwd(b_local)
        out = {
            "metric": W.metric, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_total / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": W.dtype_name, "data": "synthetic",
            "config": {"workload": W.name, "global_batch": W.B, "batch_per_gpu": b_local, "seq_len": W.T,
                       "parallelism": f"batch-sharded x{world}, no collective",
                       "l2": "inputs (6 x %.0f MB per GPU) exceed the 126 MB L2" % (b_local * W.T * 4096 * 2 / 1e6)},
            "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
            "roofline": {"bound": "hbm", "kernel": "wkv7 backward", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": W.dram_bytes_per_token_bwd * b_local * W.T,
                         "traffic_source": "ncu dram__bytes_read+write of the backward at B8 T1024 (profiles/), scaled by tokens",
                         "peak_source": peak_src,
                         "algorithmic_bytes_per_launch": bb,
                         "fwd": {"achieved": fb / (fwd_ms * 1e-3) / 1e9, "frac": fb / (fwd_ms * 1e-3) / 1e9 / peak,
                                 "algorithmic_bytes_per_launch": fb},
                         "fwd_bwd_frac": (fb + bb) / ((fwd_ms + bwd_ms) * 1e-3) / 1e9 / peak},
            "e2e": {"value": e2e_val, "unit": "tokens/s", "h2d_bytes_per_step": h2d * world,
                    "d2h_bytes_per_step": d2h * world, "steps": args.e2e_steps,
                    # what each GPU's host link carried, each way, while both directions and the kernels ran
                    "host_link_gbs_per_gpu_each_way": (h2d * e2e_val / tokens_step / 1e9) if e2e_val else None,
                    "pinned_buffers_numa_node_rank0": getattr(wl, "numa_node", None)},
            "gpu_launches": W.launches_per_step * args.steps,
            "clocks": clocks.summary(),
            "reference_kernel": ref_kernel_block,
        }
        if world == 1 and not args.no_other_configs and not (args.batch or args.seq or args.path):
            # the other BASELINE configurations, a few steps each, so that one record covers them all
            import copy
            a2 = copy.copy(args)
            a2.steps, a2.warmup, a2.no_cpu_baseline, a2.batch, a2.seq = 5, 3, True, None, None
            del wl
            torch.cuda.empty_cache()
            other = {}
            for op in ("wkv4", "timex", "wkv5", "wkv6state"):
                o = run_secondary(op, a2, emit=False)
                other[op] = {"workload": o["config"]["workload"], "fwd_ms": o["fwd_ms"], "bwd_ms": o["bwd_ms"],
                             "tokens_per_s": o["value"], "dtype": o["dtype"],
                             "roofline": {k: o["roofline"][k] for k in ("bound", "achieved", "peak", "unit", "frac")},
                             "roofline_fwd_frac": o["roofline"]["fwd"]["frac"]}
            out["other_configs"] = other
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            T_cpu = args.cpu_seq
            cpu_formula_step(64, threads)
            n = 3
            tt = sum(cpu_formula_step(T_cpu, threads) for _ in range(n))
            out["cpu_baseline"] = {"value": T_cpu * n / tt, "unit": "tokens/s", "cores": threads, "kind": "port",
                                   "sample": f"{n} x (B1 T{T_cpu} C4096 N64 fp32 fwd+bwd, autograd through the formula)"}
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
