#!/usr/bin/env python
"""Benchmark of the data-parallel training hot path (forward + backward + gradient mean-allreduce + Adam).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the configuration the headline metric is quoted on at 1/2/4/8 GPUs): an 8-block MLP, each block
LayerNorm(4096) -> Dense(4096=>4096, gelu), then Dense(4096=>1000); Float32; synthetic input ~N(0,1) at global
batch 8192 split over the ranks in contiguous column blocks; random integer labels 1..1000; logitcrossentropy;
Adam(1e-3); gradients averaged over the ranks with NCCL.  One "step" = one training step on one global batch.
Prints ONE JSON line (rank 0).  `value` is device-timed with the batch resident in HBM; `e2e` runs the same
public call (`fluxb200.trainstep`) with the batch coming from pinned host memory every step.

`--impl reference` times the CPU restatement of Flux's path (oracle/, numpy Float32 on all host cores) on a
bounded sample of the same workload; Flux itself needs Julia, which this machine does not have.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "flux.jl_b200"))

D, NBLOCKS, NCLASS, GLOBAL_BATCH = 4096, 8, 1000, 8192
METRIC = "fwd+bwd samples/sec (device-timed)"
WORKLOAD = "dp_mlp: 8x[LayerNorm(4096)+Dense(4096=>4096,gelu)]+Dense(4096=>1000), Float32, global batch 8192, logitcrossentropy+Adam"
FLOPS_PER_SAMPLE = 6 * (NBLOCKS * D * D + D * NCLASS)


def make_params(seed=3):
    """Glorot-uniform weights (src/utils.jl:81-86), zero biases, gamma = 1, beta = 0."""
    rng = np.random.default_rng(seed)

    def glorot(o, i):
        return ((rng.random((o, i), dtype=np.float32) - np.float32(0.5)) * np.float32(np.sqrt(24.0 / (o + i)))).astype(np.float32)

    blocks = [{"gamma": np.ones(D, np.float32), "beta": np.zeros(D, np.float32), "W": glorot(D, D), "b": np.zeros(D, np.float32)}
              for _ in range(NBLOCKS)]
    head = {"W": glorot(NCLASS, D), "b": np.zeros(NCLASS, np.float32)}
    return blocks, head


# ------------------------------------------------------------------------------------- clocks ---
class ClockSampler:
    """Samples SM clock and clock-event reasons of one GPU while the timed region runs: NVML reads every 5 ms from a
    thread (a timed region can be shorter than one nvidia-smi period); nvidia-smi -lms 100 when NVML is missing."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = (("sw_power_cap", 0x4), ("hw_slowdown", 0x8), ("sw_thermal_slowdown", 0x20), ("hw_thermal_slowdown", 0x40))

    def __init__(self, gpu_index):
        self.proc = None
        self.lines = []
        self.samples = []          # (sm_mhz, reasons bitmask) from NVML
        self.max_mhz = None
        self.stop_flag = threading.Event()
        self.nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            try:
                import torch
                pr = torch.cuda.get_device_properties(gpu_index)
                bus = "%08x:%02x:%02x.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
                self.handle = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _poll(self):
        nv = self.nvml
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self.stop_flag.is_set():
            try:
                self.samples.append((float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)), int(get_reasons(self.handle))))
            except Exception:
                pass
            time.sleep(0.005)

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.nvml is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            sm = [a for a, _ in self.samples]
            mask = 0
            for _, r in self.samples:
                mask |= r
            reasons = sorted(name for name, bit in self.REASON_BITS if mask & bit)
            return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": self.max_mhz, "reasons": reasons,
                    "samples": len(sm), "source": "NVML, 5 ms period"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm),
                "source": "nvidia-smi -lms 100"}


# --------------------------------------------------------------------------- CPU baseline arms ---
def cpu_step_time(batch, reps=1):
    """One forward+backward+Adam step of the oracle restatement in Float32 on `batch` samples; returns seconds."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import flux_oracle as O
    blocks, head = make_params()
    rng = np.random.default_rng(11)
    x = rng.standard_normal((D, batch), dtype=np.float32)
    y = O.onehotbatch(rng.integers(1, NCLASS + 1, size=batch), NCLASS, np.float32)
    states = [{k: O.adam_init(v) for k, v in blk.items()} for blk in blocks]
    hstate = {k: O.adam_init(v) for k, v in head.items()}
    best = None
    for _ in range(reps):
        t0 = time.perf_counter()
        loss, gb, gh = O.dp_mlp_fwd_bwd(blocks, head, x, y)
        for blk, g, st in zip(blocks, gb, states):
            for k in blk:
                blk[k] = O.adam_apply(st[k], blk[k], g[k].astype(np.float32))
        for k in head:
            head[k] = O.adam_apply(hstate[k], head[k], gh[k].astype(np.float32))
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return best


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    total = max(args.steps + args.warmup, 1)
    probe = cpu_step_time(32)
    per_sample = probe / 32
    budget = 150.0 / total
    batch = int(min(GLOBAL_BATCH, max(32, budget / per_sample)))
    batch = max(32, batch // 32 * 32)
    for _ in range(args.warmup):
        cpu_step_time(batch)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step_time(batch)
    dt = time.perf_counter() - t0
    value = batch * args.steps / dt
    sample = f"{batch} of {GLOBAL_BATCH} samples per step (Float32 numpy/OpenBLAS restatement of Flux's unfused op sequence)"
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * dt / max(args.steps, 1) * (GLOBAL_BATCH / batch),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD},
            "cpu_baseline": {"value": value, "unit": "samples/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "Flux.jl itself cannot run here (no Julia toolchain); this is the oracle port on the host cores"}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------- GPU arm ---
def run_ours(args):
    import torch
    import fluxb200 as F
    from fluxb200 import lib
    DU = F.DistributedUtils

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")
    torch.cuda.set_device(local)
    F.context(local)
    backend = DU.initialize(DU.NCCLBackend, device=local)
    dist = None
    if world > 1:
        import torch.distributed as dist

    # model: identical parameters on every rank (seed 3), synchronised from rank 0 like the reference's how-to
    blocks, head = make_params()
    layers = []
    for blk in blocks:
        ln = F.LayerNorm(D)
        layers += [ln, F.Dense(blk["W"], blk["b"], "gelu")]
    layers.append(F.Dense(head["W"], head["b"]))
    model = F.Chain(*layers)
    DU.synchronize(backend, DU.FluxDistributedModel(model))
    params = F.trainables(model)
    buckets = DU.GradBuckets(backend, params, bucket_mb=args.bucket_mb)
    if args.timeline:
        buckets.enable_timeline()
    opt = F.setup(DU.DistributedOptimizer(backend, F.Adam(1e-3), buckets), model)
    DU.synchronize(backend, opt)

    # this rank's shard of the global batch (contiguous column block)
    idx = DU.shard_indices(GLOBAL_BATCH, world, rank)
    nloc = len(idx)
    rng = np.random.default_rng(100 + rank)
    x_host = torch.from_numpy(rng.standard_normal((nloc, D), dtype=np.float32).reshape(-1)).pin_memory()   # memory [n][D]
    lab_host = torch.from_numpy(rng.integers(1, NCLASS + 1, size=nloc).astype(np.int32)).pin_memory()
    x_dev = F.B200Array(x_host.cuda(non_blocking=True), (D, nloc))
    y_dev = F.OneHotLabels(F.B200Array(lab_host.cuda(non_blocking=True), (nloc,)), NCLASS)

    def loss_fn(m, x, y):
        return F.logitcrossentropy(m(x), y)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    if args.eager:
        def step(x, y):
            buckets.begin_step()
            l, gs = F.withgradient(lambda m: loss_fn(m, x, y), model, grad_sink=buckets)
            if np.isfinite(l):
                F.update(opt, model, gs[0])
            return l

        step_resident = lambda: step(x_dev, y_dev)

        def step_e2e():
            x = F.B200Array(x_host.cuda(non_blocking=True), (D, nloc))
            y = F.OneHotLabels(F.B200Array(lab_host.cuda(non_blocking=True), (nloc,)), NCLASS)
            return step(x, y)
        launches_per_step = None
    else:
        # the one-launch train step: forward, backward, bucketed all-reduce and Adam replayed from a CUDA graph
        k0 = lib.raw().fb_kernel_launches()
        gstep = F.GraphedTrainStep(loss_fn, model, opt, (x_dev, y_dev), grad_sink=buckets, shard_optimizer=not args.no_shard)
        launches_per_step = (lib.raw().fb_kernel_launches() - k0) // 2      # warm-up pass + captured pass
        step_resident = lambda: gstep(x_dev, y_dev)                          # inputs already in HBM
        # end to end: every step copies one batch from pinned host memory (the batch of the FOLLOWING step, started
        # right after this step's launch so that it travels beside the computation) and reads the loss back
        gstep.prefetch(x_host, lab_host)
        step_e2e = lambda: gstep(prefetch=(x_host, lab_host))

    for _ in range(max(args.warmup, 3)):
        step_resident()
    sampler = ClockSampler(local) if rank == 0 else None
    launches0 = lib.raw().fb_kernel_launches()
    ms = timed(step_resident, args.steps)
    launches = lib.raw().fb_kernel_launches() - launches0 if launches_per_step is None else launches_per_step * args.steps
    clocks = sampler.stop() if sampler else None
    for _ in range(2):
        step_e2e()
    ms_e2e = timed(step_e2e, args.steps)
    # dominant kernel: the tensor-core GEMM of a 4096 => 4096 Dense forward at this rank's batch, timed launch by
    # launch with CUDA events on the stream it runs on, directly after the timed steps (same clocks, same tensors)
    dense = model.layers[1]
    yb = F.empty((D, nloc))
    ctx = F.context()
    durs = []
    h0 = model.layers[0](x_dev)
    for i in range(12):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        lib.call("fb_dense_fwd", ctx.handle, ctx.stream, lib.ACT["gelu"], 0, dense.weight.ptr, dense.bias.ptr, h0.ptr, yb.ptr, None, D, D, nloc)
        e1.record()
        torch.cuda.synchronize()
        if i >= 2:
            durs.append(e0.elapsed_time(e1))
    if F.context().device_error() != 0:
        raise SystemExit("a kernel recorded a bounded-wait timeout; the numbers are invalid")

    if args.timeline and rank in (0, world - 1):
        for name, us in buckets.timeline():
            print(f"[timeline rank {rank}] {us:10.1f} us  {name}", file=sys.stderr)
    if rank != 0:
        return
    value = GLOBAL_BATCH * args.steps / (ms * 1e-3)
    # dominant kernel: the tensor-core GEMM of the 4096 => 4096 Dense forward (M = local batch, N = K = 4096)
    roof = None
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    # the kernel is timed alone (launch by launch), so the burst figure applies; TF32 runs at half the bf16 rate
    bf16 = peaks.get("bf16_tflops")
    peak_kind = "of measured (TF32 peak taken as half the measured burst bf16 cuBLAS figure)"
    if bf16 is None:
        bf16, peak_kind = 1590.0, "of fallback (TF32 peak taken as half of 1.59 PFLOP/s burst bf16)"
    if durs:
        avg_ms = float(np.mean(durs))
        alg = 2.0 * nloc * D * D / (avg_ms * 1e-3) / 1e12
        peak = bf16 / 2.0
        # DRAM bytes per launch from one ncu capture of this kernel at batch 8192 (dram__bytes_read + write = 693.6 +
        # 200.3 MB, against 335 MB algorithmic); for a smaller local batch it is scaled by the rows processed
        traffic = 893.9e6 * nloc / 8192.0
        roof = {"bound": "tensor", "achieved": alg, "peak": peak, "unit": "TFLOP/s", "frac": alg / peak, "traffic": traffic,
                "traffic_source": "ncu capture of the same kernel at batch 8192 (profiles/gemm_tc_kernel_dense4096_batch8192.md), scaled by local batch",
                "kernel": "gemm_tc_kernel (Dense 4096=>4096 forward, 3xTF32, persistent two-CTA 256x256 tiles)", "launch_ms": avg_ms, "launches_timed": len(durs),
                "issued_frac": 3.0 * alg / peak, "peak_kind": peak_kind,
                "note": "achieved = algorithmic 2*M*N*K per launch / CUDA-event launch time; 3xTF32 issues 3x that on the tensor pipe"}
    cores = os.cpu_count() or 1
    cb = 256
    cpu_t = cpu_step_time(cb, reps=2)
    line = {"metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "global_batch": GLOBAL_BATCH, "per_gpu_batch": nloc, "parallelism": f"dp{world}",
                       "matmul": "3xTF32 tcgen05", "gelu": "tanh approximation", "bucket_mb": args.bucket_mb,
                       "step": "eager launches" if args.eager else "CUDA graph replay (GraphedTrainStep)",
                       "optimizer": ("sharded Adam (reduce-scatter, 1/N update, all-gather per bucket)"
                                     if (not args.eager and getattr(gstep, "sharded", False)) else "Adam on every rank"),
                       "l2": "inputs larger than L2 (553 MB parameters, >3 GB activations per step)"},
            "tflops_algorithmic": value * FLOPS_PER_SAMPLE / 1e12,
            "e2e": {"value": GLOBAL_BATCH * args.steps / (ms_e2e * 1e-3), "unit": "samples/s",
                    "h2d_bytes_per_step": int(x_host.numel() * 4 + lab_host.numel() * 4), "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roof,
            "cpu_baseline": {"value": cb / cpu_t, "unit": "samples/s", "cores": cores, "kind": "port",
                             "sample": f"{cb} of {GLOBAL_BATCH} samples, best of 2 steps, Float32 numpy/OpenBLAS restatement (Flux CPU not runnable: no Julia)"}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------- the other four configurations ---
def run_small_config(args):
    """Configurations 1-4 of the benchmark set (single GPU): one JSON line each, same keys as the headline line."""
    import torch
    import fluxb200 as F
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import flux_oracle as O
    torch.cuda.set_device(0)
    F.context(0)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm = peaks.get("hbm_gbs", 6650.0)
    tf32 = peaks.get("bf16_tflops", 1590.0) / 2.0
    rng = np.random.default_rng(args.config)
    f64 = lambda a: a.astype(np.float64)

    def time_gpu(fn, steps, warmup):
        for _ in range(max(warmup, 3)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    def time_grad(fn, model, steps, warmup):
        """ms per forward + gradient: one CUDA-graph replay per call where the step can be captured, else eager launches."""
        try:
            gg = F.GraphedGradient(fn, model)
            return time_gpu(lambda: gg(), steps, warmup), "CUDA graph replay"
        except Exception:
            torch.cuda.synchronize()
            return time_gpu(lambda: F.withgradient(fn, model), steps, warmup), "eager launches"

    def time_cpu(fn, reps=2):
        best = None
        for _ in range(reps):
            t0 = time.perf_counter()
            fn()
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        return best

    lines = []
    if args.config == 1:
        dims = [(512, 784, "relu"), (512, 512, "relu"), (10, 512, "identity")]
        Ws = [O.glorot_uniform(np.random.default_rng(0), o, i) for o, i, _ in dims]
        x = rng.random((784, 1024), dtype=np.float32)
        labels = rng.integers(1, 11, size=1024)
        model = F.Chain(*[F.Dense(W.copy(), True, s_) for W, (_, _, s_) in zip(Ws, dims)])
        opt = F.setup(F.Adam(1e-3), model)
        xg, yg = F.gpu(x), F.onehotbatch(labels, 10)
        loss = lambda m, a, b: F.logitcrossentropy(m(a), b)
        gstep = F.GraphedTrainStep(loss, model, opt, (xg, yg))
        ms = time_gpu(lambda: gstep(xg, yg), args.steps, args.warmup)
        ms_eager = time_gpu(lambda: F.trainstep(loss, model, (xg, yg), opt), args.steps, args.warmup)
        y1h = O.onehotbatch(labels, 10, np.float32)
        layers = [(W, np.zeros(W.shape[0], np.float32), s_) for W, (_, _, s_) in zip(Ws, dims)]
        cpu = time_cpu(lambda: O.mlp_chain_fwd_bwd(layers, x, y1h), 3)
        flops = 3.286e9
        lines.append(("mlp: Chain(Dense(784=>512,relu),Dense(512=>512,relu),Dense(512=>10)), batch 1024, logitcrossentropy+Adam, CUDA graph step",
                      1024, ms, {"bound": "tensor", "achieved": flops / ms / 1e9, "peak": tf32, "unit": "TFLOP/s", "frac": flops / ms / 1e9 / tf32,
                                 "traffic": None, "note": f"launch/latency-bound (3.3 GFLOP per step); eager launches take {ms_eager:.3f} ms per step"},
                      1024 / cpu, "1024 of 1024 samples, forward+backward (no Adam), best of 3"))
    elif args.config == 2:
        xb = (rng.standard_normal((32, 32, 256, 128), dtype=np.float32) * 2 + 0.5)
        bn = F.trainmode(F.BatchNorm(256, "relu"))
        xg = F.gpu(xb)
        ms, how = time_grad(lambda m: F.sum_abs2(m(xg)), bn, args.steps, args.warmup)
        E = xb.size
        xs = xb[:, :, :, :8]
        cpu = time_cpu(lambda: (O.batchnorm_fwd_train(xs, np.ones(256, np.float32), np.zeros(256, np.float32), np.zeros(256, np.float32), np.ones(256, np.float32), sigma="relu"),
                                O.batchnorm_bwd(xs, np.ones(256, np.float32), np.zeros(256, np.float32), 2 * xs, sigma="relu")))
        by = 11.0 * E * 4
        lines.append(("batchnorm: BatchNorm(256,relu) train, 32x32x256x128 Float32, forward + gradient of sum(abs2,y)", 128, ms,
                      {"bound": "hbm", "achieved": by / ms / 1e6, "peak": hbm, "unit": "GB/s", "frac": by / ms / 1e6 / hbm, "traffic": None,
                       "note": "11 passes x 134.2 MB: layer (8) + sum(abs2) read (1) + cotangent 2y read+write (2); " + how},
                      8 / cpu, "8 of 128 samples, best of 2"))
        xl = rng.standard_normal((4096, 16384), dtype=np.float32)
        ln = F.LayerNorm(4096)
        xlg = F.gpu(xl)
        ms, how = time_grad(lambda m: F.sum_abs2(m(xlg)), ln, args.steps, args.warmup)
        xls = xl[:, :1024]
        g1, b1 = np.ones(4096, np.float32), np.zeros(4096, np.float32)
        cpu = time_cpu(lambda: (O.layernorm_fwd(xls, g1, b1), O.layernorm_bwd(xls, g1, b1, 2 * xls)))
        by = 8.0 * xl.size * 4
        lines.append(("layernorm: LayerNorm(4096) on 4096x16384 Float32, forward + gradient of sum(abs2,y)", 16384, ms,
                      {"bound": "hbm", "achieved": by / ms / 1e6, "peak": hbm, "unit": "GB/s", "frac": by / ms / 1e6 / hbm, "traffic": None,
                       "note": "8 passes x 268.4 MB: layer (5) + sum(abs2) read (1) + cotangent 2y read+write (2); " + how},
                      1024 / cpu, "1024 of 16384 samples, best of 2"))
    elif args.config == 3:
        Hh, T, B = 512, 256, 64
        r1 = np.random.default_rng(1)
        Wi, Wh = O.glorot_uniform(r1, 4 * Hh, Hh), O.glorot_uniform(r1, 4 * Hh, Hh)
        x = rng.standard_normal((Hh, T, B), dtype=np.float32)
        rnn = F.LSTM(Wi, Wh)
        xg = F.gpu(x)
        ms = time_gpu(lambda: F.withgradient(lambda m: F.sum_abs2(m(xg)), rnn), args.steps, args.warmup)
        xs, bz = x[:, :, :4], np.zeros(4 * Hh, np.float32)
        cpu = time_cpu(lambda: O.lstm_scan_bwd(Wi, Wh, bz, xs, 2 * O.lstm_scan_fwd(Wi, Wh, bz, xs)[0]), 1)
        flops = 171.8e9
        lines.append(("lstm: LSTM(512=>512) via Recurrence, 512x256x64 Float32, forward + gradient of sum(abs2,out)", 64, ms,
                      {"bound": "tensor", "achieved": flops / ms / 1e9, "peak": tf32, "unit": "TFLOP/s", "frac": flops / ms / 1e9 / tf32, "traffic": None,
                       "note": f"bounded by 2 x 256 dependent steps: {ms * 1e3 / 512:.1f} us per time step (forward and backward)"},
                      4 / cpu, "4 of 64 sequences, 1 run"))
    elif args.config == 4:
        E, S, B, Hn = 1024, 2048, 8, 16
        r2 = np.random.default_rng(2)
        Ws = [O.glorot_uniform(r2, E, E) for _ in range(4)]
        x = rng.standard_normal((E, S, B), dtype=np.float32)
        mha = F.MultiHeadAttention(*Ws, nheads=Hn)
        xg = F.gpu(x)
        ms, how = time_grad(lambda m: F.sum_abs2(m(xg, mask=F.make_causal_mask())[0]), mha, args.steps, args.warmup)
        xs = x[:, :512, :1]
        def cpu_fn():
            y, _ = O.mha_fwd(*Ws, xs, nheads=Hn, mask=O.make_causal_mask(512))
            O.mha_bwd(*Ws, xs, 2 * y, nheads=Hn, mask=O.make_causal_mask(512))
        cpu = time_cpu(cpu_fn, 1)
        flops = 652.8e9
        lines.append(("mha: MultiHeadAttention(1024, nheads=16), causal, 1024x2048x8 Float32, forward + backward (loss on y)", 8, ms,
                      {"bound": "tensor", "achieved": flops / ms / 1e9, "peak": tf32, "unit": "TFLOP/s", "frac": flops / ms / 1e9 / tf32, "traffic": None,
                       "note": "projections and the attention core (forward, dQ, dK/dV) on tcgen05 with 3xTF32; softmax and dS on TMEM read-back; " + how},
                      (1 * (512 / 2048) ** 2 * 1.0) / cpu * 1.0, "1 of 8 samples at seq 512 (1/16 of a sample's attention work, 1/4 of its projections), 1 run"))
    if F.context().device_error() != 0:
        raise SystemExit("a kernel recorded a bounded-wait timeout; the numbers are invalid")
    cores = os.cpu_count() or 1
    for workload, samples, ms, roof, cpu_v, cpu_s in lines:
        print(json.dumps({"metric": METRIC, "value": samples / (ms * 1e-3), "unit": "samples/s", "n_gpus": 1, "steps": args.steps,
                          "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                          "dtype": "f32", "data": "synthetic", "config": {"workload": workload}, "roofline": roof,
                          "cpu_baseline": {"value": cpu_v, "unit": "samples/s", "cores": cores, "kind": "port", "sample": cpu_s}}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--bucket-mb", dest="bucket_mb", type=float, default=64.0)
    ap.add_argument("--timeline", action="store_true",
                    help="print, on stderr, device time marks of the last step (compute and communication streams)")
    ap.add_argument("--no-shard", dest="no_shard", action="store_true",
                    help="N > 1: all-reduce gradients and run Adam on every rank instead of reduce-scatter + sharded Adam + all-gather")
    ap.add_argument("--eager", action="store_true", help="launch every kernel from the host each step instead of replaying a CUDA graph")
    ap.add_argument("--config", type=int, default=5, choices=[1, 2, 3, 4, 5],
                    help="5 (default): the data-parallel MLP the headline metric is quoted on; 1-4: the single-GPU configurations")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.config != 5:
        run_small_config(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
