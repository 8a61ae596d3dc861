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


def _host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


# The CPU legs (rank 0 only) use every host core whatever the launcher exported: torch.distributed.run sets
# OMP_NUM_THREADS=1 for its children, and the BLAS behind numpy reads these variables when it is first loaded.
if os.environ.get("RANK", "0") == "0":
    for _v in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[_v] = str(_host_cores())

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
def blas_threads() -> int:
    """Threads the BLAS behind numpy actually runs with (threadpoolctl), else the host core count."""
    try:
        from threadpoolctl import threadpool_info
        n = [int(d.get("num_threads", 0)) for d in threadpool_info() if d.get("user_api") == "blas"]
        if n:
            return max(n)
    except Exception:
        pass
    return _host_cores()


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
    """The reference arm: Flux's CPU path cannot run (no Julia toolchain), so the oracle port is timed on every host
    core, each step on a bounded sample of the global batch (at least 256 samples, where sgemm is near its best)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    total = max(args.steps + args.warmup, 1)
    probe = cpu_step_time(64)
    per_sample = probe / 64
    budget = 150.0 / total
    batch = int(min(GLOBAL_BATCH, max(256, budget / per_sample)))
    batch = max(256, batch // 64 * 64)
    for _ in range(args.warmup):
        cpu_step_time(batch)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step_time(batch)
    dt = time.perf_counter() - t0
    value = batch * args.steps / dt
    threads = blas_threads()
    sample = (f"{batch} of {GLOBAL_BATCH} samples per step, {threads} BLAS threads on {_host_cores()} host cores "
              "(Float32 numpy restatement of Flux's unfused op sequence)")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * dt / max(args.steps, 1),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "samples_per_timed_step": batch},
            "cpu_baseline": {"value": value, "unit": "samples/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "Flux.jl itself cannot run here (no Julia toolchain); this is the oracle port on the host cores; "
                    "ms_per_step is the time of one bounded-sample step, value = samples per second"}
    print(json.dumps(line), flush=True)


def load_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        return {}


# --------------------------------------------------------------------------------- GPU arm ---
def global_batch():
    """The global synthetic batch (one seed for every rank count): x is [GLOBAL_BATCH][D] in memory, labels 1..NCLASS."""
    rng = np.random.default_rng(100)
    x = rng.standard_normal((GLOBAL_BATCH, D), dtype=np.float32)
    labels = rng.integers(1, NCLASS + 1, size=GLOBAL_BATCH).astype(np.int32)
    return x, labels


def check_logits(F, model, x_dev, x_rows, blocks, head, ncheck=32):
    """Correctness gate: the model's logits for `ncheck` columns of this rank's batch against the float64 oracle
    (the model is column-independent).  Returns the largest error relative to max|reference|."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import flux_oracle as O   # the checker, not the product
    nloc = x_rows.shape[0]
    cols = np.unique(np.linspace(0, nloc - 1, ncheck).astype(np.int64))
    logits = F.cpu(model(x_dev))[:, cols].astype(np.float64)
    h = x_rows[cols].T.astype(np.float64)
    for blk in blocks:
        hn = O.layernorm_fwd(h, blk["gamma"].astype(np.float64), blk["beta"].astype(np.float64), 1e-5)
        h = O.dense_fwd(blk["W"].astype(np.float64), blk["b"].astype(np.float64), hn, "gelu_tanh")
    ref = O.dense_fwd(head["W"].astype(np.float64), head["b"].astype(np.float64), h)
    return float(np.max(np.abs(logits - ref)) / max(np.max(np.abs(ref)), 1e-30)), int(len(cols))


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

    # this rank's shard of the global batch (contiguous column block of one global draw)
    idx = DU.shard_indices(GLOBAL_BATCH, world, rank)
    nloc = len(idx)
    xg_all, lab_all = global_batch()
    x_rows = np.ascontiguousarray(xg_all[idx[0]:idx[-1] + 1])
    x_host = torch.from_numpy(x_rows.reshape(-1)).pin_memory()   # memory [n][D]
    lab_host = torch.from_numpy(np.ascontiguousarray(lab_all[idx[0]:idx[-1] + 1])).pin_memory()
    del xg_all
    x_dev = F.B200Array(x_host.cuda(non_blocking=True), (D, nloc))
    y_dev = F.OneHotLabels(F.B200Array(lab_host.cuda(non_blocking=True), (nloc,)), NCLASS)

    # correctness gate before anything is timed (every rank checks its own shard; the worst error is reported)
    err, ncheck = check_logits(F, model, x_dev, x_rows, blocks, head)
    if dist is not None:
        t = torch.tensor([err], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        err = float(t.item())
    check = {"what": f"logits of {ncheck} columns per rank against the float64 oracle, relative to max|reference|",
             "max_rel_err": err, "tol": 1e-4, "ok": bool(err <= 1e-4)}
    if not check["ok"]:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "check": check, "error": "correctness gate failed; nothing was timed"}), flush=True)
        raise SystemExit(3)

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
        gstep = F.GraphedTrainStep(loss_fn, model, opt, (x_dev, y_dev), grad_sink=buckets, shard_optimizer=not args.no_shard,
                                   defer_gather=not args.no_defer)
        launches_per_step = (lib.raw().fb_kernel_launches() - k0) // 2      # warm-up pass + captured pass
        step_resident = lambda: gstep(x_dev, y_dev)                          # inputs already in HBM
        # end to end: every step copies one batch from pinned host memory (the batch of the FOLLOWING step, started
        # right after this step's launch so that it travels beside the computation) and reads the loss back
        gstep.prefetch(x_host, lab_host)
        step_e2e = lambda: gstep(prefetch=(x_host, lab_host))

    first_loss = None
    for i in range(max(args.warmup, 3)):
        l = step_resident()
        if i == 0:
            first_loss = float(l)
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
    peaks = load_peaks()
    # the kernel is timed alone (launch by launch), so the burst figure applies; TF32 runs at half the bf16 rate
    bf16 = peaks.get("bf16_tflops")
    peak_kind = "of measured (TF32 peak taken as half the measured burst bf16 cuBLAS figure)"
    if bf16 is None:
        bf16, peak_kind = 1590.0, "of fallback (TF32 peak taken as half of 1.59 PFLOP/s burst bf16)"
    if durs:
        avg_ms = float(np.mean(durs))
        alg = 2.0 * nloc * D * D / (avg_ms * 1e-3) / 1e12
        peak = bf16 / 2.0
        # DRAM bytes per launch from one ncu capture of this kernel at batch 8192 (dram__bytes_read + write), against
        # 335 MB algorithmic; for a smaller local batch it is scaled by the rows processed
        traffic = GEMM_TRAFFIC_B8192 * nloc / 8192.0
        roof = {"bound": "tensor", "achieved": alg, "peak": peak, "unit": "TFLOP/s", "frac": alg / peak, "traffic": traffic,
                "traffic_source": "ncu capture of the same kernel at batch 8192 (profiles/gemm_tc_kernel_dense4096_batch8192.md), scaled by local batch",
                "kernel": "gemm_tc_kernel (Dense 4096=>4096 forward, 3xTF32, persistent two-CTA 256x256 tiles)", "launch_ms": avg_ms, "launches_timed": len(durs),
                "issued_frac": 3.0 * alg / peak, "peak_kind": peak_kind,
                "note": "achieved = algorithmic 2*M*N*K per launch / CUDA-event launch time; 3xTF32 issues 3x that on the tensor pipe"}
    cb = 256
    cpu_t = cpu_step_time(cb, reps=2)
    threads = blas_threads()
    sm = (clocks or {}).get("sm_mhz")
    line = {"metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "global_batch": GLOBAL_BATCH, "per_gpu_batch": nloc, "parallelism": f"dp{world}",
                       "matmul": "3xTF32 tcgen05", "gelu": "tanh approximation", "bucket_mb": args.bucket_mb,
                       "step": "eager launches" if args.eager else "CUDA graph replay (GraphedTrainStep)",
                       "optimizer": ("sharded Adam (reduce-scatter, 1/N update, all-gather per bucket)"
                                     if (not args.eager and getattr(gstep, "sharded", False)) else "Adam on every rank"),
                       "exchange": ("n/a" if world == 1 else
                                    ("copy engines over peer memory" if getattr(buckets, "peer", None) is not None else "NCCL collectives") +
                                    (", parameter gather deferred to the next forward pass" if getattr(buckets, "defer_gather", False) else "")),
                       "batch": "one global draw (seed 100), contiguous column block per rank",
                       "nccl_env": {k: v for k, v in os.environ.items() if k.startswith("NCCL_")},
                       "l2": "inputs larger than L2 (553 MB parameters, >3 GB activations per step)"},
            "tflops_algorithmic": value * FLOPS_PER_SAMPLE / 1e12,
            "ms_x_sm_ghz": (ms / args.steps) * sm / 1e3 if sm else None,
            "check": dict(check, first_step_loss=first_loss),
            "e2e": {"value": GLOBAL_BATCH * args.steps / (ms_e2e * 1e-3), "unit": "samples/s",
                    "h2d_bytes_per_step": int(x_host.numel() * 4 + lab_host.numel() * 4), "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roof,
            "cpu_baseline": {"value": cb / cpu_t, "unit": "samples/s", "cores": threads, "kind": "port",
                             "sample": f"{cb} of {GLOBAL_BATCH} samples, best of 2 steps, {threads} BLAS threads, Float32 numpy restatement (Flux CPU not runnable: no Julia)"}}
    if world == 1 and not args.no_configs:
        # the single-GPU configurations ride in the same line so that they are timed by the same run
        del gstep, model, opt, buckets, x_dev, y_dev, yb, h0
        torch.cuda.empty_cache()
        cfgs = []
        for c in (1, 2, 3, 4):
            try:
                cfgs += small_config_lines(c, max(args.steps, 10), args.warmup)
            except Exception as e:   # a failing side configuration must not lose the headline
                cfgs.append({"config": {"workload": f"config {c}"}, "error": f"{type(e).__name__}: {e}"})
        line["configs"] = cfgs
    print(json.dumps(line), flush=True)


GEMM_TRAFFIC_B8192 = 893.9e6   # dram__bytes_read.sum + dram__bytes_write.sum of one Dense 4096=>4096 forward GEMM at batch 8192


# ------------------------------------------------------------- the other four configurations ---
def small_config_lines(config, steps, warmup):
    """Configurations 1-4 of the benchmark set (single GPU): a list of result dicts with the headline line's keys."""
    import torch
    import fluxb200 as F
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import flux_oracle as O
    torch.cuda.set_device(0)
    F.context(0)
    peaks = load_peaks()
    hbm = peaks.get("hbm_gbs", 6650.0)
    tf32 = peaks.get("bf16_tflops", 1590.0) / 2.0
    rng = np.random.default_rng(config)

    def time_gpu(fn, steps, warmup):
        for _ in range(max(warmup, 3)):
            fn()
        torch.cuda.synchronize()
        sampler = ClockSampler(0)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps, sampler.stop()

    def grad_runner(fn, model):
        """forward + gradient: one CUDA-graph replay per call where the step can be captured, else eager launches."""
        try:
            gg = F.GraphedGradient(fn, model)
            return (lambda: gg()[0]), "CUDA graph replay"
        except Exception:
            torch.cuda.synchronize()
            return (lambda: F.withgradient(fn, model)[0]), "eager launches"

    def e2e_of(run, dev_inputs, host_inputs):
        """Same call with the inputs coming from pinned host memory every step and the loss read back."""
        pinned = [torch.from_numpy(np.ascontiguousarray(h.reshape(-1, order="F"))).pin_memory() for h in host_inputs]

        def fn():
            for d, p in zip(dev_inputs, pinned):
                d.copy_(p, non_blocking=True)
            out = run()
            return float(out.t.item()) if hasattr(out, "t") else float(out)
        ms, _ = time_gpu(fn, steps, warmup)
        return ms, int(sum(p.numel() * p.element_size() for p in pinned))

    def time_cpu(fn, reps=2):
        best = None
        for _ in range(reps):
            t0 = time.perf_counter()
            fn()
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        return best

    lines = []

    def add(workload, samples, ms, clocks, roof, e2e_ms, h2d, cpu_value, cpu_sample, dtype="f32"):
        lines.append({"metric": METRIC, "value": samples / (ms * 1e-3), "unit": "samples/s", "n_gpus": 1, "steps": steps,
                      "warmup": max(warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                      "dtype": dtype, "data": "synthetic", "config": {"workload": workload}, "roofline": roof, "clocks": clocks,
                      "e2e": {"value": samples / (e2e_ms * 1e-3), "unit": "samples/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
                      "cpu_baseline": {"value": cpu_value, "unit": "samples/s", "cores": blas_threads(), "kind": "port", "sample": cpu_sample}})

    if config == 1:
        dims = [(512, 784, "relu"), (512, 512, "relu"), (10, 512, "identity")]
        r0 = np.random.default_rng(0)
        Ws = [O.glorot_uniform(r0, o, i) for o, i, _ in dims]
        x = rng.random((784, 1024), dtype=np.float32)
        labels = rng.integers(1, 11, size=1024).astype(np.int32)
        model = F.Chain(*[F.Dense(W.copy(), True, s_) for W, (_, _, s_) in zip(Ws, dims)])
        opt = F.setup(F.Adam(1e-3), model)
        xg, yg = F.gpu(x), F.onehotbatch(labels, 10)
        loss = lambda m, a, b: F.logitcrossentropy(m(a), b)
        gstep = F.GraphedTrainStep(loss, model, opt, (xg, yg))
        ms, clocks = time_gpu(lambda: gstep(xg, yg), steps, warmup)
        xh = torch.from_numpy(np.ascontiguousarray(x.reshape(-1, order="F"))).pin_memory()
        lh = torch.from_numpy(labels).pin_memory()
        ms_e2e, _ = time_gpu(lambda: gstep(xh, lh), steps, warmup)
        ms_eager, _ = time_gpu(lambda: F.trainstep(loss, model, (xg, yg), opt), steps, warmup)
        y1h = O.onehotbatch(labels, 10, np.float32)
        layers = [(W, np.zeros(W.shape[0], np.float32), s_) for W, (_, _, s_) in zip(Ws, dims)]
        cpu = time_cpu(lambda: O.mlp_chain_fwd_bwd(layers, x, y1h), 3)
        flops = 3.286e9
        add("mlp: Chain(Dense(784=>512,relu),Dense(512=>512,relu),Dense(512=>10)), batch 1024, logitcrossentropy+Adam, CUDA graph step",
            1024, ms, clocks, {"bound": "tensor", "achieved": flops / ms / 1e9, "peak": tf32, "unit": "TFLOP/s", "frac": flops / ms / 1e9 / tf32,
                               "traffic": None, "flops_per_step": flops,
                               "note": f"launch/latency-bound (3.3 GFLOP per step); eager launches take {ms_eager:.3f} ms per step"},
            ms_e2e, int(xh.numel() * 4 + lh.numel() * 4), 1024 / cpu, "1024 of 1024 samples, forward+backward (no Adam), best of 3")
    elif config == 2:
        xb = (rng.standard_normal((32, 32, 256, 128), dtype=np.float32) * 2 + 0.5)
        bn = F.trainmode(F.BatchNorm(256, "relu"))
        xg = F.gpu(xb)
        run, how = grad_runner(lambda m: F.sum_abs2(m(xg)), bn)
        ms, clocks = time_gpu(run, steps, warmup)
        ms_e2e, h2d = e2e_of(run, [xg.t], [xb])
        E = xb.size
        xs = xb[:, :, :, :8]
        one, zero = np.ones(256, np.float32), np.zeros(256, np.float32)
        cpu = time_cpu(lambda: (O.batchnorm_fwd_train(xs, one, zero, zero.copy(), one.copy(), sigma="relu"),
                                O.batchnorm_bwd(xs, one, zero, 2 * xs, sigma="relu")))
        by = 11.0 * E * 4
        add("batchnorm: BatchNorm(256,relu) train, 32x32x256x128 Float32, forward + gradient of sum(abs2,y)", 128, ms, clocks,
            {"bound": "hbm", "achieved": by / ms / 1e6, "peak": hbm, "unit": "GB/s", "frac": by / ms / 1e6 / hbm, "traffic": None,
             "bytes_per_step": by,
             "note": "11 passes x 134.2 MB: layer (8) + sum(abs2) read (1) + cotangent 2y read+write (2); " + how},
            ms_e2e, h2d, 8 / cpu, "8 of 128 samples, best of 2")
        del xg, run, bn
        torch.cuda.empty_cache()
        xl = rng.standard_normal((4096, 16384), dtype=np.float32)
        ln = F.LayerNorm(4096)
        xlg = F.gpu(xl)
        run, how = grad_runner(lambda m: F.sum_abs2(m(xlg)), ln)
        ms, clocks = time_gpu(run, steps, warmup)
        ms_e2e, h2d = e2e_of(run, [xlg.t], [xl])
        xls = xl[:, :1024]
        g1, b1 = np.ones(4096, np.float32), np.zeros(4096, np.float32)
        cpu = time_cpu(lambda: (O.layernorm_fwd(xls, g1, b1), O.layernorm_bwd(xls, g1, b1, 2 * xls)))
        by = 8.0 * xl.size * 4
        add("layernorm: LayerNorm(4096) on 4096x16384 Float32, forward + gradient of sum(abs2,y)", 16384, ms, clocks,
            {"bound": "hbm", "achieved": by / ms / 1e6, "peak": hbm, "unit": "GB/s", "frac": by / ms / 1e6 / hbm, "traffic": None,
             "bytes_per_step": by,
             "note": "8 passes x 268.4 MB: layer (5) + sum(abs2) read (1) + cotangent 2y read+write (2); " + how},
            ms_e2e, h2d, 1024 / cpu, "1024 of 16384 samples, best of 2")
    elif config == 3:
        Hh, T, B = 512, 256, 64
        r1 = np.random.default_rng(1)
        Wi, Wh = O.glorot_uniform(r1, 4 * Hh, Hh), O.glorot_uniform(r1, 4 * Hh, Hh)
        x = rng.standard_normal((Hh, T, B), dtype=np.float32)
        rnn = F.LSTM(Wi, Wh)
        xg = F.gpu(x)
        run = lambda: F.withgradient(lambda m: F.sum_abs2(m(xg)), rnn)[0]
        ms, clocks = time_gpu(run, steps, warmup)
        ms_e2e, h2d = e2e_of(run, [xg.t], [x])
        xs, bz = x[:, :, :4], np.zeros(4 * Hh, np.float32)
        cpu = time_cpu(lambda: O.lstm_scan_bwd(Wi, Wh, bz, xs, 2 * O.lstm_scan_fwd(Wi, Wh, bz, xs)[0]), 1)
        flops = 171.8e9
        add("lstm: LSTM(512=>512) via Recurrence, 512x256x64 Float32, forward + gradient of sum(abs2,out)", 64, ms, clocks,
            {"bound": "tensor", "achieved": flops / ms / 1e9, "peak": tf32, "unit": "TFLOP/s", "frac": flops / ms / 1e9 / tf32, "traffic": None,
             "flops_per_step": flops, "us_per_time_step": ms * 1e3 / 512,
             "note": f"bounded by 2 x 256 dependent steps: {ms * 1e3 / 512:.1f} us per time step (forward and backward); eager launches (persistent kernels)"},
            ms_e2e, h2d, 4 / cpu, "4 of 64 sequences, 1 run")
    elif config == 4:
        E, S, B, Hn = 1024, 2048, 8, 16
        r2 = np.random.default_rng(2)
        Ws = [O.glorot_uniform(r2, E, E) for _ in range(4)]
        x = rng.standard_normal((E, S, B), dtype=np.float32)
        xs = x[:, :512, :1]

        def cpu_fn():
            y, _ = O.mha_fwd(*Ws, xs, nheads=Hn, mask=O.make_causal_mask(512))
            O.mha_bwd(*Ws, xs, 2 * y, nheads=Hn, mask=O.make_causal_mask(512))
        cpu = time_cpu(cpu_fn, 1)
        flops = 652.8e9
        for dtype in MHA_DTYPES:
            mha = F.MultiHeadAttention(*[w.copy() for w in Ws], nheads=Hn)
            xg = F.gpu(x)
            if dtype == "bf16":
                mha = F.bf16(mha)
                xg = F.bf16(xg)
            run, how = grad_runner(lambda m: F.sum_abs2(m(xg, mask=F.make_causal_mask())[0]), mha)
            ms, clocks = time_gpu(run, steps, warmup)
            ms_e2e, h2d = e2e_of(run, [xg.t], [x])
            peak = tf32 if dtype == "f32" else 2 * tf32
            add(f"mha: MultiHeadAttention(1024, nheads=16), causal, 1024x2048x8 {'Float32' if dtype == 'f32' else 'BFloat16'}, forward + backward (loss on y)",
                8, ms, clocks,
                {"bound": "tensor", "achieved": flops / ms / 1e9, "peak": peak, "unit": "TFLOP/s", "frac": flops / ms / 1e9 / peak, "traffic": None,
                 "flops_per_step": flops,
                 "note": ("projections and the attention core (forward, dQ, dK/dV) on tcgen05 with 3xTF32; softmax and dS on TMEM read-back; "
                          if dtype == "f32" else "the opt-in bf16 path (fluxb200.bf16); ") + how},
                ms_e2e, h2d, (1 * (512 / 2048) ** 2 * 1.0) / cpu,
                "1 of 8 samples at seq 512 (1/16 of a sample's attention work, 1/4 of its projections), Float32, 1 run", dtype=dtype)
            del mha, xg, run
            torch.cuda.empty_cache()
    if F.context().device_error() != 0:
        raise SystemExit("a kernel recorded a bounded-wait timeout; the numbers are invalid")
    return lines


MHA_DTYPES = ("f32", "bf16")


# ----------------------------------------------------------- single-kernel cases (profiling) ---
CASES = """gemm_fwd    Dense 4096=>4096 forward at --batch (3xTF32 tcgen05 GEMM, K-major x MN-major)
gemm_dw     the dW GEMM of the same layer (MN-major x MN-major, K = batch)
gemm_dx     the dX GEMM of the same layer (K-major x K-major)
gemm_bf16_fwd / gemm_bf16_dw / gemm_bf16_dx   the same three products with BFloat16 storage (tcgen05 kind::f16)
layernorm   LayerNorm(4096) forward + backward on 4096 x 8192
batchnorm   BatchNorm(256, relu) training forward + backward on 32 x 32 x 256 x 128
adam        Adam step over 32 Mi parameters in 4 leaves
attention   causal attention forward + backward, E = 1024, 16 heads, S = 1024, B = 2
lstm        LSTM(512=>512) forward + backward, T = 32, B = 64
gru         GRU(512=>512) forward + backward, T = 32, B = 64
xent        logitcrossentropy forward + backward, 1000 x 8192"""


def run_case(args):
    """One small single-kernel workload for Nsight Compute captures (`--case NAME --iters 1`) and CUDA-event timing
    (`--time`: L2 flushed between iterations, achieved GB/s or TFLOP/s against the algorithmic bytes / flops).  Each
    case holds well under a few GB on the device; inputs exceed the 126 MB L2 so that DRAM counters mean something."""
    import ctypes as C
    import torch
    from fluxb200 import lib
    P = lambda t: C.c_void_p(t.data_ptr()) if t is not None else None
    torch.cuda.set_device(0)
    h = C.c_void_p()
    lib.call("fb_ctx_create", 0, C.byref(h))
    st = lambda: C.c_void_p(torch.cuda.current_stream().cuda_stream)
    call = lambda name, *a: lib.call(name, h, st(), *a)
    g = torch.Generator(device="cuda").manual_seed(0)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g)
    em = lambda n: torch.empty(n, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    case = args.case
    if case in ("gemm_fwd", "gemm_dw", "gemm_dx"):
        n, d = args.batch, 4096
        W, x, dy = rn(d * d) * 0.02, rn(n * d), rn(n * d)
        y, dW, dx, b = em(n * d), em(d * d), em(n * d), rn(d)
        if case == "gemm_fwd":
            fn = lambda: call("fb_dense_fwd", 4, 0, P(W), P(b), P(x), P(y), None, d, d, n)
        elif case == "gemm_dw":
            fn = lambda: call("fb_gemm_f32", 0, 1, d, d, n, P(dy), d, P(x), d, P(dW), d, 0, 0)       # dW = dy * x'
        else:
            fn = lambda: call("fb_gemm_f32", 1, 0, d, n, d, P(W), d, P(dy), d, P(dx), d, 0, 0)       # dx = W' * dy
        work = (2.0 * n * d * d, "TFLOP/s")
    elif case in ("gemm_bf16_fwd", "gemm_bf16_dw", "gemm_bf16_dx"):
        n, d = args.batch, 4096
        bfr = lambda k: rn(k).to(torch.bfloat16)
        W, x, dy, b = bfr(d * d) * 0.02, bfr(n * d), bfr(n * d), bfr(d)
        eb = lambda k: torch.empty(k, dtype=torch.bfloat16, device="cuda")
        y, dW, dx = eb(n * d), eb(d * d), eb(n * d)
        if case == "gemm_bf16_fwd":
            fn = lambda: call("fb_dense_fwd_bf16", 4, P(W), P(b), P(x), P(y), None, d, d, n)
        elif case == "gemm_bf16_dw":
            fn = lambda: call("fb_gemm_bf16", 0, 1, d, d, n, P(dy), d, P(x), d, P(dW), d, 0, 0)
        else:
            fn = lambda: call("fb_gemm_bf16", 1, 0, d, n, d, P(W), d, P(dy), d, P(dx), d, 0, 0)
        work = (2.0 * n * d * d, "TFLOP/s")
    elif case == "layernorm":
        d, n = 4096, 8192
        x, dy, gam, bet = rn(d * n), rn(d * n), rn(d), rn(d)
        y, dx, mean, rstd, dg, db = em(d * n), em(d * n), em(n), em(n), em(d), em(d)

        def fn():
            call("fb_layernorm_fwd", P(x), P(gam), P(bet), P(y), P(mean), P(rstd), d, n, 1e-5, 0)
            call("fb_layernorm_bwd", P(x), P(gam), P(bet), P(mean), P(rstd), P(dy), P(dx), P(dg), P(db), d, n, 0)
        work = (5.0 * d * n * 4, "GB/s")
    elif case == "batchnorm":
        s, c, n = 1024, 256, 128
        x, dy, gam, bet = rn(s * c * n) * 2 + 0.5, rn(s * c * n), rn(c), rn(c)
        rm, rv = torch.zeros(c, device="cuda"), torch.ones(c, device="cuda")
        y, dx = torch.empty_like(x), torch.empty_like(x)
        sm, sr, dg, db = (em(c) for _ in range(4))

        def fn():
            call("fb_batchnorm_fwd_train", P(x), P(gam), P(bet), P(rm), P(rv), P(y), P(sm), P(sr), s, c, n, 1e-5, 0.1, 1, 1)
            call("fb_batchnorm_bwd", P(x), P(gam), P(bet), P(sm), P(sr), P(dy), P(dx), P(dg), P(db), s, c, n, 1)
        work = (8.0 * s * c * n * 4, "GB/s")
    elif case == "adam":
        k, cnt = 4, 8 << 20
        w, gr, m, v = ([rn(cnt) for _ in range(k)] for _ in range(4))
        arr = C.c_void_p * k
        tabs = [arr(*[t.data_ptr() for t in ts]) for ts in (w, gr, m, v)]
        counts = (C.c_int64 * k)(*([cnt] * k))
        fn = lambda: call("fb_adam_step", k, tabs[0], tabs[1], tabs[2], tabs[3], counts, 1e-3, 0.9, 0.999, 1e-8, 0.9, 0.999, 1.0)
        work = (7.0 * k * cnt * 4, "GB/s")
    elif case == "attention":
        E, S, B, H = 1024, args.seq, 2, 16
        q, k_, v_, do = rn(E * S * B), rn(E * S * B), rn(E * S * B), rn(E * S * B)
        o, dq, dk, dv = (em(E * S * B) for _ in range(4))
        lse = em(S * H * B)

        def fn():
            call("fb_attn_fwd", P(q), P(k_), P(v_), None, P(o), P(lse), E, E, S, S, B, H, 1)
            call("fb_attn_bwd", P(q), P(k_), P(v_), None, P(o), P(lse), P(do), P(dq), P(dk), P(dv), E, E, S, S, B, H, 1)
        work = (3.5 * 0.5 * 4.0 * S * S * (E // H) * H * B, "TFLOP/s")
    elif case == "lstm":
        I, Hd, T, B = 512, 512, 32, 64
        Wi, Wh, b, x = rn(4 * Hd * I) * 0.05, rn(4 * Hd * Hd) * 0.05, rn(4 * Hd) * 0.1, rn(I * T * B)
        out, hT, cT, dout = em(Hd * T * B), em(Hd * B), em(Hd * B), rn(Hd * T * B)
        cache = em(lib.raw().fb_lstm_cache_bytes(I, Hd, T, B) // 4)
        dWi, dWh, db, dx = torch.empty_like(Wi), torch.empty_like(Wh), torch.empty_like(b), torch.empty_like(x)

        def fn():
            call("fb_lstm_fwd", P(Wi), P(Wh), P(b), P(x), None, None, P(out), P(hT), P(cT), P(cache), I, Hd, T, B)
            call("fb_lstm_bwd", P(Wi), P(Wh), P(x), None, None, P(out), P(cache), P(dout), None, None, P(dWi), P(dWh), P(db), P(dx), I, Hd, T, B)
        work = (6.0 * 2 * 4 * Hd * (I + Hd) * T * B / 2, "TFLOP/s")
    elif case == "gru":
        I, Hd, T, B = 512, 512, 32, 64
        Wi, Wh, b, x = rn(3 * Hd * I) * 0.05, rn(3 * Hd * Hd) * 0.05, rn(3 * Hd) * 0.1, rn(I * T * B)
        out, hT, dout = em(Hd * T * B), em(Hd * B), rn(Hd * T * B)
        cache = em(lib.raw().fb_gru_cache_bytes(I, Hd, T, B) // 4)
        dWi, dWh, db, dx = torch.empty_like(Wi), torch.empty_like(Wh), torch.empty_like(b), torch.empty_like(x)

        def fn():
            call("fb_gru_fwd", P(Wi), P(Wh), P(b), P(x), None, P(out), P(hT), P(cache), I, Hd, T, B)
            call("fb_gru_bwd", P(Wi), P(Wh), P(x), None, P(out), P(cache), P(dout), None, P(dWi), P(dWh), P(db), P(dx), I, Hd, T, B)
        work = (6.0 * 2 * 3 * Hd * (I + Hd) * T * B / 2, "TFLOP/s")
    elif case == "xent":
        c, n = 1000, 8192
        yh, lab = rn(c * n), torch.randint(1, c + 1, (n,), device="cuda", dtype=torch.int32)
        loss, d = em(1), em(c * n)
        fn = lambda: call("fb_logitcrossentropy_labels", P(yh), P(lab), P(loss), P(d), c, n, 1.0)
        work = (2.0 * c * n * 4, "GB/s")
    else:
        raise SystemExit(f"unknown case {case}; cases:\n{CASES}")

    for _ in range(args.iters):
        fn()
    torch.cuda.synchronize()
    if args.time:
        times = []
        for _ in range(10):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        ms = float(np.median(times))
        q, unit = work
        rate = q / (ms * 1e-3) / (1e12 if unit == "TFLOP/s" else 1e9)
        print(f"{case}: median {ms:.4f} ms over 10 L2-flushed iterations -> {rate:.1f} {unit} (algorithmic)")
    err = C.c_int32(0)
    lib.call("fb_device_error", h, st(), C.byref(err))
    assert err.value == 0, "a kernel recorded a bounded-wait timeout"


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
    ap.add_argument("--no-defer", dest="no_defer", action="store_true",
                    help="N > 1: gather the updated parameter blocks inside the step that made them instead of beside the next forward pass")
    ap.add_argument("--eager", action="store_true", help="launch every kernel from the host each step instead of replaying a CUDA graph")
    ap.add_argument("--config", type=int, default=5, choices=[1, 2, 3, 4, 5],
                    help="5 (default): the data-parallel MLP the headline metric is quoted on (at 1 GPU its line carries "
                         "configurations 1-4 under `configs`); 1-4: only that single-GPU configuration, one line each")
    ap.add_argument("--no-configs", dest="no_configs", action="store_true", help="1 GPU: leave configurations 1-4 out of the line")
    ap.add_argument("--case", default=None, help="run one single-kernel profiling case instead of the benchmark:\n" + CASES)
    ap.add_argument("--iters", type=int, default=3, help="--case: untimed iterations")
    ap.add_argument("--time", action="store_true", help="--case: time the case with CUDA events")
    ap.add_argument("--batch", type=int, default=4096, help="--case gemm_*: batch size (8192 = the headline shape)")
    ap.add_argument("--seq", type=int, default=1024, help="--case attention: sequence length")
    args = ap.parse_args()
    if args.case is not None:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    elif args.config != 5:
        for line in small_config_lines(args.config, args.steps, args.warmup):
            print(json.dumps(line), flush=True)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
