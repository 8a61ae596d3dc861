"""Small single-kernel workloads for Nsight Compute captures and CUDA-event timing.

    python flux.jl_b200/profile_cases.py <case> [--iters N] [--time] [--batch B]

Cases (each holds well under a few GB on the device; inputs exceed the 126 MB L2 so DRAM counters mean something):
    gemm_fwd    Dense 4096=>4096 forward, batch 4096 (3xTF32 tcgen05 GEMM, K-major x MN-major)
    gemm_dw     the dW GEMM of the same layer (MN-major x MN-major, K = batch)
    gemm_dx     the dX GEMM of the same layer (K-major x K-major)
    layernorm   LayerNorm(4096) forward + backward on 4096 x 8192
    batchnorm   BatchNorm(256, relu) training forward + backward on 32 x 32 x 256 x 128
    adam        Adam step over 32 Mi parameters in 4 leaves
    attention   causal attention forward + backward, E = 1024, 16 heads, S = 1024, B = 2
    lstm        LSTM(512=>512) forward + backward, T = 32, B = 64
    xent        logitcrossentropy forward + backward, 1000 x 8192
With --time the case is also timed with CUDA events (L2 flushed between iterations) and achieved GB/s or TFLOP/s
against the algorithmic bytes / flops is printed.
"""
from __future__ import annotations

import argparse
import ctypes as C
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from fluxb200 import lib  # noqa: E402


def P(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--time", action="store_true")
    ap.add_argument("--batch", type=int, default=4096, help="batch size of the gemm_* cases (8192 = the headline bench shape)")
    args = ap.parse_args()
    torch.cuda.set_device(0)
    h = C.c_void_p()
    lib.call("fb_ctx_create", 0, C.byref(h))
    st = lambda: C.c_void_p(torch.cuda.current_stream().cuda_stream)
    call = lambda name, *a: lib.call(name, h, st(), *a)
    g = torch.Generator(device="cuda").manual_seed(0)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    case = args.case
    work = None      # (algorithmic quantity per iteration, unit)
    if case in ("gemm_fwd", "gemm_dw", "gemm_dx"):
        n, d = args.batch, 4096
        W, x, dy = rn(d * d) * 0.02, rn(n * d), rn(n * d)
        y, dW, dx, b = torch.empty(n * d, device="cuda"), torch.empty(d * d, device="cuda"), torch.empty(n * d, device="cuda"), rn(d)
        if case == "gemm_fwd":
            fn = lambda: call("fb_dense_fwd", 4, 0, P(W), P(b), P(x), P(y), None, d, d, n)
        elif case == "gemm_dw":
            fn = lambda: call("fb_gemm_f32", 0, 1, d, d, n, P(dy), d, P(x), d, P(dW), d, 0, 0)       # dW = dy * x'
        else:
            fn = lambda: call("fb_gemm_f32", 1, 0, d, n, d, P(W), d, P(dy), d, P(dx), d, 0, 0)       # dx = W' * dy
        work = (2.0 * n * d * d, "TFLOP/s")
    elif case == "layernorm":
        d, n = 4096, 8192
        x, dy, gam, bet = rn(d * n), rn(d * n), rn(d), rn(d)
        y, dx, mean, rstd, dg, db = (torch.empty(d * n, device="cuda"), torch.empty(d * n, device="cuda"), torch.empty(n, device="cuda"),
                                     torch.empty(n, device="cuda"), torch.empty(d, device="cuda"), torch.empty(d, device="cuda"))

        def fn():
            call("fb_layernorm_fwd", P(x), P(gam), P(bet), P(y), P(mean), P(rstd), d, n, 1e-5, 0)
            call("fb_layernorm_bwd", P(x), P(gam), P(bet), P(mean), P(rstd), P(dy), P(dx), P(dg), P(db), d, n, 0)
        work = (5.0 * d * n * 4, "GB/s")
    elif case == "batchnorm":
        s, c, n = 1024, 256, 128
        x, dy, gam, bet = rn(s * c * n) * 2 + 0.5, rn(s * c * n), rn(c), rn(c)
        rm, rv = torch.zeros(c, device="cuda"), torch.ones(c, device="cuda")
        y, dx = torch.empty_like(x), torch.empty_like(x)
        sm, sr, dg, db = (torch.empty(c, device="cuda") for _ in range(4))

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
        E, S, B, H = 1024, 1024, 2, 16
        q, k_, v_, do = rn(E * S * B), rn(E * S * B), rn(E * S * B), rn(E * S * B)
        o, dq, dk, dv = (torch.empty(E * S * B, device="cuda") for _ in range(4))
        lse = torch.empty(S * H * B, device="cuda")

        def fn():
            call("fb_attn_fwd", P(q), P(k_), P(v_), None, P(o), P(lse), E, E, S, S, B, H, 1)
            call("fb_attn_bwd", P(q), P(k_), P(v_), None, P(o), P(lse), P(do), P(dq), P(dk), P(dv), E, E, S, S, B, H, 1)
        work = (3.5 * 0.5 * 4.0 * S * S * (E // H) * H * B, "TFLOP/s")
    elif case == "lstm":
        I, Hd, T, B = 512, 512, 32, 64
        Wi, Wh, b, x = rn(4 * Hd * I) * 0.05, rn(4 * Hd * Hd) * 0.05, rn(4 * Hd) * 0.1, rn(I * T * B)
        out, hT, cT, dout = torch.empty(Hd * T * B, device="cuda"), torch.empty(Hd * B, device="cuda"), torch.empty(Hd * B, device="cuda"), rn(Hd * T * B)
        cache = torch.empty(lib.raw().fb_lstm_cache_bytes(I, Hd, T, B) // 4, device="cuda")
        dWi, dWh, db, dx = torch.empty_like(Wi), torch.empty_like(Wh), torch.empty_like(b), torch.empty_like(x)

        def fn():
            call("fb_lstm_fwd", P(Wi), P(Wh), P(b), P(x), None, None, P(out), P(hT), P(cT), P(cache), I, Hd, T, B)
            call("fb_lstm_bwd", P(Wi), P(Wh), P(x), None, None, P(out), P(cache), P(dout), None, None, P(dWi), P(dWh), P(db), P(dx), I, Hd, T, B)
        work = (6.0 * 2 * 4 * Hd * (I + Hd) * T * B / 2, "TFLOP/s")
    elif case == "xent":
        c, n = 1000, 8192
        yh, lab = rn(c * n), torch.randint(1, c + 1, (n,), device="cuda", dtype=torch.int32)
        loss, d = torch.empty(1, device="cuda"), torch.empty(c * n, device="cuda")
        fn = lambda: call("fb_logitcrossentropy_labels", P(yh), P(lab), P(loss), P(d), c, n, 1.0)
        work = (2.0 * c * n * 4, "GB/s")
    else:
        raise SystemExit(f"unknown case {case}")

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


if __name__ == "__main__":
    main()
