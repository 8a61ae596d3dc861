"""The allocation-free LayerNorm backward (fb_layernorm_bwd_noalloc) against the regular entry point and the oracle.

The entry point serves callers that may not allocate device memory (a fixed start-up memory budget, code under
stream capture, runtime threads that must avoid cudaMalloc's implicit synchronisation); its scratch is a fixed
array inside the library.  This file is collected last so that a failure here cannot hide another test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import flux_oracle as O
from util import P, close, dempty, dev, host, stream

pytestmark = pytest.mark.gpu


def _run_pair(lib, ctx, d, n, seed, act=0):
    rng = np.random.default_rng(seed)
    x = (rng.normal(size=(d, n)) * 1.5 + 0.2).astype(np.float32)
    g = (rng.normal(size=d) * 0.5 + 1).astype(np.float32)
    b = (rng.normal(size=d) * 0.5).astype(np.float32)
    dy = rng.normal(size=(d, n)).astype(np.float32)
    tx, tg, tb, tdy = dev(x), dev(g), dev(b), dev(dy)
    y, mean, rstd = dempty(d, n), dempty(n), dempty(n)
    lib.call("fb_layernorm_fwd", ctx, stream(), P(tx), P(tg), P(tb), P(y), P(mean), P(rstd), d, n, 1e-5, act)
    ref = [dempty(d, n), dempty(d), dempty(d)]
    got = [torch.full_like(ref[0], float("nan")), torch.full_like(ref[1], float("nan")), torch.full_like(ref[2], float("nan"))]
    lib.call("fb_layernorm_bwd", ctx, stream(), P(tx), P(tg), P(tb), P(mean), P(rstd), P(tdy), P(ref[0]), P(ref[1]), P(ref[2]), d, n, act)
    lib.call("fb_layernorm_bwd_noalloc", stream(), P(tx), P(tg), P(tb), P(mean), P(rstd), P(tdy), P(got[0]), P(got[1]), P(got[2]), d, n, act)
    torch.cuda.synchronize()
    acts = {0: "identity", 2: "tanh"}
    x64, g64, b64, dy64 = (a.astype(np.float64) for a in (x, g, b, dy))
    oracle = O.layernorm_bwd(x64, g64, b64, dy64, 1e-5, acts[act])
    rs = O.layernorm_fwd(x64, g64, b64, 1e-5, "identity", return_stats=True)[2]
    term = float(np.max(np.abs(dy64 * g64.reshape(-1, 1) * rs)))
    for a, r, o, shape, name in zip(got, ref, oracle, [(d, n), (d,), (d,)], ["dx", "dgamma", "dbeta"]):
        close(host(a, shape), host(r, shape), rtol=2e-4, atol_scale=2e-4, name=f"{name} d={d} n={n} (against fb_layernorm_bwd)")
        floor = 1e-2 * term if name == "dx" else 0.0   # dx is a difference of terms of size |dy * gamma * rstd|
        np.testing.assert_allclose(host(a, shape), o, rtol=2e-4, atol=2e-4 * max(float(np.max(np.abs(o))), floor),
                                   err_msg=f"{name} d={d} n={n} (against the oracle)")


def test_noalloc_layernorm_bwd_matches_regular_entry_point_twice():
    from fluxb200 import lib
    ctx = C.c_void_p()
    lib.call("fb_ctx_create", 0, C.byref(ctx))
    try:
        # two calls in a row share the fixed scratch: the second (smaller, different data, odd width) must not see
        # anything the first left behind
        _run_pair(lib, ctx, 4096, 700, seed=1)
        _run_pair(lib, ctx, 1000, 37, seed=2)
        _run_pair(lib, ctx, 257, 9, seed=3, act=2)
        # 16384 features x 300 rows: 296 row groups would need more partials than the fixed array holds, so the
        # number of groups is cut to what fits (128)
        _run_pair(lib, ctx, 16384, 300, seed=4)
        # a width beyond the fixed scratch is rejected with a clear message, nothing is launched
        big = (4 << 20) // 2 + 4
        a = dempty(8)
        st = lib.raw().fb_layernorm_bwd_noalloc(stream(), P(a), P(a), P(a), P(a), P(a), P(a), P(a), P(a), P(a), big, 1, 0)
        assert st == -7 and "exceeds the fixed scratch" in lib.last_error()
    finally:
        lib.call("fb_ctx_destroy", ctx)
