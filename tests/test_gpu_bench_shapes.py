"""GPU parity at the shapes the benchmark configurations run (the code paths a small shape never enters: the
two-CTA GEMM over several waves and with its split-K tail, the multi-row LayerNorm backward ring, the persistent
recurrent kernels at 256 steps, attention at 32 key blocks, BatchNorm over 131 072 values per channel), through the
C ABI against the float64 oracle.  Where the full float64 result would take minutes on the host, rows and columns
are sampled so that every output tile of the kernel is touched."""
import ctypes as C

import numpy as np
import pytest
import torch

import flux_oracle as O
from util import P, close, dempty, dev, host, stream

pytestmark = pytest.mark.gpu

ACT = {"identity": 0, "relu": 1, "tanh": 2, "sigmoid": 3, "gelu_tanh": 4, "gelu_erf": 5}


@pytest.fixture(scope="module")
def fb():
    from fluxb200 import lib
    h = C.c_void_p()
    lib.call("fb_ctx_create", 0, C.byref(h))

    class FB:
        ctx = h
        raw = lib.raw()

        @staticmethod
        def call(name, *a):
            lib.call(name, h, stream(), *a)

        @staticmethod
        def device_error():
            out = C.c_int32(0)
            lib.call("fb_device_error", h, stream(), C.byref(out))
            return out.value

    yield FB
    torch.cuda.synchronize()
    assert FB.device_error() == 0, "a kernel recorded a bounded-wait timeout"
    lib.call("fb_ctx_destroy", h)


def _two_per_block(total, block, rng):
    """Two indices out of every `block` consecutive ones: every tile row / column of the kernel is sampled."""
    idx = []
    for s in range(0, total, block):
        hi = min(s + block, total)
        idx += list(rng.choice(np.arange(s, hi), size=min(2, hi - s), replace=False))
    return np.array(sorted(idx))


# ---------------------------------------------------- Dense 4096 => 4096 gelu (the benchmark's dominant GEMMs) ---
@pytest.mark.parametrize("n", [1024, 2048, 4096, 8192])
def test_dense_4096_gelu_at_benchmark_batches(fb, n):
    """Per-GPU batches of the data-parallel benchmark at 8 / 4 / 2 / 1 GPUs: 64, 128, 256 and 512 two-CTA tiles on
    74 SM pairs, i.e. one wave, one wave + a split-K tail, and several waves + a tail."""
    d = 4096
    rng = np.random.default_rng(n)
    W = O.glorot_uniform(rng, d, d)
    b = (rng.normal(size=d) * 0.1).astype(np.float32)
    x = rng.normal(size=(d, n)).astype(np.float32)
    dy = rng.normal(size=(d, n)).astype(np.float32)
    tW, tb, tx, tdy = dev(W), dev(b), dev(x), dev(dy)
    y, z, delta = dempty(d, n), dempty(d, n), dempty(d, n)
    dW, db, dx = dempty(d, d), dempty(d), dempty(d, n)
    fb.call("fb_dense_fwd", ACT["gelu_tanh"], 0, P(tW), P(tb), P(tx), P(y), P(z), d, d, n)
    fb.call("fb_dense_bwd", ACT["gelu_tanh"], 0, P(tW), P(tx), P(y), P(z), P(tdy), P(delta), P(dW), P(db), P(dx), d, d, n)
    torch.cuda.synchronize()
    W64, x64 = W.astype(np.float64), x.astype(np.float64)
    z64 = W64 @ x64 + b.astype(np.float64)[:, None]
    close(host(z, (d, n)), z64, name="z")
    close(host(y, (d, n)), O.act("gelu_tanh", z64), name="y")
    delta64 = dy.astype(np.float64) * O.act_grad("gelu_tanh", z64)
    close(host(delta, (d, n)), delta64, name="delta")
    close(host(db, (d,)), delta64.sum(1), name="db")
    gW, gx = host(dW, (d, d)), host(dx, (d, n))
    # dW[out, in] = delta x': the kernel's tiles are 256 (in) x 256 (out)
    J = _two_per_block(d, 128, rng)
    close(gW[:, J], delta64 @ x64[J, :].T, name="dW columns")
    close(gW[J, :], delta64[J, :] @ x64.T, name="dW rows")
    # dx[in, n] = W' delta: tiles are 256 (n) x 256 (in)
    cols = _two_per_block(n, 128, rng)
    close(gx[:, cols], W64.T @ delta64[:, cols], name="dx columns")
    close(gx[J, :], W64[:, J].T @ delta64, name="dx rows")


def test_dense_classifier_1000x4096_batch_8192(fb):
    """The benchmark's last layer (out = 1000 is not a multiple of the tile width: ragged last tile column)."""
    o, d, n = 1000, 4096, 8192
    rng = np.random.default_rng(7)
    W = O.glorot_uniform(rng, o, d)
    b = (rng.normal(size=o) * 0.1).astype(np.float32)
    x = rng.normal(size=(d, n)).astype(np.float32)
    dy = (rng.normal(size=(o, n)) / n).astype(np.float32)
    tW, tb, tx, tdy = dev(W), dev(b), dev(x), dev(dy)
    y, dW, db, dx = dempty(o, n), dempty(o, d), dempty(o), dempty(d, n)
    fb.call("fb_dense_fwd", 0, 0, P(tW), P(tb), P(tx), P(y), None, o, d, n)
    fb.call("fb_dense_bwd", 0, 0, P(tW), P(tx), P(y), None, P(tdy), None, P(dW), P(db), P(dx), o, d, n)
    W64, x64, dy64 = W.astype(np.float64), x.astype(np.float64), dy.astype(np.float64)
    close(host(y, (o, n)), W64 @ x64 + b.astype(np.float64)[:, None], name="y")
    close(host(dW, (o, d)), dy64 @ x64.T, name="dW")
    close(host(db, (o,)), dy64.sum(1), name="db")
    close(host(dx, (d, n)), W64.T @ dy64, name="dx")


# ------------------------------------------------------------- LayerNorm(4096) at the benchmark batches ---
@pytest.mark.parametrize("n", [8192, 16384])
def test_layernorm_4096_multi_row_ring(fb, n):
    """Every CTA of the backward kernel owns ~28 (55) rows: the shared-memory ring wraps and its phases flip."""
    d = 4096
    rng = np.random.default_rng(n + 1)
    x = (rng.normal(size=(d, n)) * 1.3 + 0.2).astype(np.float32)
    g = (rng.normal(size=d) * 0.5 + 1).astype(np.float32)
    b = (rng.normal(size=d) * 0.5).astype(np.float32)
    dy = rng.normal(size=(d, n)).astype(np.float32)
    tx, tg, tb, tdy = dev(x), dev(g), dev(b), dev(dy)
    y, mean, rstd = dempty(d, n), dempty(n), dempty(n)
    dx, dg, dbeta = dempty(d, n), dempty(d), dempty(d)
    fb.call("fb_layernorm_fwd", P(tx), P(tg), P(tb), P(y), P(mean), P(rstd), d, n, 1e-5, 0)
    fb.call("fb_layernorm_bwd", P(tx), P(tg), P(tb), P(mean), P(rstd), P(tdy), P(dx), P(dg), P(dbeta), d, n, 0)
    x64, g64, b64, dy64 = (a.astype(np.float64) for a in (x, g, b, dy))
    yref, mu, rs = O.layernorm_fwd(x64, g64, b64, 1e-5, "identity", return_stats=True)
    close(host(y, (d, n)), yref, name="y")
    close(host(rstd, (n,)), rs.reshape(-1), name="rstd")
    dxr, dgr, dbr = O.layernorm_bwd(x64, g64, b64, dy64, 1e-5, "identity")
    term = float(np.max(np.abs(dy64 * g64.reshape(-1, 1) * rs)))
    np.testing.assert_allclose(host(dx, (d, n)), dxr, rtol=2e-4, atol=2e-4 * max(float(np.max(np.abs(dxr))), 1e-2 * term), err_msg="dx")
    close(host(dg, (d,)), dgr, name="dgamma", rtol=2e-4, atol_scale=2e-4)
    close(host(dbeta, (d,)), dbr, name="dbeta", rtol=2e-4, atol_scale=2e-4)


# ------------------------------------------------------------------ BatchNorm(256, relu) on 32x32x256x128 ---
def test_batchnorm_32x32x256x128(fb):
    shape = (32, 32, 256, 128)
    s, c, n = 1024, 256, 128
    rng = np.random.default_rng(2)
    x = (rng.standard_normal(shape, dtype=np.float32) * 2 + 0.5)
    g = (rng.normal(size=c) * 0.5 + 1.2).astype(np.float32)
    b = (rng.normal(size=c) * 0.5).astype(np.float32)
    dy = rng.standard_normal(shape, dtype=np.float32)
    tx, tg, tb, tdy = dev(x), dev(g), dev(b), dev(dy)
    rm, rv = dev(np.zeros(c, np.float32)), dev(np.ones(c, np.float32))
    y, sm, sr = dempty(*shape), dempty(c), dempty(c)
    dx, dg, dbeta = dempty(*shape), dempty(c), dempty(c)
    fb.call("fb_batchnorm_fwd_train", P(tx), P(tg), P(tb), P(rm), P(rv), P(y), P(sm), P(sr), s, c, n, 1e-5, 0.1, ACT["relu"], 1)
    fb.call("fb_batchnorm_bwd", P(tx), P(tg), P(tb), P(sm), P(sr), P(tdy), P(dx), P(dg), P(dbeta), s, c, n, ACT["relu"])
    x64, g64, b64, dy64 = (a.astype(np.float64) for a in (x, g, b, dy))
    yref, nm, nv = O.batchnorm_fwd_train(x64, g64, b64, np.zeros(c), np.ones(c), 0.1, 1e-5, "relu")
    close(host(y, shape), yref, name="y")
    close(host(rm, (c,)), nm, name="running mean")
    close(host(rv, (c,)), nv, name="running var")
    dxr, dgr, dbr = O.batchnorm_bwd(x64, g64, b64, dy64, 1e-5, "relu")
    got_dx = host(dx, shape).astype(np.float64)
    unsure = np.abs(O.batchnorm_fwd_train(x64, g64, b64, None, None, sigma="identity", track_stats=False)[0]) < 1e-5
    got_dx[unsure] = dxr[unsure]
    close(got_dx, dxr, name="dx", rtol=2e-4, atol_scale=2e-4)
    # an element within rounding of the relu threshold may flip in dgamma / dbeta: 131 072-term sums absorb it
    close(host(dg, (c,)), dgr, name="dgamma", rtol=2e-4, atol_scale=2e-4)
    close(host(dbeta, (c,)), dbr, name="dbeta", rtol=2e-4, atol_scale=2e-4)


# ------------------------------------------------------------ LSTM / GRU (512 => 512), T = 256, B = 64 ---
@pytest.mark.parametrize("kind", ["lstm", "gru"])
def test_recurrent_512_256_64(fb, kind):
    I = H = 512
    T, B = 256, 64
    ng = 4 if kind == "lstm" else 3
    r1 = np.random.default_rng(1)
    Wi, Wh = O.glorot_uniform(r1, ng * H, I), O.glorot_uniform(r1, ng * H, H)
    b = np.zeros(ng * H, np.float32)
    x = np.random.default_rng(3).standard_normal((I, T, B), dtype=np.float32)
    nbytes = getattr(fb.raw, f"fb_{kind}_cache_bytes")(I, H, T, B)
    cache = torch.empty(nbytes // 4, dtype=torch.float32, device="cuda")
    tWi, tWh, tb, tx = dev(Wi), dev(Wh), dev(b), dev(x)
    out, hT, cT = dempty(H, T, B), dempty(H, B), dempty(H, B)
    Wi64, Wh64, b64, x64 = (a.astype(np.float64) for a in (Wi, Wh, b, x))
    if kind == "lstm":
        fb.call("fb_lstm_fwd", P(tWi), P(tWh), P(tb), P(tx), None, None, P(out), P(hT), P(cT), P(cache), I, H, T, B)
        oref, (href, cref) = O.lstm_scan_fwd(Wi64, Wh64, b64, x64)
        close(host(cT, (H, B)), cref, name="cT")
    else:
        fb.call("fb_gru_fwd", P(tWi), P(tWh), P(tb), P(tx), None, P(out), P(hT), P(cache), I, H, T, B)
        oref, href = O.gru_scan_fwd(Wi64, Wh64, b64, x64)
    close(host(out, (H, T, B)), oref, name="out")
    close(host(hT, (H, B)), href, name="hT")
    dout = O.sum_abs2_bwd(oref)
    tdout = dev(dout, np.float32)
    dWi, dWh, db, dx = dempty(ng * H, I), dempty(ng * H, H), dempty(ng * H), dempty(I, T, B)
    if kind == "lstm":
        fb.call("fb_lstm_bwd", P(tWi), P(tWh), P(tx), None, None, P(out), P(cache), P(tdout), None, None, P(dWi), P(dWh), P(db),
                P(dx), I, H, T, B)
        rWi, rWh, rb, rx = O.lstm_scan_bwd(Wi64, Wh64, b64, x64, dout)
    else:
        fb.call("fb_gru_bwd", P(tWi), P(tWh), P(tx), None, P(out), P(cache), P(tdout), None, P(dWi), P(dWh), P(db), P(dx),
                I, H, T, B)
        rWi, rWh, rb, rx = O.gru_scan_bwd(Wi64, Wh64, b64, x64, dout)
    close(host(dWi, (ng * H, I)), rWi, name="dWi", rtol=2e-4, atol_scale=2e-4)
    close(host(dWh, (ng * H, H)), rWh, name="dWh", rtol=2e-4, atol_scale=2e-4)
    close(host(db, (ng * H,)), rb, name="db", rtol=2e-4, atol_scale=2e-4)
    close(host(dx, (I, T, B)), rx, name="dx", rtol=2e-4, atol_scale=2e-4)


# -------------------------------------------------------- attention: E = 1024, 16 heads, S = 2048, causal ---
def test_attention_1024_16heads_seq2048_causal(fb):
    """32 key blocks per query tile: the stated limit of accumulation in tensor memory in the backward kernels."""
    E, heads, S, B = 1024, 16, 2048, 1
    rng = np.random.default_rng(4)
    q, k, v, do = (rng.standard_normal((E, S, B), dtype=np.float32) for _ in range(4))
    tq, tk, tv, tdo = dev(q), dev(k), dev(v), dev(do)
    o, lse = dempty(E, S, B), dempty(S, heads, B)
    dq, dk, dv = dempty(E, S, B), dempty(E, S, B), dempty(E, S, B)
    fb.call("fb_attn_fwd", P(tq), P(tk), P(tv), None, P(o), P(lse), E, E, S, S, B, heads, 1)
    fb.call("fb_attn_bwd", P(tq), P(tk), P(tv), None, P(o), P(lse), P(tdo), P(dq), P(dk), P(dv), E, E, S, S, B, heads, 1)
    q64, k64, v64, do64 = (a.astype(np.float64) for a in (q, k, v, do))
    mask = O.make_causal_mask(S)
    oref, _ = O.dot_product_attention(q64, k64, v64, None, heads, mask)
    close(host(o, (E, S, B)), oref, name="o")
    rq, rk, rv = O.dot_product_attention_bwd(q64, k64, v64, do64, None, heads, mask)
    close(host(dq, (E, S, B)), rq, name="dq", rtol=2e-4, atol_scale=2e-4)
    close(host(dk, (E, S, B)), rk, name="dk", rtol=2e-4, atol_scale=2e-4)
    close(host(dv, (E, S, B)), rv, name="dv", rtol=2e-4, atol_scale=2e-4)


# ------------------------------------- the data-parallel benchmark model at width 4096, per-GPU batch 1024 ---
def test_dp_mlp_width_4096_batch_1024_loss_and_all_gradients():
    import fluxb200 as F
    D, NB, NC, N = 4096, 8, 1000, 1024
    rng = np.random.default_rng(3)
    blocks = [{"gamma": (1 + 0.1 * rng.normal(size=D)).astype(np.float32), "beta": (0.1 * rng.normal(size=D)).astype(np.float32),
               "W": O.glorot_uniform(rng, D, D), "b": (0.1 * rng.normal(size=D)).astype(np.float32)} for _ in range(NB)]
    head = {"W": O.glorot_uniform(rng, NC, D), "b": np.zeros(NC, np.float32)}
    x = rng.standard_normal((D, N), dtype=np.float32)
    labels = rng.integers(1, NC + 1, size=N)
    layers = []
    for blk in blocks:
        ln = F.LayerNorm(D)
        ln.diag.scale, ln.diag.bias = F.gpu(blk["gamma"]), F.gpu(blk["beta"])
        layers += [ln, F.Dense(blk["W"], blk["b"], "gelu")]
    layers.append(F.Dense(head["W"], head["b"]))
    model = F.Chain(*layers)
    xg, yg = F.gpu(x), F.onehotbatch(labels, NC)
    loss, (g,) = F.withgradient(lambda m: F.logitcrossentropy(m(xg), yg), model)
    to64 = lambda dct: {k: v.astype(np.float64) for k, v in dct.items()}
    lref, gb, gh = O.dp_mlp_fwd_bwd([to64(b) for b in blocks], to64(head), x.astype(np.float64), O.onehotbatch(labels, NC, np.float64))
    close(loss, lref, name="loss")
    for i in range(NB):
        gl = g["layers"]
        close(F.cpu(gl[2 * i]["diag"]["scale"]), gb[i]["gamma"], name=f"dgamma {i}", rtol=2e-4, atol_scale=2e-4)
        close(F.cpu(gl[2 * i]["diag"]["bias"]), gb[i]["beta"], name=f"dbeta {i}", rtol=2e-4, atol_scale=2e-4)
        close(F.cpu(gl[2 * i + 1]["weight"]), gb[i]["W"], name=f"dW {i}", rtol=2e-4, atol_scale=2e-4)
        close(F.cpu(gl[2 * i + 1]["bias"]), gb[i]["b"], name=f"db {i}", rtol=2e-4, atol_scale=2e-4)
    close(F.cpu(g["layers"][-1]["weight"]), gh["W"], name="dW head", rtol=2e-4, atol_scale=2e-4)
    close(F.cpu(g["layers"][-1]["bias"]), gh["b"], name="db head", rtol=2e-4, atol_scale=2e-4)
    assert F.context().device_error() == 0
