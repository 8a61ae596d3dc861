"""GPU parity tests: every compute entry point of libfluxb200.so, called through the C ABI, against the
numpy oracle on the same seeded inputs (fp32 tolerance rtol = 1e-4, atol = 1e-4 * max|ref|)."""
import ctypes as C

import numpy as np
import pytest
import torch

import flux_oracle as O
from util import P, close, dempty, dev, host, stream

pytestmark = pytest.mark.gpu

ACT = {"identity": 0, "relu": 1, "tanh": 2, "sigmoid": 3, "gelu_tanh": 4, "gelu_erf": 5}
PREC = {"default": 0, "simt": 1, "3xtf32": 2, "tf32": 3, "pair": 4}


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
        def status(name, *a):
            return getattr(lib.raw(), name)(h, stream(), *a), lib.last_error()

        @staticmethod
        def device_error():
            out = C.c_int32(0)
            lib.call("fb_device_error", h, stream(), C.byref(out))
            return out.value

    yield FB
    torch.cuda.synchronize()
    assert FB.device_error() == 0, "a kernel recorded a bounded-wait timeout"
    lib.call("fb_ctx_destroy", h)


def f64(*arrs):
    return [None if a is None else np.asarray(a, dtype=np.float64) for a in arrs]


# ------------------------------------------------------------------------------------ matmul ---
@pytest.mark.parametrize("prec", ["simt", "3xtf32"])
@pytest.mark.parametrize("ta,tb", [(0, 0), (1, 0), (0, 1), (1, 1)])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (200, 136, 100), (512, 384, 1000), (4, 8, 12), (1000, 520, 36)])
def test_gemm_all_layouts(fb, prec, ta, tb, m, n, k):
    rng = np.random.default_rng(m * 7 + n * 3 + k + ta * 2 + tb)
    A = rng.normal(size=(k, m) if ta else (m, k)).astype(np.float32)
    B = rng.normal(size=(n, k) if tb else (k, n)).astype(np.float32)
    dA, dB, dC = dev(A), dev(B), dempty(m, n)
    fb.call("fb_gemm_f32", ta, tb, m, n, k, P(dA), A.shape[0], P(dB), B.shape[0], P(dC), m, 0, PREC[prec])
    ref = (A.T if ta else A).astype(np.float64) @ (B.T if tb else B).astype(np.float64)
    close(host(dC, (m, n)), ref, name=f"gemm {prec} ta={ta} tb={tb}")
    # accumulate: C += op(A) op(B)
    fb.call("fb_gemm_f32", ta, tb, m, n, k, P(dA), A.shape[0], P(dB), B.shape[0], P(dC), m, 1, PREC[prec])
    close(host(dC, (m, n)), 2 * ref, name="gemm accumulate")


@pytest.mark.parametrize("ta,tb", [(0, 0), (1, 0), (0, 1), (1, 1)])
@pytest.mark.parametrize("m,n,k", [(512, 768, 300), (260, 1000, 2100), (1024, 256, 4100)])
def test_gemm_cta_pair_tiles(fb, ta, tb, m, n, k):
    """The cta_group::2 variant (256 x 256 tiles computed by two CTAs) in all four operand layouts, with ragged
    edges and more than one accumulation segment."""
    rng = np.random.default_rng(m + n + k + ta * 2 + tb)
    A = rng.normal(size=(k, m) if ta else (m, k)).astype(np.float32)
    B = rng.normal(size=(n, k) if tb else (k, n)).astype(np.float32)
    dA, dB, dC = dev(A), dev(B), dempty(m, n)
    fb.call("fb_gemm_f32", ta, tb, m, n, k, P(dA), A.shape[0], P(dB), B.shape[0], P(dC), m, 0, PREC["pair"])
    ref = (A.T if ta else A).astype(np.float64) @ (B.T if tb else B).astype(np.float64)
    close(host(dC, (m, n)), ref, name=f"pair gemm ta={ta} tb={tb}")
    fb.call("fb_gemm_f32", ta, tb, m, n, k, P(dA), A.shape[0], P(dB), B.shape[0], P(dC), m, 1, PREC["pair"])
    close(host(dC, (m, n)), 2 * ref, name="pair gemm accumulate")


def test_gemm_3xtf32_is_fp32_accurate_and_tf32_is_not(fb):
    """The error-compensated path must stay far inside 1e-4 at K = 4096; one TF32 pass does not."""
    rng = np.random.default_rng(0)
    m, n, k = 256, 512, 4096
    A = rng.normal(size=(m, k)).astype(np.float32)
    B = rng.normal(size=(k, n)).astype(np.float32)
    ref = A.astype(np.float64) @ B.astype(np.float64)
    dA, dB, dC = dev(A), dev(B), dempty(m, n)
    errs = {}
    for prec in ("3xtf32", "tf32", "simt"):
        fb.call("fb_gemm_f32", 0, 0, m, n, k, P(dA), m, P(dB), k, P(dC), m, 0, PREC[prec])
        errs[prec] = np.max(np.abs(host(dC, (m, n)) - ref)) / np.max(np.abs(ref))
    # the tensor core accumulates with truncation; K is cut into 2048-long segments to bound the drift
    assert errs["3xtf32"] < 3e-5, errs
    assert errs["simt"] < 5e-6, errs
    assert 1e-4 < errs["tf32"] < 5e-3, errs


def test_gemm_3xtf32_long_k_stays_inside_tolerance(fb):
    """K = 16384 (the LSTM dWi reduction length): segment-wise accumulation keeps the error far inside 1e-4."""
    rng = np.random.default_rng(1)
    m, n, k = 256, 384, 16384
    A = rng.normal(size=(m, k)).astype(np.float32)
    B = rng.normal(size=(n, k)).astype(np.float32)
    ref = A.astype(np.float64) @ B.astype(np.float64).T
    dA, dB, dC = dev(A), dev(B), dempty(m, n)
    fb.call("fb_gemm_f32", 0, 1, m, n, k, P(dA), m, P(dB), n, P(dC), m, 0, PREC["3xtf32"])
    err = np.max(np.abs(host(dC, (m, n)) - ref)) / np.max(np.abs(ref))
    assert err < 3e-5, err


def test_gemm_rejects_bad_arguments(fb):
    st, msg = fb.status("fb_gemm_f32", 0, 0, 4, 4, 4, None, 4, None, 4, None, 4, 0, 0)
    assert st == -1 and "NULL" in msg
    a = dempty(16)
    st, msg = fb.status("fb_gemm_f32", 0, 0, 4, 4, 4, P(a), 2, P(a), 4, P(a), 4, 0, 0)
    assert st == -2
    # unaligned leading dimension cannot go to the tensor-core kernel when it is forced
    st, msg = fb.status("fb_gemm_f32", 0, 0, 6, 6, 6, P(a), 6, P(a), 6, P(dempty(36)), 6, 0, PREC["3xtf32"])
    assert st == -7 and "tensor-core" in msg


# ------------------------------------------------------------------------------------- Dense ---
def test_dense_ones_known_answers(fb):
    """test/layers/basic.jl:85-89."""
    for out, ncol, xs, bias in [(1, 1, np.ones((10, 1)), True), (1, 2, np.ones((10, 2)), True),
                                (2, 1, np.ones((10, 1)), True),
                                (2, 2, np.concatenate([np.ones((10, 1)), 2 * np.ones((10, 1))], 1), True),
                                (2, 2, np.concatenate([np.ones((10, 1)), 2 * np.ones((10, 1))], 1), False)]:
        W, b = dev(np.ones((out, 10), np.float32)), dev(np.zeros(out, np.float32))
        x, y = dev(xs, np.float32), dempty(out, ncol)
        fb.call("fb_dense_fwd", 0, 0, P(W), P(b) if bias else None, P(x), P(y), None, out, 10, ncol)
        assert (host(y, (out, ncol)) == O.dense_fwd(np.ones((out, 10)), None, xs)).all()


@pytest.mark.parametrize("prec", ["simt", "3xtf32", "default"])
@pytest.mark.parametrize("act", list(ACT))
@pytest.mark.parametrize("out_dim,in_dim,n", [(128, 64, 256), (512, 784, 1024), (10, 512, 64), (1000, 256, 96), (36, 20, 7)])
def test_dense_fwd_bwd(fb, prec, act, out_dim, in_dim, n):
    if prec == "3xtf32" and (out_dim % 4 or in_dim % 4):
        pytest.skip("forced tensor-core path needs leading dimensions that are multiples of 4")
    if act not in ("relu", "gelu_tanh", "identity") and (out_dim, in_dim, n) != (128, 64, 256):
        pytest.skip("remaining activations are covered on one shape")
    rng = np.random.default_rng(out_dim + in_dim + n)
    W = O.glorot_uniform(rng, out_dim, in_dim)
    b = (rng.normal(size=out_dim) * 0.1).astype(np.float32)
    x = rng.normal(size=(in_dim, n)).astype(np.float32)
    dy = rng.normal(size=(out_dim, n)).astype(np.float32)
    dW_, db_, dx_, y_, z_ = dempty(out_dim, in_dim), dempty(out_dim), dempty(in_dim, n), dempty(out_dim, n), dempty(out_dim, n)
    delta = dempty(out_dim, n)
    tW, tb_, tx, tdy = dev(W), dev(b), dev(x), dev(dy)
    fb.call("fb_dense_fwd", ACT[act], PREC[prec], P(tW), P(tb_), P(tx), P(y_), P(z_), out_dim, in_dim, n)
    W64, b64, x64, dy64 = f64(W, b, x, dy)
    yref, zref = O.dense_fwd(W64, b64, x64, act, return_preact=True)
    close(host(y_, (out_dim, n)), yref, name="y")
    close(host(z_, (out_dim, n)), zref, name="z")
    fb.call("fb_dense_bwd", ACT[act], PREC[prec], P(tW), P(tx), P(y_), P(z_), P(tdy), P(delta), P(dW_), P(db_), P(dx_),
            out_dim, in_dim, n)
    dW, db, dx = O.dense_bwd(W64, b64, x64, dy64, act)
    if act == "relu":
        # the mask is taken from the fp32 forward output; recompute the reference with that mask
        mask = host(y_, (out_dim, n)) > 0
        delta_ref = dy64 * mask
        dW, db, dx = delta_ref @ x64.T, delta_ref.sum(1), W64.T @ delta_ref
    close(host(dW_, (out_dim, in_dim)), dW, name="dW")
    close(host(db_, (out_dim,)), db, name="db")
    close(host(dx_, (in_dim, n)), dx, name="dx")
    # no bias, no dx
    fb.call("fb_dense_bwd", ACT[act], PREC[prec], P(tW), P(tx), P(y_), P(z_), P(tdy), P(delta), P(dW_), None, None,
            out_dim, in_dim, n)
    close(host(dW_, (out_dim, in_dim)), dW, name="dW (no db/dx)")


# --------------------------------------------------------------------------------- LayerNorm ---
@pytest.mark.parametrize("d,n", [(4096, 64), (1024, 33), (2, 3), (100, 17), (8192, 8), (12288, 4), (257, 5), (512, 1)])
@pytest.mark.parametrize("affine,act", [(True, "identity"), (False, "identity"), (True, "tanh"), (True, "relu")])
def test_layernorm_fwd_bwd(fb, d, n, affine, act):
    rng = np.random.default_rng(d + n)
    x = (rng.normal(size=(d, n)) * 1.7 + 0.3).astype(np.float32)
    g = (rng.normal(size=d) * 0.5 + 1).astype(np.float32) if affine else None
    b = (rng.normal(size=d) * 0.5).astype(np.float32) if affine else None
    dy = rng.normal(size=(d, n)).astype(np.float32)
    tx, tg, tb_, tdy = dev(x), dev(g) if affine else None, dev(b) if affine else None, dev(dy)
    y, mean, rstd = dempty(d, n), dempty(n), dempty(n)
    fb.call("fb_layernorm_fwd", P(tx), P(tg), P(tb_), P(y), P(mean), P(rstd), d, n, 1e-5, ACT[act])
    x64, g64, b64, dy64 = f64(x, g, b, dy)
    yref, mu, rs = O.layernorm_fwd(x64, g64, b64, 1e-5, act, return_stats=True)
    close(host(y, (d, n)), yref, name="y")
    close(host(mean, (n,)), mu.reshape(-1), name="mean", atol_scale=1e-5)
    close(host(rstd, (n,)), rs.reshape(-1), name="rstd")
    dx, dg, db = dempty(d, n), dempty(d), dempty(d)
    fb.call("fb_layernorm_bwd", P(tx), P(tg), P(tb_), P(mean), P(rstd), P(tdy), P(dx), P(dg) if affine else None,
            P(db) if affine else None, d, n, ACT[act])
    dxr, dgr, dbr = O.layernorm_bwd(x64, g64, b64, dy64, 1e-5, act)
    got_dx = host(dx, (d, n)).astype(np.float64)
    if act == "relu":   # elements whose pre-activation sits within rounding of 0 may take either branch
        unsure = np.abs(O.layernorm_fwd(x64, g64, b64, 1e-5, "identity")) < 1e-5
        got_dx[unsure] = dxr[unsure]
    # dx is a difference of terms of size |dy * gamma * rstd|; that is the scale rounding errors live on
    term = float(np.max(np.abs(dy64 * (g64.reshape(-1, 1) if affine else 1.0) * rs)))
    np.testing.assert_allclose(got_dx, dxr, rtol=2e-4, atol=2e-4 * max(float(np.max(np.abs(dxr))), 1e-2 * term), err_msg="dx")
    if affine:
        close(host(dg, (d,)), dgr, name="dgamma", rtol=2e-4, atol_scale=2e-4)
        close(host(db, (d,)), dbr, name="dbeta", rtol=2e-4, atol_scale=2e-4)


def test_layernorm_empty_batch_and_bad_args(fb):
    fb.call("fb_layernorm_fwd", None, None, None, None, None, None, 8, 0, 1e-5, 0)
    st, msg = fb.status("fb_layernorm_fwd", None, None, None, None, None, None, 0, 4, 1e-5, 0)
    assert st == -2
    st, msg = fb.status("fb_layernorm_fwd", None, None, None, None, None, None, 8, 4, 1e-5, 99)
    assert st == -1 and "activation" in msg


# --------------------------------------------------------------------------------- BatchNorm ---
def test_batchnorm_known_answers(fb):
    """test/layers/normalisation.jl:125-159: y, running mean / variance, inference value."""
    x = np.array([[1.0, 3.0, 5.0], [2.0, 4.0, 6.0]], np.float32)   # Julia [C=2, N=3]
    tx, g, b = dev(x), dev(np.ones(2, np.float32)), dev(np.zeros(2, np.float32))
    mu, var = dev(np.zeros(2, np.float32)), dev(np.ones(2, np.float32))
    y, sm, sr = dempty(2, 3), dempty(2), dempty(2)
    fb.call("fb_batchnorm_fwd_train", P(tx), P(g), P(b), P(mu), P(var), P(y), P(sm), P(sr), 1, 2, 3, 1e-5, 0.1, 0, 1)
    np.testing.assert_allclose(host(y, (2, 3)), [[-1.22474, 0, 1.22474], [-1.22474, 0, 1.22474]], atol=1e-5)
    np.testing.assert_allclose(host(mu, (2,)), [0.3, 0.4], rtol=1e-6)
    np.testing.assert_allclose(host(var, (2,)), [1.3, 1.3], rtol=1e-6)
    fb.call("fb_batchnorm_fwd_infer", P(tx), P(g), P(b), P(mu), P(var), P(y), 1, 2, 3, 1e-5, 0)
    assert abs(host(y, (2, 3))[0, 0] - (1 - 0.3) / np.sqrt(1.3)) < 1e-5
    # with sigmoid (normalisation.jl:188-191)
    fb.call("fb_batchnorm_fwd_infer", P(tx), P(g), P(b), P(mu), P(var), P(y), 1, 2, 3, 1e-5, ACT["sigmoid"])
    m_, v_ = host(mu, (2,)), host(var, (2,))
    ref = 1 / (1 + np.exp(-((x - m_[:, None]) / np.sqrt(v_[:, None] + 1e-5))))
    np.testing.assert_allclose(host(y, (2, 3)), ref, atol=1e-6)
    # a single value per channel is rejected in training (normalisation.jl:176-185)
    st, msg = fb.status("fb_batchnorm_fwd_train", P(tx), P(g), P(b), P(mu), P(var), P(y), P(sm), P(sr), 1, 1, 1, 1e-5, 0.1, 0, 1)
    assert st == -2 and "more than 1 value per channel" in msg


@pytest.mark.parametrize("shape", [(32, 32, 16, 8), (3, 2, 1), (2, 3, 2, 1), (2, 2, 3, 2, 1), (7, 5, 3), (16, 64), (5, 6, 4, 9)])
@pytest.mark.parametrize("act", ["identity", "relu"])
def test_batchnorm_fwd_bwd(fb, shape, act):
    rng = np.random.default_rng(sum(shape))
    x = (rng.normal(size=shape) * 2 + 0.5).astype(np.float32)
    c, n = shape[-2], shape[-1]
    s = int(np.prod(shape[:-2])) if len(shape) > 2 else 1
    g = (rng.normal(size=c) * 0.5 + 1.2).astype(np.float32)
    b = (rng.normal(size=c) * 0.5).astype(np.float32)
    dy = rng.normal(size=shape).astype(np.float32)
    rm, rv = rng.normal(size=c).astype(np.float32), (rng.random(c) + 0.5).astype(np.float32)
    tx, tg, tb_, tdy, trm, trv = dev(x), dev(g), dev(b), dev(dy), dev(rm), dev(rv)
    y, sm, sr = dempty(*shape), dempty(c), dempty(c)
    fb.call("fb_batchnorm_fwd_train", P(tx), P(tg), P(tb_), P(trm), P(trv), P(y), P(sm), P(sr), s, c, n, 1e-5, 0.1, ACT[act], 1)
    x64, g64, b64, dy64, rm64, rv64 = f64(x, g, b, dy, rm, rv)
    yref, nm, nv = O.batchnorm_fwd_train(x64, g64, b64, rm64, rv64, 0.1, 1e-5, act)
    close(host(y, shape), yref, name="y")
    close(host(trm, (c,)), nm, name="running mean")
    close(host(trv, (c,)), nv, name="running var")
    dx, dg, db = dempty(*shape), dempty(c), dempty(c)
    fb.call("fb_batchnorm_bwd", P(tx), P(tg), P(tb_), P(sm), P(sr), P(tdy), P(dx), P(dg), P(db), s, c, n, ACT[act])
    dxr, dgr, dbr = O.batchnorm_bwd(x64, g64, b64, dy64, 1e-5, act)
    got_dx = host(dx, shape).astype(np.float64)
    if act == "relu":   # elements whose pre-activation sits within rounding of 0 may take either branch
        unsure = np.abs(O.batchnorm_fwd_train(x64, g64, b64, None, None, sigma="identity", track_stats=False)[0]) < 1e-5
        got_dx[unsure] = dxr[unsure]
    close(got_dx, dxr, name="dx", rtol=2e-4, atol_scale=2e-4)
    close(host(dg, (c,)), dgr, name="dgamma", rtol=2e-4, atol_scale=2e-4)
    close(host(db, (c,)), dbr, name="dbeta", rtol=2e-4, atol_scale=2e-4)
    # track_stats = 0 leaves the running statistics alone
    before = host(trm, (c,)).copy()
    fb.call("fb_batchnorm_fwd_train", P(tx), P(tg), P(tb_), P(trm), P(trv), P(y), P(sm), P(sr), s, c, n, 1e-5, 0.1, ACT[act], 0)
    assert (host(trm, (c,)) == before).all()
    # inference with the running statistics
    fb.call("fb_batchnorm_fwd_infer", P(tx), P(tg), P(tb_), P(trm), P(trv), P(y), s, c, n, 1e-5, ACT[act])
    close(host(y, shape), O.batchnorm_fwd_infer(x64, g64, b64, nm, nv, 1e-5, act), name="inference")


def test_batchnorm_nd_equals_permuted_2d(fb):
    """test/layers/normalisation.jl:201-220 (the reference asserts ==; the device reduction order differs
    between the two layouts, so the check here is 1e-6)."""
    x = np.arange(1, 13, dtype=np.float32).reshape((2, 3, 2, 1), order="F")
    g, b = dev(np.ones(2, np.float32)), dev(np.zeros(2, np.float32))
    y4, sm, sr = dempty(12), dempty(2), dempty(2)
    tx4 = dev(x)
    fb.call("fb_batchnorm_fwd_train", P(tx4), P(g), P(b), None, None, P(y4), P(sm), P(sr), 6, 2, 1, 1e-5, 0.1, 0, 0)
    x2 = np.transpose(x, (2, 0, 1, 3)).reshape((2, -1), order="F")
    y2, tx2 = dempty(12), dev(x2)
    fb.call("fb_batchnorm_fwd_train", P(tx2), P(g), P(b), None, None, P(y2), P(sm), P(sr), 1, 2, 6, 1e-5, 0.1, 0, 0)
    y2n = np.transpose(host(y2, (2, 6)).reshape((2, 2, 3, 1), order="F"), (1, 2, 0, 3))
    np.testing.assert_allclose(host(y4, (2, 3, 2, 1)), y2n, atol=1e-6)


def test_batchnorm_large_mean_is_stable(fb):
    rng = np.random.default_rng(9)
    x = (rng.normal(size=(64, 8, 32)) * 0.01 + 1000.0).astype(np.float32)
    y, sm, sr, tx = dempty(*x.shape), dempty(8), dempty(8), dev(x)
    fb.call("fb_batchnorm_fwd_train", P(tx), None, None, None, None, P(y), P(sm), P(sr), 64, 8, 32, 1e-5, 0.1, 0, 0)
    ref, _, _ = O.batchnorm_fwd_train(x.astype(np.float64), None, None, None, None, track_stats=False)
    # the saved mean is a Float32 near 1000 (ulp 6e-5) against a standard deviation of 0.01: xhat cannot be
    # better than ~1e-2 absolute; a naive sum-of-squares variance would be off by orders of magnitude
    np.testing.assert_allclose(host(y, x.shape), ref, rtol=0, atol=3e-2)
    assert 0.9 < float(np.std(host(y, x.shape))) < 1.1


# ------------------------------------------------------------------------------ loss / helpers ---
def test_logitcrossentropy_known_answers(fb):
    """test/losses.jl:43-54, 79-83 and the doctest at src/losses/functions.jl:255-264."""
    v = np.log(0.1 / 0.9)
    logyhat = np.array([[v, 0.0], [0.0, v], [0.0, v], [v, 0.0]], np.float32).T
    labels = np.array([2, 2, 1, 1], np.int32)    # onehotbatch([1,1,0,0], 0:1) -> rows (0,1): class index 1-based
    loss, t1, t2 = dempty(1), dev(logyhat), dev(labels)
    fb.call("fb_logitcrossentropy_labels", P(t1), P(t2), P(loss), None, 2, 4, 1.0)
    assert abs(float(loss.item()) - 1.203972804325936) < 1e-6
    y_model = np.concatenate([np.arange(-9, 1), np.arange(0, 10), [7.5]]).astype(np.float32).reshape((3, 7), order="F")
    lab = np.array([1, 2, 3, 1, 2, 1, 1], np.int32)
    t3, t4, t5 = dev(y_model), dev(lab), dev(O.onehotbatch(lab, 3))
    fb.call("fb_logitcrossentropy_labels", P(t3), P(t4), P(loss), None, 3, 7, 1.0)
    assert abs(float(loss.item()) - 1.5791205) < 2e-6
    fb.call("fb_logitcrossentropy_dense", P(t3), P(t5), P(loss), None, 3, 7, 1.0)
    assert abs(float(loss.item()) - 1.5791205) < 2e-6


@pytest.mark.parametrize("c,n", [(10, 1024), (1000, 512), (3, 7), (33, 1)])
def test_logitcrossentropy_fwd_bwd(fb, c, n):
    rng = np.random.default_rng(c + n)
    yhat = (rng.normal(size=(c, n)) * 3).astype(np.float32)
    lab = rng.integers(1, c + 1, size=n).astype(np.int32)
    y = O.onehotbatch(lab, c, np.float64)
    loss, d, tyh, tlab = dempty(1), dempty(c, n), dev(yhat), dev(lab)
    fb.call("fb_logitcrossentropy_labels", P(tyh), P(tlab), P(loss), P(d), c, n, 1.0)
    close(loss.item(), O.logitcrossentropy(yhat.astype(np.float64), y))
    close(host(d, (c, n)), O.logitcrossentropy_bwd(yhat.astype(np.float64), y))
    ys = y * 0.8 + 0.2 / c
    tys = dev(ys, np.float32)
    fb.call("fb_logitcrossentropy_dense", P(tyh), P(tys), P(loss), P(d), c, n, 0.5)
    close(loss.item(), O.logitcrossentropy(yhat.astype(np.float64), ys))
    close(host(d, (c, n)), O.logitcrossentropy_bwd(yhat.astype(np.float64), ys, 0.5))


@pytest.mark.parametrize("count", [1, 3, 1000, 1 << 20, (1 << 20) + 5])
def test_sumsq_scale_axpy(fb, count):
    rng = np.random.default_rng(count)
    x = rng.normal(size=count).astype(np.float32)
    y = rng.normal(size=count).astype(np.float32)
    out, tx, ty, tz = dempty(1), dev(x), dev(y), dempty(count)
    fb.call("fb_sumsq", P(tx), count, P(out))
    close(out.item(), np.sum(x.astype(np.float64) ** 2), rtol=2e-6)
    fb.call("fb_scale", P(tx), 2.0, P(tz), count)
    assert (host(tz, (count,)) == 2 * x).all()
    fb.call("fb_axpy", -0.5, P(tx), P(ty), count)
    np.testing.assert_allclose(host(ty, (count,)), y - 0.5 * x, rtol=1e-6, atol=1e-6)
    # unaligned views
    if count > 8:
        fb.call("fb_sumsq", C.c_void_p(tx.data_ptr() + 4), count - 1, P(out))
        close(out.item(), np.sum(x[1:].astype(np.float64) ** 2), rtol=2e-6)


def test_bf16_cast_is_bit_exact(fb):
    """src/functor.jl:161-166; test/utils.jl:311."""
    rng = np.random.default_rng(3)
    x = np.concatenate([np.array([1, 1.5, -2.25, 96, np.nan, np.inf, -np.inf, 0.0, -0.0], np.float32),
                        np.array([0x3F808000, 0x3F818000, 0x3F808001, 0x7F7FFFFF], np.uint32).view(np.float32),
                        (rng.normal(size=100000) * 10 ** rng.uniform(-20, 20, 100000)).astype(np.float32)])
    tx = dev(x)
    out = torch.empty(x.size, dtype=torch.int16, device="cuda")
    fb.call("fb_cast_f32_bf16", P(tx), P(out), x.size)
    got = out.cpu().numpy().view(np.uint16)
    assert (got == O.to_bf16_bits(x)).all()
    back = dempty(x.size)
    fb.call("fb_cast_bf16_f32", P(out), P(back), x.size)
    ref = O.bf16_bits_to_f32(O.to_bf16_bits(x))
    assert (host(back, (x.size,)).view(np.uint32) == ref.view(np.uint32)).all()
    assert (host(back[:4], (4,)) == np.array([1, 1.5, -2.25, 96], np.float32)).all()


def test_adam_matches_oracle_over_ten_steps(fb):
    rng = np.random.default_rng(5)
    sizes = [(7,), (512, 784), (10,), (33, 5), (1,)] + [(16,)] * 40   # more than one 32-leaf launch
    ws = [rng.normal(size=s).astype(np.float32) for s in sizes]
    tw = [dev(w) for w in ws]
    tm = [torch.zeros_like(t) for t in tw]
    tv = [torch.zeros_like(t) for t in tw]
    states = [O.adam_init(w) for w in ws]
    k = len(ws)
    arr = C.c_void_p * k
    bt = (np.float32(0.9), np.float32(0.999))
    for step in range(10):
        gs = [(rng.normal(size=s) * (10.0 ** rng.integers(-3, 2))).astype(np.float32) for s in sizes]
        tg = [dev(g) for g in gs]
        fb.call("fb_adam_step", k, arr(*[t.data_ptr() for t in tw]), arr(*[t.data_ptr() for t in tg]),
                arr(*[t.data_ptr() for t in tm]), arr(*[t.data_ptr() for t in tv]),
                (C.c_int64 * k)(*[t.numel() for t in tw]), 1e-3, 0.9, 0.999, 1e-8, float(bt[0]), float(bt[1]), 1.0)
        bt = (bt[0] * np.float32(0.9), bt[1] * np.float32(0.999))
        ws = [O.adam_apply(st, w, g) for st, w, g in zip(states, ws, gs)]
    for t, w, s in zip(tw, ws, sizes):
        np.testing.assert_allclose(host(t, s), w, rtol=1e-5, atol=1e-7)
    for t, st, s in zip(tm, states, sizes):
        np.testing.assert_allclose(host(t, s), st[0], rtol=1e-5, atol=1e-6 * float(np.max(np.abs(st[0]))))


# --------------------------------------------------------------------------------- recurrent ---
# (24, 64, 6, 32) and (40, 144, 5, 16): H and B multiples of 16, the register-tiled persistent forward kernel
@pytest.mark.parametrize("I,H,T,B", [(3, 4, 5, 2), (16, 32, 7, 3), (64, 128, 12, 70), (20, 130, 4, 5), (24, 64, 6, 32), (40, 144, 5, 16)])
@pytest.mark.parametrize("bias,state", [(True, False), (False, True)])
def test_lstm_fwd_bwd(fb, I, H, T, B, bias, state):
    rng = np.random.default_rng(I + H + T + B)
    Wi, Wh = O.glorot_uniform(rng, 4 * H, I), O.glorot_uniform(rng, 4 * H, H)
    b = (rng.normal(size=4 * H) * 0.1).astype(np.float32) if bias else None
    x = rng.normal(size=(I, T, B)).astype(np.float32)
    h0 = rng.normal(size=(H, B)).astype(np.float32) if state else None
    c0 = rng.normal(size=(H, B)).astype(np.float32) if state else None
    nbytes = fb.raw.fb_lstm_cache_bytes(I, H, T, B)
    cache = torch.empty(nbytes // 4, dtype=torch.float32, device="cuda")
    tWi, tWh, tb_, tx = dev(Wi), dev(Wh), dev(b) if bias else None, dev(x)
    th0, tc0 = (dev(h0), dev(c0)) if state else (None, None)
    out, hT, cT = dempty(H, T, B), dempty(H, B), dempty(H, B)
    fb.call("fb_lstm_fwd", P(tWi), P(tWh), P(tb_), P(tx), P(th0), P(tc0), P(out), P(hT), P(cT), P(cache), I, H, T, B)
    Wi64, Wh64, b64, x64, h064, c064 = f64(Wi, Wh, b, x, h0, c0)
    oref, (href, cref) = O.lstm_scan_fwd(Wi64, Wh64, b64, x64, h064, c064)
    close(host(out, (H, T, B)), oref, name="out")
    close(host(hT, (H, B)), href, name="hT")
    close(host(cT, (H, B)), cref, name="cT")
    # forward without a cache gives the same output
    out2 = dempty(H, T, B)
    fb.call("fb_lstm_fwd", P(tWi), P(tWh), P(tb_), P(tx), P(th0), P(tc0), P(out2), None, None, None, I, H, T, B)
    assert torch.equal(out, out2)
    if state:
        return   # the oracle's BPTT covers the zero-state case
    dout = O.sum_abs2_bwd(oref)
    dWi, dWh, db, dx = dempty(4 * H, I), dempty(4 * H, H), dempty(4 * H), dempty(I, T, B)
    tdout = dev(dout, np.float32)
    fb.call("fb_lstm_bwd", P(tWi), P(tWh), P(tx), None, None, P(out), P(cache), P(tdout), None, None,
            P(dWi), P(dWh), P(db) if bias else None, P(dx), I, H, T, B)
    rWi, rWh, rb, rx = O.lstm_scan_bwd(Wi64, Wh64, b64, x64, dout)
    close(host(dWi, (4 * H, I)), rWi, name="dWi", rtol=2e-4, atol_scale=2e-4)
    close(host(dWh, (4 * H, H)), rWh, name="dWh", rtol=2e-4, atol_scale=2e-4)
    close(host(dx, (I, T, B)), rx, name="dx", rtol=2e-4, atol_scale=2e-4)
    if bias:
        close(host(db, (4 * H,)), rb, name="db", rtol=2e-4, atol_scale=2e-4)


@pytest.mark.parametrize("I,H,T,B", [(3, 4, 5, 2), (16, 32, 7, 3), (64, 128, 12, 70), (20, 130, 4, 5), (24, 96, 6, 16), (40, 144, 5, 32)])
@pytest.mark.parametrize("bias", [True, False])
def test_gru_fwd_bwd(fb, I, H, T, B, bias):
    rng = np.random.default_rng(I + H + T + B + 1)
    Wi, Wh = O.glorot_uniform(rng, 3 * H, I), O.glorot_uniform(rng, 3 * H, H)
    b = (rng.normal(size=3 * H) * 0.1).astype(np.float32) if bias else None
    x = rng.normal(size=(I, T, B)).astype(np.float32)
    nbytes = fb.raw.fb_gru_cache_bytes(I, H, T, B)
    cache = torch.empty(nbytes // 4, dtype=torch.float32, device="cuda")
    tWi, tWh, tb_, tx = dev(Wi), dev(Wh), dev(b) if bias else None, dev(x)
    out, hT = dempty(H, T, B), dempty(H, B)
    fb.call("fb_gru_fwd", P(tWi), P(tWh), P(tb_), P(tx), None, P(out), P(hT), P(cache), I, H, T, B)
    Wi64, Wh64, b64, x64 = f64(Wi, Wh, b, x)
    oref, href = O.gru_scan_fwd(Wi64, Wh64, b64, x64)
    close(host(out, (H, T, B)), oref, name="out")
    close(host(hT, (H, B)), href, name="hT")
    dout = O.sum_abs2_bwd(oref)
    dWi, dWh, db, dx = dempty(3 * H, I), dempty(3 * H, H), dempty(3 * H), dempty(I, T, B)
    tdout = dev(dout, np.float32)
    fb.call("fb_gru_bwd", P(tWi), P(tWh), P(tx), None, P(out), P(cache), P(tdout), None, P(dWi), P(dWh),
            P(db) if bias else None, P(dx), I, H, T, B)
    rWi, rWh, rb, rx = O.gru_scan_bwd(Wi64, Wh64, b64, x64, dout)
    close(host(dWi, (3 * H, I)), rWi, name="dWi", rtol=2e-4, atol_scale=2e-4)
    close(host(dWh, (3 * H, H)), rWh, name="dWh", rtol=2e-4, atol_scale=2e-4)
    close(host(dx, (I, T, B)), rx, name="dx", rtol=2e-4, atol_scale=2e-4)
    if bias:
        close(host(db, (3 * H,)), rb, name="db", rtol=2e-4, atol_scale=2e-4)


# --------------------------------------------------------------------------------- attention ---
@pytest.mark.parametrize("E,Ev,heads,Lq,Lk,B", [(4, 4, 2, 3, 3, 5), (64, 64, 1, 70, 70, 2), (128, 64, 2, 65, 130, 3),
                                               (256, 256, 2, 33, 33, 1), (96, 96, 4, 128, 128, 2),
                                               # head size 64: the tensor-core kernels (several key / query blocks, ragged
                                               # tails, Lq != Lk); with an explicit mask the same shapes run on the FMA kernels
                                               (128, 128, 2, 200, 200, 2), (64, 64, 1, 130, 300, 1), (256, 256, 4, 520, 520, 1)])
@pytest.mark.parametrize("mode", ["none", "causal", "mask"])
def test_attention_fwd_bwd_scores(fb, E, Ev, heads, Lq, Lk, B, mode):
    if mode == "causal" and Lq != Lk:
        pytest.skip("causal masks are square in the reference")
    rng = np.random.default_rng(E + Lq + Lk + B)
    q = rng.normal(size=(E, Lq, B)).astype(np.float32)
    k = rng.normal(size=(E, Lk, B)).astype(np.float32)
    v = rng.normal(size=(Ev, Lk, B)).astype(np.float32)
    do = rng.normal(size=(Ev, Lq, B)).astype(np.float32)
    mask = None
    if mode == "causal":
        mask = O.make_causal_mask(Lq)
    elif mode == "mask":
        mask = rng.random((Lk, Lq)) > 0.3
        mask[0, :] = True   # no fully masked query
    tq, tk, tv, tdo = dev(q), dev(k), dev(v), dev(do)
    tm = dev(mask.astype(np.uint8)) if mode == "mask" else None
    causal = 1 if mode == "causal" else 0
    o, lse = dempty(Ev, Lq, B), dempty(Lq, heads, B)
    fb.call("fb_attn_fwd", P(tq), P(tk), P(tv), P(tm), P(o), P(lse), E, Ev, Lq, Lk, B, heads, causal)
    q64, k64, v64, do64 = f64(q, k, v, do)
    oref, aref = O.dot_product_attention(q64, k64, v64, None, heads, mask)
    close(host(o, (Ev, Lq, B)), oref, name="o")
    alpha = dempty(Lk, Lq, heads, B)
    fb.call("fb_attn_scores", P(tq), P(tk), P(tm), P(lse), P(alpha), E, Lq, Lk, B, heads, causal)
    close(host(alpha, (Lk, Lq, heads, B)), aref, name="alpha", atol_scale=1e-5)
    if mode == "causal":
        a = host(alpha, (Lk, Lq, heads, B))
        assert (a[1, 0, :, :] == 0).all()                 # test/layers/attention.jl:38-43
        assert np.allclose(a[:, :, 0, 0], np.triu(a[:, :, 0, 0]))
    dq, dk, dv = dempty(E, Lq, B), dempty(E, Lk, B), dempty(Ev, Lk, B)
    fb.call("fb_attn_bwd", P(tq), P(tk), P(tv), P(tm), P(o), P(lse), P(tdo), P(dq), P(dk), P(dv), E, Ev, Lq, Lk, B, heads, causal)
    rq, rk, rv = O.dot_product_attention_bwd(q64, k64, v64, do64, None, heads, mask)
    close(host(dq, (E, Lq, B)), rq, name="dq", rtol=2e-4, atol_scale=2e-4)
    close(host(dk, (E, Lk, B)), rk, name="dk", rtol=2e-4, atol_scale=2e-4)
    close(host(dv, (Ev, Lk, B)), rv, name="dv", rtol=2e-4, atol_scale=2e-4)


def test_attention_rejects_bad_head_split(fb):
    a = dempty(64)
    st, msg = fb.status("fb_attn_fwd", P(a), P(a), P(a), None, P(a), P(a), 6, 6, 2, 2, 1, 4, 0)
    assert st == -2 and "divisible by nheads" in msg


# --------------------------------------------------------------- committed golden fixture ---
def test_against_committed_golden_vectors(fb):
    """The CUDA library against tests/golden/oracle_vectors.npz (made by tests/golden/make_golden.py)."""
    import os
    G = np.load(os.path.join(os.path.dirname(__file__), "golden", "oracle_vectors.npz"))
    keep = []

    def d(name, dtype=np.float32):
        t = dev(G[name], dtype)
        keep.append(t)
        return t

    # Dense
    for act in ("relu", "gelu_tanh"):
        y, z, delta = dempty(6, 7), dempty(6, 7), dempty(6, 7)
        dW, db, dx = dempty(6, 5), dempty(6), dempty(5, 7)
        fb.call("fb_dense_fwd", ACT[act], 0, P(d("dense_W")), P(d("dense_b")), P(d("dense_x")), P(y), P(z), 6, 5, 7)
        close(host(y, (6, 7)), G[f"dense_y_{act}"])
        fb.call("fb_dense_bwd", ACT[act], 0, P(d("dense_W")), P(d("dense_x")), P(y), P(z), P(d("dense_dy")), P(delta), P(dW),
                P(db), P(dx), 6, 5, 7)
        close(host(dW, (6, 5)), G[f"dense_dW_{act}"])
        close(host(db, (6,)), G[f"dense_db_{act}"])
        close(host(dx, (5, 7)), G[f"dense_dx_{act}"])
    # LayerNorm
    y, mean, rstd, dx, dg, db = dempty(8, 5), dempty(5), dempty(5), dempty(8, 5), dempty(8), dempty(8)
    fb.call("fb_layernorm_fwd", P(d("ln_x")), P(d("ln_g")), P(d("ln_b")), P(y), P(mean), P(rstd), 8, 5, 1e-5, 0)
    close(host(y, (8, 5)), G["ln_y"])
    fb.call("fb_layernorm_bwd", P(d("ln_x")), P(d("ln_g")), P(d("ln_b")), P(mean), P(rstd), P(d("ln_dy")), P(dx), P(dg), P(db), 8, 5, 0)
    close(host(dx, (8, 5)), G["ln_dx"], rtol=2e-4, atol_scale=2e-4)
    close(host(dg, (8,)), G["ln_dg"], rtol=2e-4, atol_scale=2e-4)
    close(host(db, (8,)), G["ln_db"], rtol=2e-4, atol_scale=2e-4)
    # BatchNorm
    shp = (3, 2, 4, 5)
    rm, rv = dev(np.zeros(4, np.float32)), dev(np.ones(4, np.float32))
    y, sm, sr, dx, dg, db = dempty(*shp), dempty(4), dempty(4), dempty(*shp), dempty(4), dempty(4)
    fb.call("fb_batchnorm_fwd_train", P(d("bn_x")), P(d("bn_g")), P(d("bn_b")), P(rm), P(rv), P(y), P(sm), P(sr), 6, 4, 5, 1e-5, 0.1,
            ACT["relu"], 1)
    close(host(y, shp), G["bn_y"])
    close(host(rm, (4,)), G["bn_mean"])
    close(host(rv, (4,)), G["bn_var"])
    fb.call("fb_batchnorm_bwd", P(d("bn_x")), P(d("bn_g")), P(d("bn_b")), P(sm), P(sr), P(d("bn_dy")), P(dx), P(dg), P(db), 6, 4, 5,
            ACT["relu"])
    close(host(dx, shp), G["bn_dx"], rtol=2e-4, atol_scale=2e-4)
    close(host(dg, (4,)), G["bn_dg"], rtol=2e-4, atol_scale=2e-4)
    close(host(db, (4,)), G["bn_db"], rtol=2e-4, atol_scale=2e-4)
    # LSTM / GRU
    for name, ng in (("lstm", 4), ("gru", 3)):
        nbytes = getattr(fb.raw, f"fb_{name}_cache_bytes")(3, 4, 5, 2)
        cache = torch.empty(nbytes // 4, dtype=torch.float32, device="cuda")
        out, hT, cT = dempty(4, 5, 2), dempty(4, 2), dempty(4, 2)
        dWi, dWh, dbb, dxs = dempty(ng * 4, 3), dempty(ng * 4, 4), dempty(ng * 4), dempty(3, 5, 2)
        tdout = dev(2 * G[f"{name}_out"], np.float32)
        if name == "lstm":
            fb.call("fb_lstm_fwd", P(d("lstm_Wi")), P(d("lstm_Wh")), P(d("lstm_b")), P(d("lstm_x")), None, None, P(out), P(hT), P(cT),
                    P(cache), 3, 4, 5, 2)
            fb.call("fb_lstm_bwd", P(d("lstm_Wi")), P(d("lstm_Wh")), P(d("lstm_x")), None, None, P(out), P(cache), P(tdout), None, None,
                    P(dWi), P(dWh), P(dbb), P(dxs), 3, 4, 5, 2)
        else:
            fb.call("fb_gru_fwd", P(d("gru_Wi")), P(d("gru_Wh")), P(d("gru_b")), P(d("gru_x")), None, P(out), P(hT), P(cache), 3, 4, 5, 2)
            fb.call("fb_gru_bwd", P(d("gru_Wi")), P(d("gru_Wh")), P(d("gru_x")), None, P(out), P(cache), P(tdout), None, P(dWi), P(dWh),
                    P(dbb), P(dxs), 3, 4, 5, 2)
        close(host(out, (4, 5, 2)), G[f"{name}_out"])
        close(host(dWi, (ng * 4, 3)), G[f"{name}_dWi"], rtol=2e-4, atol_scale=2e-4)
        close(host(dWh, (ng * 4, 4)), G[f"{name}_dWh"], rtol=2e-4, atol_scale=2e-4)
        close(host(dbb, (ng * 4,)), G[f"{name}_db"], rtol=2e-4, atol_scale=2e-4)
        close(host(dxs, (3, 5, 2)), G[f"{name}_dx"], rtol=2e-4, atol_scale=2e-4)
    # attention
    o, lse, alpha = dempty(8, 6, 2), dempty(6, 2, 2), dempty(6, 6, 2, 2)
    dq, dk, dv = dempty(8, 6, 2), dempty(8, 6, 2), dempty(8, 6, 2)
    fb.call("fb_attn_fwd", P(d("attn_q")), P(d("attn_k")), P(d("attn_v")), None, P(o), P(lse), 8, 8, 6, 6, 2, 2, 1)
    close(host(o, (8, 6, 2)), G["attn_o"])
    fb.call("fb_attn_scores", P(d("attn_q")), P(d("attn_k")), None, P(lse), P(alpha), 8, 6, 6, 2, 2, 1)
    close(host(alpha, (6, 6, 2, 2)), G["attn_alpha"], atol_scale=1e-5)
    fb.call("fb_attn_bwd", P(d("attn_q")), P(d("attn_k")), P(d("attn_v")), None, P(o), P(lse), P(d("attn_do")), P(dq), P(dk), P(dv),
            8, 8, 6, 6, 2, 2, 1)
    close(host(dq, (8, 6, 2)), G["attn_dq"], rtol=2e-4, atol_scale=2e-4)
    close(host(dk, (8, 6, 2)), G["attn_dk"], rtol=2e-4, atol_scale=2e-4)
    close(host(dv, (8, 6, 2)), G["attn_dv"], rtol=2e-4, atol_scale=2e-4)
    # loss
    loss, dyh = dempty(1), dempty(5, 9)
    fb.call("fb_logitcrossentropy_labels", P(d("xent_yhat")), P(d("xent_labels", np.int32)), P(loss), P(dyh), 5, 9, 1.0)
    close(loss.item(), G["xent_loss"])
    close(host(dyh, (5, 9)), G["xent_dyhat"])
    # Adam
    w, m, v = d("adam_w0").clone(), torch.zeros(11, device="cuda"), torch.zeros(11, device="cuda")
    bt = (np.float32(0.9), np.float32(0.999))
    one = C.c_void_p * 1
    for step in range(3):
        g = dev(G["adam_g"][step])
        fb.call("fb_adam_step", 1, one(w.data_ptr()), one(g.data_ptr()), one(m.data_ptr()), one(v.data_ptr()), (C.c_int64 * 1)(11),
                1e-3, 0.9, 0.999, 1e-8, float(bt[0]), float(bt[1]), 1.0)
        bt = (bt[0] * np.float32(0.9), bt[1] * np.float32(0.999))
    np.testing.assert_allclose(host(w, (11,)), G["adam_w3"], rtol=1e-5, atol=1e-7)
    np.testing.assert_allclose(host(v, (11,)), G["adam_v3"], rtol=1e-5, atol=1e-10)


# ------------------------------------------------------------- failure path of bounded waits ---
def test_a_bounded_wait_that_runs_out_is_reported_and_the_next_launch_works():
    """A wait that nothing satisfies (fb_selftest_bounded_wait: a barrier nobody signals, a few dozen polls) must end by
    itself, leave its code in the device error word, and not poison the context: while the word is set the tensor-core
    GEMM returns without computing; once the word has been read (which clears it) the same launch gives the right
    result."""
    from fluxb200 import lib
    h = C.c_void_p()
    lib.call("fb_ctx_create", 0, C.byref(h))
    try:
        def err():
            out = C.c_int32(0)
            lib.call("fb_device_error", h, stream(), C.byref(out))
            return out.value

        assert err() == 0
        lib.call("fb_selftest_bounded_wait", h, stream(), 64)
        assert err() == 9001          # reported ...
        assert err() == 0             # ... and cleared by the read
        rng = np.random.default_rng(0)
        m = n = k = 256
        A, B = rng.normal(size=(m, k)).astype(np.float32), rng.normal(size=(k, n)).astype(np.float32)
        dA, dB = dev(A), dev(B)
        dC = torch.full((m * n,), 7.0, device="cuda")
        lib.call("fb_selftest_bounded_wait", h, stream(), 64)
        lib.call("fb_gemm_f32", h, stream(), 0, 0, m, n, k, P(dA), m, P(dB), k, P(dC), m, 0, PREC["3xtf32"])
        torch.cuda.synchronize()
        assert (dC == 7.0).all()      # the GEMM saw the word and did not start
        assert err() == 9001
        lib.call("fb_gemm_f32", h, stream(), 0, 0, m, n, k, P(dA), m, P(dB), k, P(dC), m, 0, PREC["3xtf32"])
        close(host(dC, (m, n)), A.astype(np.float64) @ B.astype(np.float64), name="gemm after the error was read")
        assert err() == 0
        st = lib.raw().fb_selftest_bounded_wait(h, stream(), 1 << 20)
        assert st == -1               # the self test refuses long waits
    finally:
        lib.call("fb_ctx_destroy", h)


@pytest.mark.parametrize("E,heads,Lq,Lk,B", [(8, 2, 5, 7, 3), (128, 2, 70, 130, 2), (96, 4, 64, 64, 1)])
@pytest.mark.parametrize("bias_kind,p,with_dalpha,causal", [("shared", 0.0, False, 0), ("full", 0.0, True, 0), (None, 0.3, False, 1),
                                                          ("heads", 0.25, True, 0)])
def test_attention_bias_dropout_alpha_cotangent(fb, E, heads, Lq, Lk, B, bias_kind, p, with_dalpha, causal):
    """The remaining arguments of NNlib.dot_product_attention (src/layers/attention.jl:120-128): additive bias
    (broadcast over heads / batch or full), dropout on the attention weights (mask regenerated by the oracle from the
    same counter-based stream), and a cotangent of the returned weights (test/layers/attention.jl:45-61)."""
    if causal and Lq != Lk:
        pytest.skip("causal masks are square in the reference")
    rng = np.random.default_rng(E + Lq + Lk + B + heads)
    q = rng.normal(size=(E, Lq, B)).astype(np.float32)
    k = rng.normal(size=(E, Lk, B)).astype(np.float32)
    v = rng.normal(size=(E, Lk, B)).astype(np.float32)
    do = rng.normal(size=(E, Lq, B)).astype(np.float32)
    bias, sh, sb = None, 0, 0
    if bias_kind == "shared":
        bias = rng.normal(size=(Lk, Lq)).astype(np.float32)
    elif bias_kind == "heads":
        bias, sh = rng.normal(size=(Lk, Lq, heads, 1)).astype(np.float32), Lk * Lq
    elif bias_kind == "full":
        bias, sh, sb = rng.normal(size=(Lk, Lq, heads, B)).astype(np.float32), Lk * Lq, Lk * Lq * heads
    seed, off = 1234567, 17
    drop = None
    if p > 0:
        drop = O.dropout_mask(Lk * Lq * heads * B, p, seed, off).reshape((Lk, Lq, heads, B), order="F") / (1 - p)
    dalpha = rng.normal(size=(Lk, Lq, heads, B)).astype(np.float32) if with_dalpha else None
    mask = O.make_causal_mask(Lq) if causal else None
    tq, tk, tv, tdo = dev(q), dev(k), dev(v), dev(do)
    tb = dev(bias) if bias is not None else None
    tda = dev(dalpha) if with_dalpha else None
    o, lse, alpha = dempty(E, Lq, B), dempty(Lq, heads, B), dempty(Lk, Lq, heads, B)
    fb.call("fb_attn_fwd_ex", P(tq), P(tk), P(tv), None, P(tb), sh, sb, p, seed, off, P(o), P(lse), E, E, Lq, Lk, B, heads, causal)
    fb.call("fb_attn_scores_ex", P(tq), P(tk), None, P(tb), sh, sb, p, seed, off, P(lse), P(alpha), E, Lq, Lk, B, heads, causal)
    q64, k64, v64, do64 = f64(q, k, v, do)
    b64 = None if bias is None else bias.astype(np.float64)
    oref, aref = O.dot_product_attention(q64, k64, v64, b64, heads, mask, drop=drop)
    close(host(o, (E, Lq, B)), oref, name="o")
    close(host(alpha, (Lk, Lq, heads, B)), aref, name="alpha", atol_scale=1e-5)
    dq, dk, dv = dempty(E, Lq, B), dempty(E, Lk, B), dempty(E, Lk, B)
    fb.call("fb_attn_bwd_ex", P(tq), P(tk), P(tv), None, P(tb), sh, sb, p, seed, off, P(o), P(lse), P(tdo), P(tda), P(dq), P(dk), P(dv),
            E, E, Lq, Lk, B, heads, causal)
    rq, rk, rv = O.dot_product_attention_bwd(q64, k64, v64, do64, b64, heads, mask, dalpha=None if dalpha is None else dalpha.astype(np.float64),
                                             drop=drop)
    close(host(dq, (E, Lq, B)), rq, name="dq", rtol=2e-4, atol_scale=2e-4)
    close(host(dk, (E, Lk, B)), rk, name="dk", rtol=2e-4, atol_scale=2e-4)
    close(host(dv, (E, Lk, B)), rv, name="dv", rtol=2e-4, atol_scale=2e-4)
    st, msg = fb.status("fb_attn_fwd_ex", P(tq), P(tk), P(tv), None, None, 0, 0, 1.0, 0, 0, P(o), P(lse), E, E, Lq, Lk, B, heads, 0)
    assert st == -1 and "dropout probability" in msg
