"""The oracle against the reference's own known-answer tests, and float64 finite-difference
checks of every hand-written backward (the method of the reference's test/test_module.jl:111-182)."""
import json
import os

import numpy as np
import pytest

import flux_oracle as O

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def fd_check(f, args, grads, idx, rtol=1e-5, atol=1e-7):
    def g(xv):
        a = list(args)
        a[idx] = xv
        return f(*a)
    num = O.finite_difference(g, args[idx])
    np.testing.assert_allclose(grads, num, rtol=rtol, atol=atol)


# ---- Dense: test/layers/basic.jl:78-89 -------------------------------------------------
def test_dense_ones_known_answers():
    ones = np.ones
    assert (O.dense_fwd(ones((1, 10)), np.zeros(1), ones((10, 1))) == 10 * ones((1, 1))).all()
    assert (O.dense_fwd(ones((1, 10)), np.zeros(1), ones((10, 2))) == 10 * ones((1, 2))).all()
    assert (O.dense_fwd(ones((2, 10)), np.zeros(2), ones((10, 1))) == 10 * ones((2, 1))).all()
    x = np.concatenate([ones((10, 1)), 2 * ones((10, 1))], axis=1)
    assert (O.dense_fwd(ones((2, 10)), np.zeros(2), x) == np.array([[10, 20], [10, 20]])).all()
    assert (O.dense_fwd(ones((2, 10)), None, x) == np.array([[10, 20], [10, 20]])).all()


def test_dense_nd_shapes_and_size_check():
    W = np.zeros((5, 10))
    for shp in [(10,), (10, 2), (10, 2, 3), (10, 2, 3, 4)]:
        assert O.dense_fwd(W, np.zeros(5), np.zeros(shp)).shape == (5,) + shp[1:]
    with pytest.raises(ValueError):
        O.dense_fwd(W, np.zeros(5), np.zeros((11, 2, 3)))


@pytest.mark.parametrize("sigma", O.ACTS)
def test_dense_bwd_fd(sigma):
    rng = np.random.default_rng(0)
    W, b, x = rng.normal(size=(4, 3)), rng.normal(size=4), rng.normal(size=(3, 5))
    x += 0.05 * np.sign(x)
    dy = rng.normal(size=(4, 5))
    loss = lambda W_, b_, x_: (O.dense_fwd(W_, b_, x_, sigma) * dy).sum()
    dW, db, dx = O.dense_bwd(W, b, x, dy, sigma)
    fd_check(loss, (W, b, x), dW, 0)
    fd_check(loss, (W, b, x), db, 1)
    fd_check(loss, (W, b, x), dx, 2)


# ---- BatchNorm: test/layers/normalisation.jl:125-159, 188-191, 201-220 -------------------
def test_batchnorm_known_answers():
    x = np.array([[1.0, 3.0, 5.0], [2.0, 4.0, 6.0]])
    g, b, mu, var = np.ones(2), np.zeros(2), np.zeros(2), np.ones(2)
    y, mu1, var1 = O.batchnorm_fwd_train(x, g, b, mu, var, 0.1, 1e-5)
    np.testing.assert_allclose(y, [[-1.22474, 0, 1.22474], [-1.22474, 0, 1.22474]], atol=1e-5)
    np.testing.assert_allclose(mu1, [0.3, 0.4])
    np.testing.assert_allclose(var1, 0.1 * x.var(axis=1) * (3 / 2) + 0.9 * np.ones(2))
    np.testing.assert_allclose(var1, [1.3, 1.3])
    yi = O.batchnorm_fwd_infer(x, g, b, mu1, var1, 1e-5)
    assert abs(yi[0, 0] - (1 - 0.3) / np.sqrt(1.3)) < 1e-5


def test_batchnorm_sigmoid_and_single_value_error():
    x = np.array([[1.0, 3.0, 5.0], [2.0, 4.0, 6.0]], dtype=np.float32)
    g, b = np.ones(2, np.float32), np.zeros(2, np.float32)
    mu, var = np.zeros(2, np.float32), np.ones(2, np.float32)
    y = O.batchnorm_fwd_infer(x, g, b, mu, var, 1e-5, "sigmoid")
    ref = 1 / (1 + np.exp(-((x - mu[:, None]) / np.sqrt(var[:, None] + 1e-5))))
    np.testing.assert_allclose(y, ref, atol=1e-7)
    with pytest.raises(ValueError):
        O.batchnorm_fwd_train(np.zeros((1, 1), np.float32), g[:1], b[:1], mu[:1], var[:1])
    O.batchnorm_fwd_train(np.arange(4, dtype=np.float32).reshape(4, 1, 1), g[:1], b[:1], mu[:1], var[:1])


def test_batchnorm_nd_equals_permuted_2d():
    g, b, mu, var = np.ones(2, np.float32), np.zeros(2, np.float32), np.zeros(2, np.float32), np.ones(2, np.float32)
    # Julia reshape is column-major: build with order="F"
    x = np.arange(1, 13, dtype=np.float32).reshape((2, 3, 2, 1), order="F")
    y4, _, _ = O.batchnorm_fwd_train(x, g, b, mu, var)
    x2 = np.transpose(x, (2, 0, 1, 3)).reshape((2, -1), order="F")
    y2, _, _ = O.batchnorm_fwd_train(x2, g, b, mu, var)
    y2 = np.transpose(y2.reshape((2, 2, 3, 1), order="F"), (1, 2, 0, 3))
    assert (y4 == y2).all()


@pytest.mark.parametrize("sigma", ["identity", "relu", "tanh"])
def test_batchnorm_bwd_fd(sigma):
    rng = np.random.default_rng(1)
    x = rng.normal(size=(3, 2, 4, 5)) * 2 + 0.5
    g, b = rng.normal(size=4) + 1.5, rng.normal(size=4)
    dy = rng.normal(size=x.shape)
    loss = lambda x_, g_, b_: (O.batchnorm_fwd_train(x_, g_, b_, None, None, sigma=sigma, track_stats=False)[0] * dy).sum()
    dx, dg, db = O.batchnorm_bwd(x, g, b, dy, sigma=sigma)
    fd_check(loss, (x, g, b), dx, 0, rtol=2e-5, atol=1e-6)
    fd_check(loss, (x, g, b), dg, 1, rtol=2e-5, atol=1e-6)
    fd_check(loss, (x, g, b), db, 2, rtol=2e-5, atol=1e-6)


# ---- LayerNorm: test/layers/normalisation.jl:370-391 --------------------------------------
def test_layernorm_matches_normalise_and_fd():
    rng = np.random.default_rng(2)
    x = rng.random((2, 3, 4, 5))
    y = O.layernorm_fwd(x, np.ones(2), np.zeros(2), 1e-5)
    mu = x.mean(axis=0, keepdims=True)
    ref = (x - mu) / np.sqrt(x.var(axis=0, keepdims=True) + 1e-5)
    np.testing.assert_allclose(y, ref)
    y2 = O.layernorm_fwd(x, np.ones((2, 3)), np.zeros((2, 3)), 1e-5, nd=2)
    mu2 = x.mean(axis=(0, 1), keepdims=True)
    np.testing.assert_allclose(y2, (x - mu2) / np.sqrt(x.var(axis=(0, 1), keepdims=True) + 1e-5))
    xt = rng.random(2)
    np.testing.assert_allclose(O.layernorm_fwd(xt, np.ones(2), np.zeros(2), 1e-5, "tanh"),
                               np.tanh((xt - xt.mean()) / np.sqrt(xt.var() + 1e-5)))
    x = rng.normal(size=(6, 4))
    g, b, dy = rng.normal(size=6), rng.normal(size=6), rng.normal(size=(6, 4))
    for sigma in ("identity", "tanh"):
        loss = lambda x_, g_, b_: (O.layernorm_fwd(x_, g_, b_, 1e-5, sigma) * dy).sum()
        dx, dg, db = O.layernorm_bwd(x, g, b, dy, 1e-5, sigma)
        fd_check(loss, (x, g, b), dx, 0, rtol=2e-5, atol=1e-6)
        fd_check(loss, (x, g, b), dg, 1, rtol=2e-5, atol=1e-6)
        fd_check(loss, (x, g, b), db, 2, rtol=2e-5, atol=1e-6)


# ---- losses: test/losses.jl:43-54, 79-83; src/losses/functions.jl:255-264 ----------------
def test_logitcrossentropy_known_answers():
    y = np.array([[0, 0, 1, 1], [1, 1, 0, 0]], dtype=np.float64)  # onehotbatch([1,1,0,0], 0:1)
    v = np.log(0.1 / 0.9)
    logyhat = np.array([[v, 0.0], [0.0, v], [0.0, v], [v, 0.0]]).T
    assert abs(O.logitcrossentropy(logyhat, y) - 1.203972804325936) < 1e-12
    y_model = np.concatenate([np.arange(-9, 1), np.arange(0, 10), [7.5]]).astype(np.float32).reshape((3, 7), order="F")
    labels = np.array([1, 2, 3, 1, 2, 1, 1])
    y_label = O.onehotbatch(labels, 3)
    assert abs(O.logitcrossentropy(y_model, y_label) - np.float32(1.5791205)) < 2e-6


def test_logitcrossentropy_bwd_fd():
    rng = np.random.default_rng(3)
    yhat = rng.normal(size=(5, 7))
    y = O.onehotbatch(rng.integers(1, 6, size=7), 5, np.float64)
    fd_check(lambda a: O.logitcrossentropy(a, y), (yhat,), O.logitcrossentropy_bwd(yhat, y), 0)
    ys = y * 0.8 + 0.04  # label-smoothed: general y
    fd_check(lambda a: O.logitcrossentropy(a, ys), (yhat,), O.logitcrossentropy_bwd(yhat, ys), 0)


# ---- recurrent: test/layers/recurrent.jl (FD self-consistency; zero initial state) ---------
def test_lstm_bwd_fd_and_zero_state():
    rng = np.random.default_rng(4)
    I, H, T, B = 3, 4, 5, 2
    Wi, Wh, b = rng.normal(size=(4 * H, I)) * .5, rng.normal(size=(4 * H, H)) * .5, rng.normal(size=4 * H) * .1
    x = rng.normal(size=(I, T, B))
    out, (h, c) = O.lstm_scan_fwd(Wi, Wh, b, x)
    out0, _ = O.lstm_scan_fwd(Wi, Wh, b, x, np.zeros(H), np.zeros(H))
    np.testing.assert_array_equal(out, out0)
    assert out.shape == (H, T, B) and h.shape == (H, B) and c.shape == (H, B)
    np.testing.assert_array_equal(out[:, -1, :], h)
    loss = lambda Wi_, Wh_, b_, x_: O.sum_abs2(O.lstm_scan_fwd(Wi_, Wh_, b_, x_)[0])
    dWi, dWh, db, dx = O.lstm_scan_bwd(Wi, Wh, b, x, O.sum_abs2_bwd(out))
    for i, g in enumerate((dWi, dWh, db, dx)):
        fd_check(loss, (Wi, Wh, b, x), g, i, rtol=1e-5, atol=1e-6)


def test_gru_bwd_fd():
    rng = np.random.default_rng(5)
    I, H, T, B = 3, 4, 5, 2
    Wi, Wh, b = rng.normal(size=(3 * H, I)) * .5, rng.normal(size=(3 * H, H)) * .5, rng.normal(size=3 * H) * .1
    x = rng.normal(size=(I, T, B))
    out, h = O.gru_scan_fwd(Wi, Wh, b, x)
    np.testing.assert_array_equal(out[:, -1, :], h)
    loss = lambda Wi_, Wh_, b_, x_: O.sum_abs2(O.gru_scan_fwd(Wi_, Wh_, b_, x_)[0])
    dWi, dWh, db, dx = O.gru_scan_bwd(Wi, Wh, b, x, O.sum_abs2_bwd(out))
    for i, g in enumerate((dWi, dWh, db, dx)):
        fd_check(loss, (Wi, Wh, b, x), g, i, rtol=1e-5, atol=1e-6)


# ---- attention: test/layers/attention.jl:3-63 ------------------------------------------------
def test_attention_shapes_and_causal_pattern():
    rng = np.random.default_rng(6)
    dim, nheads, L, B = 4, 2, 3, 5
    W = [rng.normal(size=(dim, dim)) for _ in range(4)]
    q = rng.normal(size=(dim, L, B))
    y, a = O.mha_fwd(*W, q, nheads=nheads)
    assert y.shape == (dim, L, B) and a.shape == (L, L, nheads, B)
    np.testing.assert_allclose(a.sum(axis=0), 1.0)
    y, a = O.mha_fwd(*W, q, nheads=nheads, mask=O.make_causal_mask(L))
    assert (a[1, 0, :, :] == 0).all()                      # alpha[2,1,:,:] == 0 (1-based)
    np.testing.assert_allclose(a[:, :, 0, 0], np.triu(a[:, :, 0, 0]))
    # bias used as a mask gives the same zero pattern (test/layers/attention.jl:45-54)
    bias = np.where(O.make_causal_mask(L), 0.0, -np.inf)
    y2, a2 = O.mha_fwd(*W, q, nheads=nheads, bias=bias)
    np.testing.assert_allclose(a2, a)
    # key/value of different length
    kv = rng.normal(size=(dim, 4, B))
    y3, a3 = O.mha_fwd(*W, q, kv, nheads=nheads)
    assert y3.shape == (dim, L, B) and a3.shape == (4, L, nheads, B)


def test_attention_bwd_fd():
    rng = np.random.default_rng(7)
    dim, nheads, L, B = 4, 2, 3, 2
    W = [rng.normal(size=(dim, dim)) * .5 for _ in range(4)]
    x = rng.normal(size=(dim, L, B))
    mask = O.make_causal_mask(L)
    y, _ = O.mha_fwd(*W, x, nheads=nheads, mask=mask)
    grads = O.mha_bwd(*W, x, O.sum_abs2_bwd(y), nheads=nheads, mask=mask)
    loss = lambda Wq, Wk, Wv, Wo, x_: O.sum_abs2(O.mha_fwd(Wq, Wk, Wv, Wo, x_, nheads=nheads, mask=mask)[0])
    for i, g in enumerate(grads):
        fd_check(loss, (*W, x), g, i, rtol=2e-5, atol=1e-6)


def test_attention_bias_dropout_and_alpha_cotangent_fd():
    """dot_product_attention with an additive bias, dropout on the weights and a loss that also reads the returned
    weights (test/layers/attention.jl:45-61): finite differences of q, k, v."""
    rng = np.random.default_rng(8)
    E, H, Lq, Lk, B = 4, 2, 3, 5, 2
    q, k, v = rng.normal(size=(E, Lq, B)), rng.normal(size=(E, Lk, B)), rng.normal(size=(E, Lk, B))
    bias = rng.normal(size=(Lk, Lq, H, 1))
    drop = (rng.random((Lk, Lq, H, B)) > 0.3) / 0.7
    wx, wa = rng.normal(size=(E, Lq, B)), rng.normal(size=(Lk, Lq, H, B))

    def loss(q_, k_, v_):
        x, a = O.dot_product_attention(q_, k_, v_, bias, H, None, drop=drop)
        return (x * wx).sum() + (a * wa).sum()
    grads = O.dot_product_attention_bwd(q, k, v, wx, bias, H, None, dalpha=wa, drop=drop)
    for i, g in enumerate(grads):
        fd_check(loss, (q, k, v), g, i, rtol=2e-5, atol=1e-6)


# ---- bf16 / init: test/utils.jl:311, 53-59, 95-104 -----------------------------------------
def test_bf16_exact_and_rounding():
    v = np.array([1, 1.5, -2.25, 96], dtype=np.float32)
    assert (O.bf16_round(v) == v).all()
    assert O.to_bf16_bits(np.float32(np.nan)) == 0x7FC0
    # round to nearest even on the 16 discarded bits
    u = np.array([0x3F808000, 0x3F818000, 0x3F808001], dtype=np.uint32).view(np.float32)
    assert list(O.to_bf16_bits(u)) == [0x3F80, 0x3F82, 0x3F81]


def test_nfan_and_glorot_variance():
    assert O.nfan() == (1, 1)
    assert O.nfan(100) == (1, 100)
    assert O.nfan(100, 10) == (10, 100)
    assert O.nfan(2, 30, 40) == (2 * 30, 2 * 40)
    assert O.nfan(2, 3, 40, 50) == (2 * 3 * 40, 2 * 3 * 50)
    rng = np.random.default_rng(0)
    for dims in [(1000,), (100, 100), (100, 400), (2, 3, 32, 64)]:
        v = O.glorot_uniform(rng, *dims)
        fi, fo = O.nfan(*dims)
        s2 = 2 / (fi + fo)
        assert 0.9 * s2 < v.var() < 1.1 * s2
        assert v.dtype == np.float32


# ---- Adam + training semantics: test/train.jl:37-47 (Descent known answer is host logic) ---
def test_adam_first_step_is_eta_sign():
    x = np.array([1.0, -2.0, 3.0], dtype=np.float32)
    g = np.array([0.5, -0.25, 4.0], dtype=np.float32)
    st = O.adam_init(x)
    x1 = O.adam_apply(st, x, g)
    np.testing.assert_allclose(x - x1, 1e-3 * np.sign(g), rtol=1e-4)
    assert st[2] == pytest.approx((0.81, 0.998001), rel=1e-6)


# ---- DistributedUtils: test/ext_distributed/{common,data}.jl --------------------------------
def test_distributed_closed_forms():
    for n in (2, 3, 4):
        bufs = [np.full(512, r + 1.0) for r in range(n)]
        assert all((b == sum(range(1, n + 1))).all() for b in O.allreduce(bufs, "+"))
        assert all((b == sum(range(1, n + 1)) / n).all() for b in O.allreduce(bufs, "avg"))
        assert all((b == 1.0).all() for b in O.bcast([np.ones(512) if r == 0 else np.zeros(512) for r in range(n)]))
        red = O.reduce(bufs, "+", root=0)
        assert (red[0] == sum(range(1, n + 1))).all() and (red[1] == 2.0).all()
        data = np.random.default_rng(0).random(10)
        shards = [O.distributed_shard_indices(10, n, r) for r in range(n) if r * int(np.ceil(10 / n)) < 10]
        assert len(shards[0]) == int(np.ceil(10 / n))
        assert sum(len(s) for s in shards) == 10
        assert abs(sum(data[s].sum() for s in shards) - data.sum()) < 1e-12


def test_committed_golden_fixture_roundtrip():
    """tests/golden/oracle_vectors.npz is generated by tests/golden/make_golden.py from this oracle
    on seeded inputs; the check guards the oracle against silent drift."""
    path = os.path.join(GOLD, "oracle_vectors.npz")
    if not os.path.exists(path):
        pytest.skip("golden fixture not generated yet")
    import sys
    sys.path.insert(0, GOLD)
    import make_golden
    fresh = make_golden.generate()
    stored = np.load(path)
    assert set(stored.files) == set(fresh.keys())
    for k in stored.files:
        np.testing.assert_allclose(stored[k], fresh[k], rtol=1e-12, atol=0, err_msg=k)


# ---- GroupNorm / InstanceNorm: test/layers/normalisation.jl:236-300, 392-445 --------------------
def test_groupnorm_frozen_literals():
    """The reference's frozen outputs for GroupNorm(4, 2) on reshape(1:24, 3, 4, 2), plain and with sigmoid
    (test/layers/normalisation.jl:410, 431)."""
    x = np.arange(1, 25, dtype=np.float64).reshape((3, 4, 2), order="F")
    y = O.groupnorm_fwd(x, np.ones(4), np.zeros(4), 2)
    ref1 = np.array([[-1.4638476, 0.29276943, -1.4638476, 0.29276943], [-0.87830865, 0.87830853, -0.8783088, 0.8783083],
                     [-0.29276967, 1.4638474, -0.2927699, 1.4638472]])
    ref2 = np.array([[-1.4638476, 0.29276943, -1.4638472, 0.29276943], [-0.8783083, 0.8783083, -0.8783083, 0.8783083],
                     [-0.29276943, 1.4638472, -0.29276943, 1.4638472]])
    np.testing.assert_allclose(y[:, :, 0], ref1, atol=1e-5)
    np.testing.assert_allclose(y[:, :, 1], ref2, atol=1e-5)
    ys = O.groupnorm_fwd(x, np.ones(4), np.zeros(4), 2, sigma="sigmoid")
    refs = np.array([[0.18787955, 0.57267404, 0.18787955, 0.57267404], [0.2935284, 0.70647156, 0.29352835, 0.70647156],
                     [0.42732593, 0.81212044, 0.42732587, 0.8121204]])
    np.testing.assert_allclose(ys[:, :, 0], refs, atol=1e-5)
    with pytest.raises(ValueError):
        O.groupnorm_fwd(x, np.ones(4), np.zeros(4), 3)


def test_instancenorm_known_answers():
    """test/layers/normalisation.jl:236-275: running mean [0.5, 0.8], running variance rule with n/(n-1); instance norm
    equals group norm with one channel per group (:441-445) and batch norm with channel and batch squashed (:348-352)."""
    x = np.arange(1, 13, dtype=np.float64).reshape((3, 2, 2), order="F")
    y, mu, var = O.instancenorm_fwd_train(x, np.ones(2), np.zeros(2), np.zeros(2), np.ones(2), 0.1, 1e-5, track_stats=True)
    np.testing.assert_allclose(mu, [0.5, 0.8])
    s2 = x.var(axis=0)          # biased variance over the spatial dim, shape (C, N)
    np.testing.assert_allclose(var, 0.1 * (3 / 2) * s2.mean(axis=1) + 0.9)
    xin = np.arange(1, 2 * 2 * 3 * 4 * 5 + 1, dtype=np.float64).reshape((2, 2, 3, 4, 5), order="F")
    a = O.instancenorm_fwd_train(xin, np.ones(4), np.zeros(4), None, None)[0]
    np.testing.assert_allclose(a, O.groupnorm_fwd(xin, np.ones(4), np.zeros(4), 4), rtol=1e-12)
    x6 = np.arange(1, 5 * 5 * 3 * 4 * 2 * 6 + 1, dtype=np.float64).reshape((5, 5, 3, 4, 2, 6), order="F")
    b = O.instancenorm_fwd_train(x6, np.ones(2), np.zeros(2), None, None)[0]
    xb = x6.reshape((5, 5, 3, 4, 12, 1), order="F")
    bn = O.batchnorm_fwd_train(xb, np.ones(12), np.zeros(12), None, None, track_stats=False)[0]
    np.testing.assert_allclose(b, bn.reshape(x6.shape, order="F"), rtol=1e-10, atol=1e-12)


@pytest.mark.parametrize("sigma,G", [("identity", 2), ("tanh", 1), ("relu", 4)])
def test_groupnorm_bwd_fd(sigma, G):
    rng = np.random.default_rng(1)
    x, g, b = rng.normal(size=(3, 2, 4, 2)), rng.normal(size=4) + 1.5, rng.normal(size=4)
    dy = rng.normal(size=x.shape)
    loss = lambda x_, g_, b_: (O.groupnorm_fwd(x_, g_, b_, G, sigma=sigma) * dy).sum()
    dx, dg, db = O.groupnorm_bwd(x, g, b, dy, G, sigma=sigma)
    fd_check(loss, (x, g, b), dx, 0, rtol=1e-4, atol=1e-6)
    fd_check(loss, (x, g, b), dg, 1, rtol=1e-4, atol=1e-6)
    fd_check(loss, (x, g, b), db, 2, rtol=1e-4, atol=1e-6)


# ---- Embedding: src/layers/basic.jl:752-776 (doctest values) -------------------------------------
def test_embedding_known_answers_and_gradient():
    W = np.zeros((4, 26))
    W[np.arange(4), np.arange(4)] = 22.0          # identity_init(gain = 22)
    np.testing.assert_array_equal(O.embedding_fwd(W, 2), [0, 22, 0, 0])
    y = O.embedding_fwd(W, np.array([3, 1, 20, 14, 4, 15, 7]))
    assert y.shape == (4, 7) and y[2, 0] == 22 and y[0, 1] == 22 and y[3, 4] == 22 and y.sum() == 66
    assert O.embedding_fwd(W, np.ones((10, 1, 12), int)).shape == (4, 10, 1, 12)
    rng = np.random.default_rng(0)
    W = rng.normal(size=(3, 5))
    idx = np.array([[1, 2, 2], [5, 1, 2]])
    assert (O.embedding_fwd(W, idx, padding_idx=1)[:, 0, 0] == 0).all()
    dy = rng.normal(size=(3, 2, 3))
    dW = O.embedding_bwd(W, idx, dy, padding_idx=1)
    fd_check(lambda W_: (O.embedding_fwd(W_, idx, padding_idx=1) * dy).sum(), (W,), dW, 0)
    assert (dW[:, 0] == 0).all() and (dW[:, 2] == 0).all()
    with pytest.raises(IndexError):
        O.embedding_fwd(W, np.array([6]))


# ---- Dropout mask generator ------------------------------------------------------------------------
def test_philox_known_answers_and_dropout_statistics():
    """Philox4x32-10 known-answer vectors of the Random123 distribution (kat_vectors: all-zero and all-ones inputs do
    not fit this generator's (64-bit counter, 64-bit key) form, so the zero vector and the round structure are pinned;
    the keep rate is checked statistically like test/layers/normalisation.jl:10-30 does for Dropout)."""
    out = O.philox4x32_10(np.array([0], dtype=np.uint64), 0)[0]
    assert [hex(int(v)) for v in out] == ["0x6627e8d5", "0xe169c58d", "0xbc57ac4c", "0x9b00dbd8"]
    m = O.dropout_mask(100000, 0.3, seed=7)
    assert abs(m.mean() - 0.7) < 0.01
    assert (O.dropout_mask(1000, 0.0, 1)).all() and not O.dropout_mask(1000, 1.0, 1).any()
    # disjoint counter ranges give independent masks; the same (seed, offset) reproduces the mask
    assert (O.dropout_mask(64, 0.5, 3, offset=16) == O.dropout_mask(128, 0.5, 3)[64:]).all()
    x = np.ones(10)
    y = O.dropout_fwd(x, 0.5, O.dropout_mask(10, 0.5, 1))
    assert set(np.unique(y)) <= {0.0, 2.0}


# ---- RNNCell / GRUv3Cell: recurrent.jl:193-198, 795-809 -------------------------------------------
@pytest.mark.parametrize("sigma", ["tanh", "relu"])
def test_rnn_bwd_fd(sigma):
    rng = np.random.default_rng(2)
    I, H, T, B = 3, 4, 5, 2
    Wi, Wh, b, x = rng.normal(size=(H, I)) * .5, rng.normal(size=(H, H)) * .5, rng.normal(size=H) * .1, rng.normal(size=(I, T, B))
    dout = rng.normal(size=(H, T, B))
    loss = lambda Wi_, Wh_, b_, x_: (O.rnn_scan_fwd(Wi_, Wh_, b_, x_, sigma)[0] * dout).sum()
    dWi, dWh, db, dx = O.rnn_scan_bwd(Wi, Wh, b, x, dout, sigma)
    for i, g in enumerate((dWi, dWh, db, dx)):
        fd_check(loss, (Wi, Wh, b, x), g, i, rtol=1e-4, atol=1e-6)
    # zero initial state and cell(x) == cell(x, zeros) (test/layers/recurrent.jl:24-40)
    o1, _ = O.rnn_scan_fwd(Wi, Wh, b, x, sigma)
    o2, _ = O.rnn_scan_fwd(Wi, Wh, b, x, sigma, h0=np.zeros(H))
    assert (o1 == o2).all()


def test_gruv3_bwd_fd():
    rng = np.random.default_rng(3)
    I, H, T, B = 3, 4, 5, 2
    Wi, Wh, b = rng.normal(size=(3 * H, I)) * .5, rng.normal(size=(3 * H, H)) * .5, rng.normal(size=3 * H) * .1
    Whh, x, dout = rng.normal(size=(H, H)) * .5, rng.normal(size=(I, T, B)), rng.normal(size=(H, T, B))
    loss = lambda Wi_, Wh_, b_, Whh_, x_: (O.gruv3_scan_fwd(Wi_, Wh_, b_, Whh_, x_)[0] * dout).sum()
    grads = O.gruv3_scan_bwd(Wi, Wh, b, Whh, x, dout)
    for i, g in enumerate(grads):
        fd_check(loss, (Wi, Wh, b, Whh, x), g, i, rtol=1e-4, atol=1e-6)
    assert (grads[1][2 * H:] == 0).all()      # the third row block of Wh is never read (recurrent.jl:804)
