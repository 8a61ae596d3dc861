"""GPU tests of the host-side mirror of Flux's API (Chain / Dense / norms / Recurrence / MultiHeadAttention /
withgradient / setup / trainstep! / train!) against the oracle, written the way the reference's own layer
and training tests read (test/layers/*.jl, test/train.jl, test/ext_cuda/layers.jl)."""
import numpy as np
import pytest

import flux_oracle as O
from util import close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def F():
    import fluxb200
    yield fluxb200
    assert fluxb200.context().device_error() == 0


def test_dense_layer_shapes_errors_and_gradient_tree(F):
    """test/layers/basic.jl:70-108; gradient field names as src/gradient.jl:112."""
    rng = np.random.default_rng(0)
    W = O.glorot_uniform(rng, 5, 10)
    d = F.Dense(W)
    for shp in [(10,), (10, 2), (10, 2, 3), (10, 2, 3, 4)]:
        assert d(F.gpu(rng.normal(size=shp).astype(np.float32))).size == (5,) + shp[1:]
    with pytest.raises(F.DimensionMismatch):
        d(F.gpu(np.zeros((11, 2, 3), np.float32)))
    with pytest.raises(F.DimensionMismatch):
        d(F.gpu(np.zeros((1,), np.float32)))
    x = rng.normal(size=(10, 4))
    close(F.cpu(d(F.gpu(x))), W.astype(np.float64) @ x)          # Float64 input is converted (_match_eltype)
    d2 = F.Dense(W, False)
    x32 = F.gpu(x.astype(np.float32))
    val, (g,) = F.withgradient(lambda m: F.sum_abs2(m(x32)), d2)
    assert set(g) == {"weight", "bias", "σ"} and g["bias"] is None and g["σ"] is None   # test/ext_cuda/layers.jl:120-127
    y = W.astype(np.float64) @ x
    close(val, (y * y).sum())
    close(F.cpu(g["weight"]), 2 * y @ x.T)


def test_mlp_config1_ten_adam_steps_match_oracle(F):
    """Chain(Dense(784=>512,relu), Dense(512=>512,relu), Dense(512=>10)), batch 1024, logitcrossentropy, Adam(1e-3).

    Adam's normalised step amplifies rounding noise wherever a gradient changes sign between steps (a Float32 and
    a Float64 run of the oracle itself drift apart by several eta within ten steps), so a free-running trajectory
    is not a well-posed parity target.  Every step therefore starts from the oracle's state (parameters, moments,
    beta powers): the device runs one full trainstep from it and loss and updated parameters are compared."""
    import torch
    rng = np.random.default_rng(0)
    dims = [(512, 784, "relu"), (512, 512, "relu"), (10, 512, "identity")]
    Ws = [O.glorot_uniform(rng, o, i) for o, i, _ in dims]
    bs = [np.zeros(o, np.float32) for o, _, _ in dims]
    x = rng.random((784, 1024), dtype=np.float32)
    labels = rng.integers(1, 11, size=1024)
    model = F.Chain(*[F.Dense(W.copy(), b.copy(), s) for W, b, (_, _, s) in zip(Ws, bs, dims)])
    opt = F.setup(F.Adam(1e-3), model)
    xg, yg = F.gpu(x), F.onehotbatch(labels, 10)
    loss = lambda m, x_, y_: F.logitcrossentropy(m(x_), y_)
    W64 = [w.astype(np.float64) for w in Ws]
    b64 = [b.astype(np.float64) for b in bs]
    st = [(O.adam_init(w), O.adam_init(b)) for w, b in zip(W64, b64)]
    y1h = O.onehotbatch(labels, 10, np.float64)

    def put(arr, value):
        arr.t.copy_(torch.from_numpy(np.ascontiguousarray(value.astype(np.float32).reshape(-1, order="F"))))

    for step in range(10):
        for i, layer in enumerate(model.layers):
            for p, val, state in ((layer.weight, W64[i], st[i][0]), (layer.bias, b64[i], st[i][1])):
                leaf = opt.leaves[id(p)]
                put(p, val)
                put(leaf.state[0], state[0])
                put(leaf.state[1], state[1])
                leaf.state[2] = (float(np.float32(state[2][0])), float(np.float32(state[2][1])))
        l = F.trainstep(loss, model, (xg, yg), opt)
        lref, grads, _ = O.mlp_chain_fwd_bwd([(w, b, s) for w, b, (_, _, s) in zip(W64, b64, dims)], x.astype(np.float64), y1h)
        close(l, lref, name=f"loss step {step}")
        for i, (dW, db) in enumerate(grads):
            W64[i] = O.adam_apply(st[i][0], W64[i], dW)
            b64[i] = O.adam_apply(st[i][1], b64[i], db)
        for i, layer in enumerate(model.layers):
            gabs = np.abs(grads[i][0])
            solid = gabs > 1e-2 * gabs.max()          # gradient well above rounding noise
            got, ref = F.cpu(layer.weight), W64[i]
            # a gradient error of 1e-4 * max|g| (the parity tolerance) moves an update by at most ~1e-2 * eta here
            bad = np.abs(got[solid] - ref[solid]) > 2e-5
            assert bad.mean() < 1e-3, f"step {step} W{i}: {bad.sum()} of {bad.size} updates differ"   # relu units at 0 may flip
            assert np.max(np.abs(got - ref)) < 2.1e-3  # nothing moves further than one Adam step from the oracle


def test_mlp_gradients_match_oracle(F):
    rng = np.random.default_rng(1)
    dims = [(64, 48, "tanh"), (32, 64, "gelu"), (7, 32, "identity")]
    layers = [(O.glorot_uniform(rng, o, i), (rng.normal(size=o) * 0.1).astype(np.float32), s) for o, i, s in dims]
    x = rng.normal(size=(48, 33)).astype(np.float32)
    labels = rng.integers(1, 8, size=33)
    model = F.Chain(*[F.Dense(W, b, s) for W, b, s in layers])
    xg, yg = F.gpu(x), F.onehotbatch(labels, 7)
    val, (g,) = F.withgradient(lambda m: F.logitcrossentropy(m(xg), yg), model)
    ref_layers = [(W.astype(np.float64), b.astype(np.float64), "gelu_tanh" if s == "gelu" else s) for W, b, s in layers]
    lref, grads, _ = O.mlp_chain_fwd_bwd(ref_layers, x.astype(np.float64), O.onehotbatch(labels, 7, np.float64))
    close(val, lref)
    for gi, (dW, db) in zip(g["layers"], grads):
        close(F.cpu(gi["weight"]), dW)
        close(F.cpu(gi["bias"]), db)


def test_trainstep_semantics(F):
    """test/train.jl:37-47 (stop on NaN after 50 Descent(0.1) steps, weight == -5), :130-141 (update skipped),
    :89-94 (returned loss is pre-update)."""
    m1 = F.Dense(np.zeros((1, 1), np.float32))
    opt = F.setup(F.Descent(0.1), m1)
    one = F.gpu(np.ones((1,), np.float32))
    cnt = [0]

    def loss(m, i):
        cnt[0] += 1
        return F.scale(float("nan") if i == 51 else 1.0, F.sum_all(m(one)))

    with pytest.raises(F.DomainError):
        F.train(loss, m1, [(i,) for i in range(1, 101)], opt)
    assert cnt[0] == 51
    assert abs(F.cpu(m1.weight)[0, 0] + 5) < 1e-5
    m2 = F.Dense(np.zeros((1, 1), np.float32))
    opt2 = F.setup(F.Descent(0.1), m2)
    l = F.trainstep(lambda m, i: F.scale(float("nan"), F.sum_all(m(one))), m2, (1,), opt2)
    assert not np.isfinite(l)
    assert F.cpu(m2.weight)[0, 0] == 0 and F.cpu(m2.bias)[0] == 0
    m3 = F.Dense(np.ones((1, 1), np.float32))
    opt3 = F.setup(F.Descent(0.1), m3)
    l3 = F.trainstep(lambda m: F.sum_all(m(one)), m3, (), opt3)
    assert abs(l3 - 1.0) < 1e-6 and abs(F.cpu(m3.weight)[0, 0] - 0.9) < 1e-6


def test_batchnorm_layer_modes(F):
    """test/layers/normalisation.jl:125-159 and test/ext_cuda/layers.jl:129-181: statistics are tracked only
    in gradient / train mode; test mode uses them."""
    x = np.array([[1.0, 3.0, 5.0], [2.0, 4.0, 6.0]], np.float32)
    m = F.BatchNorm(2)
    assert len(F.trainables(m)) == 2
    xg = F.gpu(x)
    y = F.cpu(m(xg))                                   # outside a gradient call: inference with mu = 0, var = 1
    np.testing.assert_allclose(y, x / np.sqrt(1 + 1e-5), rtol=1e-6)
    np.testing.assert_allclose(F.cpu(m.μ), [0, 0])
    val, (g,) = F.withgradient(lambda mm: F.sum_abs2(mm(xg)), m)
    np.testing.assert_allclose(F.cpu(m.μ), [0.3, 0.4], rtol=1e-6)
    np.testing.assert_allclose(F.cpu(m.σ2), [1.3, 1.3], rtol=1e-6)
    assert g["μ"] is None and g["γ"] is not None
    F.trainmode(m)
    np.testing.assert_allclose(F.cpu(m(xg)), [[-1.22474, 0, 1.22474]] * 2, atol=1e-5)
    F.testmode(m)
    assert abs(F.cpu(m(xg))[0, 0] - (1 - F.cpu(m.μ)[0]) / np.sqrt(F.cpu(m.σ2)[0] + 1e-5)) < 1e-5
    m1 = F.trainmode(F.BatchNorm(1))
    with pytest.raises(F.ArgumentError):
        m1(F.gpu(np.zeros((1, 1), np.float32)))
    m1(F.gpu(np.arange(4, dtype=np.float32).reshape(4, 1, 1)))
    with pytest.raises(F.DimensionMismatch):
        F.BatchNorm(3)(xg)


def test_layernorm_layer(F):
    rng = np.random.default_rng(2)
    x = rng.random((2, 3, 4, 5)).astype(np.float32)
    y = F.cpu(F.LayerNorm(2)(F.gpu(x)))
    x64 = x.astype(np.float64)
    close(y, (x64 - x64.mean(0, keepdims=True)) / np.sqrt(x64.var(0, keepdims=True) + 1e-5))
    y2 = F.cpu(F.LayerNorm(2, 3)(F.gpu(x)))
    close(y2, (x64 - x64.mean((0, 1), keepdims=True)) / np.sqrt(x64.var((0, 1), keepdims=True) + 1e-5))
    m = F.LayerNorm((2, 3, 4))
    assert len(F.trainables(m)) == 2 and len(F.trainables(F.LayerNorm((2, 3, 4), affine=False))) == 0
    with pytest.raises(F.DimensionMismatch):
        F.LayerNorm(3)(F.gpu(x))


def test_recurrence_lstm_gru(F):
    """test/layers/recurrent.jl:113-197, 336-356: zero initial state, state shapes, Recurrence(cell) == LSTM(...)."""
    rng = np.random.default_rng(3)
    I, H, T, B = 5, 8, 6, 4
    x = rng.normal(size=(I, T, B)).astype(np.float32)
    xg = F.gpu(x)
    for ng, Cell, Wrap, fwd, bwd in [(4, F.LSTMCell, F.LSTM, O.lstm_scan_fwd, O.lstm_scan_bwd),
                                     (3, F.GRUCell, F.GRU, O.gru_scan_fwd, O.gru_scan_bwd)]:
        Wi, Wh = O.glorot_uniform(rng, ng * H, I), O.glorot_uniform(rng, ng * H, H)
        b = (rng.normal(size=ng * H) * 0.1).astype(np.float32)
        rnn = F.Recurrence(Cell(Wi, Wh, b))
        y = rnn(xg)
        assert y.size == (H, T, B)
        ref = fwd(*[a.astype(np.float64) for a in (Wi, Wh, b, x)])[0]
        close(F.cpu(y), ref)
        close(F.cpu(Wrap(Wi, Wh, b)(xg)), ref)
        y0 = rnn(xg, rnn.cell.initialstates())            # explicit zero state vectors broadcast over the batch
        np.testing.assert_array_equal(F.cpu(y0), F.cpu(y))
        out, state = F.Recurrence(Cell(Wi, Wh, b), return_state=True)(xg)
        hT = state[0] if ng == 4 else state
        assert hT.size == (H, B)
        np.testing.assert_array_equal(F.cpu(hT), F.cpu(out)[:, -1, :])
        val, (g,) = F.withgradient(lambda m: F.sum_abs2(m(xg)), rnn)
        dWi, dWh, db, _ = bwd(*[a.astype(np.float64) for a in (Wi, Wh, b, x)], O.sum_abs2_bwd(ref))
        close(val, (ref * ref).sum())
        close(F.cpu(g["cell"]["Wi"]), dWi, rtol=2e-4, atol_scale=2e-4)
        close(F.cpu(g["cell"]["Wh"]), dWh, rtol=2e-4, atol_scale=2e-4)
        close(F.cpu(g["cell"]["bias" if ng == 4 else "b"]), db, rtol=2e-4, atol_scale=2e-4)
        y2 = rnn(F.gpu(x[:, :, 0]))                        # 2-d input: (features, len)
        assert y2.size == (H, T)


def test_bf16_model_runs_the_low_precision_dense_path(F):
    """bf16(model) (src/functor.jl:274): parameters hold BFloat16 values, Dense multiplies them exactly and accumulates
    in Float32, outputs and gradients are BFloat16 values; tolerance 2e-2 against the Float64 oracle on the same
    rounded operands (in fact within a bf16 ulp)."""
    rng = np.random.default_rng(21)
    W1, W2 = O.glorot_uniform(rng, 96, 64), O.glorot_uniform(rng, 32, 96)
    b1 = (rng.normal(size=96) * 0.1).astype(np.float32)
    x = rng.normal(size=(64, 50)).astype(np.float32)
    model = F.bf16(F.Chain(F.Dense(W1, b1, "relu"), F.Dense(W2, False)))
    xb = F.bf16(F.gpu(x))
    is_bf16 = lambda a: ((np.asarray(a, np.float32).view(np.uint32) & 0xFFFF) == 0).all()
    assert is_bf16(F.cpu(model.layers[0].weight)) and is_bf16(F.cpu(model.layers[0].bias)) and is_bf16(F.cpu(xb))
    np.testing.assert_array_equal(F.cpu(model.layers[0].weight), O.bf16_round(W1))
    y = F.cpu(model(xb))
    assert is_bf16(y)
    W1r, W2r, b1r, xr = (O.bf16_round(a).astype(np.float64) for a in (W1, W2, b1, x))
    h = O.bf16_round(O.dense_fwd(W1r, b1r, xr, "relu").astype(np.float32)).astype(np.float64)
    yref = O.dense_fwd(W2r, None, h)
    np.testing.assert_allclose(y, yref, rtol=2e-2, atol=2e-2 * np.abs(yref).max())
    assert np.abs(y - yref).max() <= 2.0 ** -7 * np.abs(yref).max()
    val, (g,) = F.withgradient(lambda m: F.sum_abs2(m(xb)), model)
    assert is_bf16(F.cpu(g["layers"][0]["weight"])) and is_bf16(F.cpu(g["layers"][1]["weight"]))
    dy = O.sum_abs2_bwd(yref)
    dW2, _, dh = O.dense_bwd(W2r, None, h, dy)
    np.testing.assert_allclose(F.cpu(g["layers"][1]["weight"]), dW2, rtol=2e-2, atol=2e-2 * np.abs(dW2).max())
    dW1, _, _ = O.dense_bwd(W1r, b1r, xr, dh, "relu")
    np.testing.assert_allclose(F.cpu(g["layers"][0]["weight"]), dW1, rtol=2e-2, atol=2e-2 * np.abs(dW1).max())
    F.f32(model)
    assert model.layers[0].precision == "default"


def test_graphed_gradient_replays_withgradient(F):
    rng = np.random.default_rng(22)
    W = O.glorot_uniform(rng, 48, 32)
    model = F.Chain(F.LayerNorm(32), F.Dense(W, True, "gelu"))
    x0, x1 = (rng.normal(size=(32, 20)).astype(np.float32) for _ in range(2))
    xg = F.gpu(x0)
    fn = lambda m: F.sum_abs2(m(xg))
    gg = F.GraphedGradient(fn, model)
    for xv in (x0, x1, x0):
        xg.t.copy_(F.gpu(xv).t)                 # new values in the same device buffer
        loss, tree = gg()
        val, (g,) = F.withgradient(fn, model)
        assert abs(float(F.cpu(loss)) - val) <= 1e-6 * abs(val)
        np.testing.assert_allclose(F.cpu(tree["layers"][1]["weight"]), F.cpu(g["layers"][1]["weight"]), rtol=1e-6, atol=1e-7)
        np.testing.assert_allclose(F.cpu(tree["layers"][0]["diag"]["scale"]), F.cpu(g["layers"][0]["diag"]["scale"]), rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("cell,B", [("lstm", 5), ("lstm", 16), ("gru", 32)])
def test_graphed_gradient_of_a_recurrent_layer_matches_eager(F, cell, B):
    """The persistent recurrent kernels are launched cooperatively by eager calls and plainly inside a captured
    step (B = 16 / 32 take the register-tiled forward kernel): same numbers, no device error."""
    rng = np.random.default_rng(23)
    H, I, T = 32, 16, 9
    ng = 4 if cell == "lstm" else 3
    rnn = (F.LSTM if cell == "lstm" else F.GRU)(O.glorot_uniform(rng, ng * H, I), O.glorot_uniform(rng, ng * H, H))
    xg = F.gpu(rng.normal(size=(I, T, B)).astype(np.float32))
    fn = lambda m: F.sum_abs2(m(xg))
    val, (g,) = F.withgradient(fn, rnn)
    gg = F.GraphedGradient(fn, rnn)
    loss, tree = gg()
    assert abs(float(F.cpu(loss)) - val) <= 1e-5 * abs(val)

    def leaves(t):
        if isinstance(t, dict):
            for v in t.values():
                yield from leaves(v)
        elif t is not None:
            yield t
    for a, b in zip(leaves(tree), leaves(g)):
        np.testing.assert_allclose(F.cpu(a), F.cpu(b), rtol=1e-4, atol=1e-5 * float(np.abs(F.cpu(b)).max()))
    assert F.context().device_error() == 0


def test_multiheadattention_head_size_64_runs_the_tensor_core_kernels(F):
    """Same checks as the small layer test at a head size the tcgen05 attention kernels take (forward, dQ, dK / dV),
    over several key / query blocks with a ragged tail."""
    rng = np.random.default_rng(14)
    dim, nheads, L, B = 128, 2, 210, 2
    Ws = [O.glorot_uniform(rng, dim, dim) for _ in range(4)]
    mha = F.MultiHeadAttention(*Ws, nheads=nheads)
    q = rng.normal(size=(dim, L, B)).astype(np.float32)
    qg = F.gpu(q)
    W64 = [w.astype(np.float64) for w in Ws]
    for causal in (False, True):
        mk = (lambda: F.make_causal_mask(qg)) if causal else (lambda: None)
        omask = O.make_causal_mask(L) if causal else None
        y, a = mha(qg, mask=mk())
        yref, aref = O.mha_fwd(*W64, q.astype(np.float64), nheads=nheads, mask=omask)
        np.testing.assert_allclose(F.cpu(y), yref, atol=1e-4)
        np.testing.assert_allclose(F.cpu(a.materialize()), aref, atol=1e-4)
        val, (g,) = F.withgradient(lambda m: F.sum_abs2(m(qg, mask=mk())[0]), mha)
        dWq, dWk, dWv, dWo, _ = O.mha_bwd(*W64, q.astype(np.float64), O.sum_abs2_bwd(yref), nheads=nheads, mask=omask)
        for name, ref in [("q_proj", dWq), ("k_proj", dWk), ("v_proj", dWv), ("out_proj", dWo)]:
            close(F.cpu(g[name]["weight"]), ref, rtol=2e-4, atol_scale=2e-4, name=name)
    assert F.context().device_error() == 0


def test_multiheadattention_layer(F):
    """test/layers/attention.jl:3-63 and test/ext_cuda/layers.jl:343-363 (y and alpha, atol 1e-4)."""
    rng = np.random.default_rng(4)
    dim, nheads, L, B = 16, 4, 10, 3
    Ws = [O.glorot_uniform(rng, dim, dim) for _ in range(4)]
    mha = F.MultiHeadAttention(*Ws, nheads=nheads)
    q = rng.normal(size=(dim, L, B)).astype(np.float32)
    qg = F.gpu(q)
    W64 = [w.astype(np.float64) for w in Ws]
    y, a = mha(qg)
    assert y.size == (dim, L, B) and a.size == (L, L, nheads, B)
    yref, aref = O.mha_fwd(*W64, q.astype(np.float64), nheads=nheads)
    np.testing.assert_allclose(F.cpu(y), yref, atol=1e-4)
    np.testing.assert_allclose(F.cpu(a.materialize()), aref, atol=1e-4)
    y, a = mha(qg, mask=F.make_causal_mask(qg))
    al = F.cpu(a.materialize())
    assert (al[1, 0, :, :] == 0).all()
    np.testing.assert_allclose(al[:, :, 0, 0], np.triu(al[:, :, 0, 0]))
    yref, aref = O.mha_fwd(*W64, q.astype(np.float64), nheads=nheads, mask=O.make_causal_mask(L))
    np.testing.assert_allclose(F.cpu(y), yref, atol=1e-4)
    kv = rng.normal(size=(dim, 7, B)).astype(np.float32)
    y, a = mha(qg, F.gpu(kv))
    assert y.size == (dim, L, B) and a.size == (7, L, nheads, B)
    val, (g,) = F.withgradient(lambda m: F.sum_abs2(m(qg, mask=F.make_causal_mask(qg))[0]), mha)
    dWq, dWk, dWv, dWo, _ = O.mha_bwd(*W64, q.astype(np.float64), O.sum_abs2_bwd(yref), nheads=nheads, mask=O.make_causal_mask(L))
    for name, ref in [("q_proj", dWq), ("k_proj", dWk), ("v_proj", dWv), ("out_proj", dWo)]:
        close(F.cpu(g[name]["weight"]), ref, rtol=2e-4, atol_scale=2e-4, name=name)
        assert g[name]["bias"] is None
    with pytest.raises(F.ArgumentError):
        F.MultiHeadAttention(*Ws, nheads=3)


def test_dp_block_model_gradients_match_oracle(F):
    """The data-parallel benchmark model at reduced width: LayerNorm -> Dense(gelu) blocks + classifier."""
    rng = np.random.default_rng(5)
    D, Cc, N, nb = 256, 40, 96, 3
    blocks = [{"gamma": (rng.normal(size=D) * 0.1 + 1).astype(np.float32), "beta": (rng.normal(size=D) * 0.1).astype(np.float32),
               "W": O.glorot_uniform(rng, D, D), "b": np.zeros(D, np.float32)} for _ in range(nb)]
    head = {"W": O.glorot_uniform(rng, Cc, D), "b": np.zeros(Cc, np.float32)}
    x = rng.normal(size=(D, N)).astype(np.float32)
    labels = rng.integers(1, Cc + 1, size=N)
    layers = []
    for blk in blocks:
        ln = F.LayerNorm(D)
        ln.diag.scale, ln.diag.bias = F.gpu(blk["gamma"]), F.gpu(blk["beta"])
        layers += [ln, F.Dense(blk["W"], blk["b"], "gelu")]
    layers.append(F.Dense(head["W"], head["b"]))
    model = F.Chain(*layers)
    xg, yg = F.gpu(x), F.onehotbatch(labels, Cc)
    val, (g,) = F.withgradient(lambda m: F.logitcrossentropy(m(xg), yg), model)
    to64 = lambda d: {k: v.astype(np.float64) for k, v in d.items()}
    lref, gb, gh = O.dp_mlp_fwd_bwd([to64(b) for b in blocks], to64(head), x.astype(np.float64), O.onehotbatch(labels, Cc, np.float64))
    close(val, lref)
    for i, ref in enumerate(gb):
        close(F.cpu(g["layers"][2 * i]["diag"]["scale"]), ref["gamma"], rtol=2e-4, atol_scale=2e-4)
        close(F.cpu(g["layers"][2 * i]["diag"]["bias"]), ref["beta"], rtol=2e-4, atol_scale=2e-4)
        close(F.cpu(g["layers"][2 * i + 1]["weight"]), ref["W"], rtol=2e-4, atol_scale=2e-4)
        close(F.cpu(g["layers"][2 * i + 1]["bias"]), ref["b"], rtol=2e-4, atol_scale=2e-4)
    close(F.cpu(g["layers"][-1]["weight"]), gh["W"], rtol=2e-4, atol_scale=2e-4)


def test_graphed_trainstep_equals_eager_and_skips_on_nan(F):
    """The one-launch (CUDA graph) train step against the eager `trainstep` on identical models, and the
    non-finite-loss rule of `_eager_step!` (src/train.jl:377; test/train.jl:130-141) inside the graph."""
    rng = np.random.default_rng(11)
    D, Cc, N = 128, 10, 64
    Ws = [O.glorot_uniform(rng, D, D), O.glorot_uniform(rng, Cc, D)]
    x = rng.standard_normal((D, N), dtype=np.float32)
    labels = rng.integers(1, Cc + 1, size=N)

    def build():
        ln = F.LayerNorm(D)
        return F.Chain(ln, F.Dense(Ws[0].copy(), True, "gelu"), F.Dense(Ws[1].copy(), True))

    loss = lambda m, x_, y_: F.logitcrossentropy(m(x_), y_)
    xg, yg = F.gpu(x), F.onehotbatch(labels, Cc)
    m1, m2 = build(), build()
    o1, o2 = F.setup(F.Adam(1e-3), m1), F.setup(F.Adam(1e-3), m2)
    gstep = F.GraphedTrainStep(loss, m2, o2, (xg, yg))
    for step in range(4):
        l1 = F.trainstep(loss, m1, (xg, yg), o1)
        l2 = gstep(xg, yg)
        assert l1 == l2, (step, l1, l2)
    for a, b in zip(F.trainables(m1), F.trainables(m2)):
        np.testing.assert_array_equal(F.cpu(a), F.cpu(b))
    assert o1.leaves[id(F.trainables(m1)[0])].state[2] == pytest.approx(o2.leaves[id(F.trainables(m2)[0])].state[2])
    # a batch that makes the loss NaN: parameters, moments and the beta powers stay as they are
    before = [F.cpu(p).copy() for p in F.trainables(m2)]
    bt_before = gstep.bt.cpu().numpy().copy()
    xbad = x.copy()
    xbad[0, 0] = np.nan
    lbad = gstep(F.gpu(xbad), yg)
    assert not np.isfinite(lbad)
    for p, b in zip(F.trainables(m2), before):
        np.testing.assert_array_equal(F.cpu(p), b)
    np.testing.assert_array_equal(gstep.bt.cpu().numpy(), bt_before)
    # and the step keeps working afterwards
    l3 = gstep(xg, yg)
    assert np.isfinite(l3) and l3 < l2 + 1e-3
    # prefetched batches (pinned host tensors copied beside the running step) give the same steps as direct ones
    import torch
    xh = torch.from_numpy(np.ascontiguousarray(x.T).reshape(-1)).pin_memory()          # memory order of x[in, N]
    lh = torch.from_numpy(np.asarray(labels).astype(np.int32)).pin_memory()            # 1-based labels, as on the device
    assert torch.equal(yg.labels.t.cpu(), lh)
    gstep.prefetch(xh, lh)
    l4 = F.trainstep(loss, m1, (xg, yg), o1)          # m1 is one good step behind m2: bring it level first
    l5a = gstep(prefetch=(xh, lh))
    l5b = gstep()
    l4b = F.trainstep(loss, m1, (xg, yg), o1)
    l4c = F.trainstep(loss, m1, (xg, yg), o1)
    assert l4 == l3 and l5a == l4b and l5b == l4c, (l3, l4, l5a, l4b, l5b, l4c)


def test_pair_constructors_use_glorot_uniform(F):
    """Dense(in => out, σ), LSTMCell(in => out), GRUCell(in => out), MultiHeadAttention(dims; nheads)
    (basic.jl:189-192, recurrent.jl:395-407, 596-607, attention.jl:79-94): shapes, zero biases, init scale."""
    F.seed(1)
    d = F.Dense((10, 6), "relu")
    assert d.weight.size == (6, 10) and d.bias.size == (6,) and d.σ == "relu" and (F.cpu(d.bias) == 0).all()
    assert np.abs(F.cpu(d.weight)).max() <= 0.5 * np.sqrt(24 / 16) + 1e-6
    assert F.Dense((10, 6), bias=False).bias is False
    ones = F.Dense((10, 1), init=lambda o, i: np.ones((o, i), np.float32))       # test/layers/basic.jl:85
    assert F.cpu(ones(F.gpu(np.ones((10, 1), np.float32)))).item() == 10
    c = F.LSTMCell((3, 5))
    assert c.Wi.size == (20, 3) and c.Wh.size == (20, 5) and c.bias.size == (20,)
    g = F.GRUCell((3, 5))
    assert g.Wi.size == (15, 3) and g.Wh.size == (15, 5) and g.b.size == (15,)
    assert F.LSTM((3, 5))(F.gpu(np.zeros((3, 4, 2), np.float32))).size == (5, 4, 2)
    m = F.MultiHeadAttention(16, nheads=2)
    assert m.q_proj.weight.size == (16, 16) and m.q_proj.bias is False
    m2 = F.MultiHeadAttention(((4, 6, 8), ((12, 10), 14)), nheads=2, bias=True)     # (q_in,k_in,v_in) => (qk, v) => out
    assert (m2.q_proj.weight.size, m2.k_proj.weight.size, m2.v_proj.weight.size, m2.out_proj.weight.size) == \
        ((12, 4), (12, 6), (10, 8), (14, 10))
    with pytest.raises(F.ArgumentError):
        F.MultiHeadAttention(10, nheads=3)


def test_layer_applied_twice_accumulates_into_the_gradient_bucket(F):
    """A Dense used twice in one model (tied weights): both contributions must reach the flat gradient buffer of a
    GradBuckets sink, and the bucket may only start after the second one."""
    DU = F.DistributedUtils
    rng = np.random.default_rng(5)
    W, b = O.glorot_uniform(rng, 32, 32), (rng.normal(size=32) * 0.1).astype(np.float32)
    x = rng.normal(size=(32, 9)).astype(np.float32)
    layer = F.Dense(W, b, "tanh")
    model = F.Chain(layer, layer)
    backend = DU.initialize(DU.NCCLBackend)
    sink = DU.GradBuckets(backend, F.trainables(layer), bucket_mb=0.001)
    xg = F.gpu(x)
    val, (g,) = F.withgradient(lambda m: F.sum_abs2(m(xg)), model, grad_sink=sink)
    W64, b64, x64 = W.astype(np.float64), b.astype(np.float64), x.astype(np.float64)
    h = O.dense_fwd(W64, b64, x64, "tanh")
    y = O.dense_fwd(W64, b64, h, "tanh")
    dW2, db2, dh = O.dense_bwd(W64, b64, h, 2 * y, "tanh")
    dW1, db1, _ = O.dense_bwd(W64, b64, x64, dh, "tanh")
    close(val, (y * y).sum())
    close(F.cpu(sink.views[id(layer.weight)]), dW1 + dW2, name="dW in the bucket", rtol=2e-4, atol_scale=2e-4)
    close(F.cpu(sink.views[id(layer.bias)]), db1 + db2, name="db in the bucket", rtol=2e-4, atol_scale=2e-4)
    close(F.cpu(g["layers"][0]["weight"]), dW1 + dW2, name="dW in the tree", rtol=2e-4, atol_scale=2e-4)
    assert all(sink.launched)


def test_multiheadattention_bias_dropout_and_loss_on_the_weights(F):
    """test/layers/attention.jl:45-61: an additive bias that masks gives the causal zero pattern; a loss that uses the
    returned attention weights differentiates; dropout on the weights is active under `withgradient` only."""
    rng = np.random.default_rng(9)
    E, S, B, H = 32, 12, 2, 4
    Ws = [O.glorot_uniform(rng, E, E) for _ in range(4)]
    x = rng.normal(size=(E, S, B)).astype(np.float32)
    mha, xg = F.MultiHeadAttention(*Ws, nheads=H), F.gpu(x)
    bias = np.where(O.make_causal_mask(S), 0.0, -1e9).astype(np.float32)           # used as a mask
    y, alpha = mha(xg, bias=bias)
    a = F.cpu(alpha.materialize())
    assert (a[1, 0, :, :] == 0).all() and np.allclose(a[:, :, 0, 0], np.triu(a[:, :, 0, 0]))
    W64 = [w.astype(np.float64) for w in Ws]
    yref, aref = O.mha_fwd(*W64, x.astype(np.float64), nheads=H, mask=O.make_causal_mask(S))
    close(F.cpu(y), yref)
    close(a, aref, atol_scale=1e-5)

    def loss(m):                                                                      # sum(abs2, y) + sum(abs2, alpha)
        yy, al = m(xg, mask=F.make_causal_mask())
        return F.add(F.sum_abs2(yy), F.sum_abs2(al.materialize()))
    val, (g,) = F.withgradient(loss, mha)
    close(val, (yref ** 2).sum() + (aref ** 2).sum())
    x64 = x.astype(np.float64)
    qq, kk, vv = (O.dense_fwd(w, None, x64) for w in W64[:3])
    xa, _ = O.dot_product_attention(qq, kk, vv, None, H, O.make_causal_mask(S))
    dWo, _, dxa = O.dense_bwd(W64[3], None, xa, 2 * yref)
    dq, dk, dv = O.dot_product_attention_bwd(qq, kk, vv, dxa, None, H, O.make_causal_mask(S), dalpha=2 * aref)
    close(F.cpu(g["q_proj"]["weight"]), O.dense_bwd(W64[0], None, x64, dq)[0], name="dWq", rtol=2e-4, atol_scale=2e-4)
    close(F.cpu(g["k_proj"]["weight"]), O.dense_bwd(W64[1], None, x64, dk)[0], name="dWk", rtol=2e-4, atol_scale=2e-4)
    close(F.cpu(g["out_proj"]["weight"]), dWo, name="dWo", rtol=2e-4, atol_scale=2e-4)
    # dropout on the weights: inactive at inference, active (and different from call to call) in a gradient call
    md = F.MultiHeadAttention(*Ws, nheads=H, dropout_prob=0.5)
    y0 = F.cpu(md(xg)[0])
    close(y0, O.mha_fwd(*W64, x64, nheads=H)[0])
    F.trainmode(md)
    y1, y2 = F.cpu(md(xg)[0]), F.cpu(md(xg)[0])
    assert np.abs(y1 - y0).max() > 1e-3 and np.abs(y1 - y2).max() > 1e-3
    _, al = md(xg)
    assert 0.3 < (F.cpu(al.materialize()) == 0).mean() < 0.7
