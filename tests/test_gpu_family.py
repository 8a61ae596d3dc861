"""GPU parity of the rest of the layer family (GroupNorm / InstanceNorm, Embedding, Dropout, RNNCell, GRUv3Cell),
checkpointing and the device data iterator: through the C ABI / the host mirror against the float64 oracle and the
reference's own known answers (test/layers/normalisation.jl:236-445, test/layers/recurrent.jl, test/layers/basic.jl)."""
import ctypes as C

import numpy as np
import pytest
import torch

import flux_oracle as O
from util import P, close, dempty, dev, host, stream

pytestmark = pytest.mark.gpu

ACT = {"identity": 0, "relu": 1, "tanh": 2, "sigmoid": 3}


@pytest.fixture(scope="module")
def F():
    import fluxb200
    yield fluxb200
    assert fluxb200.context().device_error() == 0


def call(F, name, *a):
    F.lib.call(name, F.context().handle, stream(), *a)


def f64(*arrs):
    return [None if a is None else np.asarray(a, dtype=np.float64) for a in arrs]


# --------------------------------------------------------------------------------- GroupNorm ---
def test_groupnorm_frozen_literals(F):
    """test/layers/normalisation.jl:397-432."""
    x = np.arange(1, 25, dtype=np.float32).reshape((3, 4, 2), order="F")
    m = F.GroupNorm(4, 2)
    assert len(F.trainables(m)) == 2 and (F.cpu(m.β) == 0).all() and (F.cpu(m.γ) == 1).all() and m.μ is None and m.σ2 is None
    y = F.cpu(m(F.gpu(x)))
    ref = np.array([[-1.4638476, 0.29276943, -1.4638476, 0.29276943], [-0.87830865, 0.87830853, -0.8783088, 0.8783083],
                    [-0.29276967, 1.4638474, -0.2927699, 1.4638472]])
    np.testing.assert_allclose(y[:, :, 0], ref, atol=1e-5)
    ys = F.cpu(F.GroupNorm(4, 2, "sigmoid")(F.gpu(x)))
    refs = np.array([[0.18787955, 0.57267404, 0.18787955, 0.57267404], [0.2935284, 0.70647156, 0.29352835, 0.70647156],
                     [0.42732593, 0.81212044, 0.42732587, 0.8121204]])
    np.testing.assert_allclose(ys[:, :, 0], refs, atol=1e-5)
    with pytest.raises(F.ArgumentError):
        F.GroupNorm(5, 2)
    # N-d input == permuted 3-d input (:434-439)
    sizes = (2, 4, 1, 2, 3)
    x5 = np.arange(1, np.prod(sizes) + 1, dtype=np.float32).reshape(sizes, order="F")
    gn = F.trainmode(F.GroupNorm(2, 2))
    y3 = np.transpose(x5, (2, 0, 1, 3, 4)).reshape((-1, 2, 3), order="F")
    y3 = F.cpu(gn(F.gpu(y3))).reshape(sizes, order="F")
    np.testing.assert_allclose(F.cpu(gn(F.gpu(x5))), y3, atol=1e-6)


@pytest.mark.parametrize("shape,G", [((3, 4, 2), 2), ((8, 8, 16, 4), 4), ((5, 6, 3), 3), ((16, 8), 2), ((7, 3, 12, 5), 1)])
@pytest.mark.parametrize("act", ["identity", "relu"])
def test_groupnorm_fwd_bwd(F, shape, G, act):
    rng = np.random.default_rng(sum(shape) + G)
    x = (rng.normal(size=shape) * 2 + 0.5).astype(np.float32)
    c, n = shape[-2], shape[-1]
    s = int(np.prod(shape[:-2])) if len(shape) > 2 else 1
    g = (rng.normal(size=c) * 0.5 + 1.2).astype(np.float32)
    b = (rng.normal(size=c) * 0.5).astype(np.float32)
    dy = rng.normal(size=shape).astype(np.float32)
    tx, tg, tb, tdy = dev(x), dev(g), dev(b), dev(dy)
    y, mean, rstd = dempty(*shape), dempty(n * G), dempty(n * G)
    call(F, "fb_groupnorm_fwd", P(tx), P(tg), P(tb), P(y), P(mean), P(rstd), s, c, n, G, 1e-5, ACT[act])
    x64, g64, b64, dy64 = f64(x, g, b, dy)
    close(host(y, shape), O.groupnorm_fwd(x64, g64, b64, G, 1e-5, act), name="y")
    dx, dg, db = dempty(*shape), dempty(c), dempty(c)
    call(F, "fb_groupnorm_bwd", P(tx), P(tg), P(tb), P(mean), P(rstd), P(tdy), P(dx), P(dg), P(db), s, c, n, G, ACT[act])
    dxr, dgr, dbr = O.groupnorm_bwd(x64, g64, b64, dy64, G, 1e-5, act)
    got = host(dx, shape).astype(np.float64)
    if act == "relu":
        unsure = np.abs(O.groupnorm_fwd(x64, g64, b64, G, 1e-5, "identity")) < 1e-5
        got[unsure] = dxr[unsure]
    close(got, dxr, name="dx", rtol=2e-4, atol_scale=2e-4)
    close(host(dg, (c,)), dgr, name="dgamma", rtol=2e-4, atol_scale=2e-4)
    close(host(db, (c,)), dbr, name="dbeta", rtol=2e-4, atol_scale=2e-4)
    # no affine parameters
    call(F, "fb_groupnorm_fwd", P(tx), None, None, P(y), P(mean), P(rstd), s, c, n, G, 1e-5, ACT[act])
    close(host(y, shape), O.groupnorm_fwd(x64, None, None, G, 1e-5, act), name="y without affine")
    st = F.lib.raw().fb_groupnorm_fwd(F.context().handle, stream(), P(tx), None, None, P(y), P(mean), P(rstd), s, c, n, c + 1, 1e-5, 0)
    assert st == -2 and "must divide the number of channels" in F.lib.last_error()


def test_instancenorm_known_answers(F):
    """test/layers/normalisation.jl:236-300."""
    x = np.arange(1, 13, dtype=np.float32).reshape((3, 2, 2), order="F")
    m = F.InstanceNorm(2, affine=True, track_stats=True)
    assert len(F.trainables(m)) == 2
    xg = F.gpu(x)
    F.withgradient(lambda mm: F.sum_abs2(mm(xg)), m)            # evalwgrad: a training-mode call
    np.testing.assert_allclose(F.cpu(m.μ), [0.5, 0.8], rtol=1e-6)
    s2 = x.astype(np.float64).var(axis=0)
    np.testing.assert_allclose(F.cpu(m.σ2), 0.1 * 1.5 * s2.mean(axis=1) + 0.9, rtol=1e-5)
    y = F.cpu(m(xg))                                             # inference with the tracked statistics
    mu, var = F.cpu(m.μ).reshape(1, 2, 1), F.cpu(m.σ2).reshape(1, 2, 1)
    np.testing.assert_allclose(y, (x - mu) / np.sqrt(var + 1e-5), atol=1e-5)
    # no tracked statistics, sigmoid (:290-312)
    m2 = F.InstanceNorm(2, "sigmoid")
    assert len(F.trainables(m2)) == 0
    x64 = x.astype(np.float64)
    ref = 1 / (1 + np.exp(-(x64 - x64.mean(axis=0)) / np.sqrt(x64.var(axis=0) + 1e-5)))
    np.testing.assert_allclose(F.cpu(m2(xg)), ref, atol=1e-6)
    # InstanceNorm == GroupNorm with one channel per group (:441-445) == BatchNorm with channel and batch squashed (:348-352)
    sizes = (2, 2, 3, 4, 5)
    x5 = np.arange(1, np.prod(sizes) + 1, dtype=np.float32).reshape(sizes, order="F")
    a = F.cpu(F.trainmode(F.InstanceNorm(4, affine=True))(F.gpu(x5)))
    b = F.cpu(F.trainmode(F.GroupNorm(4, 4))(F.gpu(x5)))
    np.testing.assert_allclose(a, b, atol=1e-6)
    sizes6 = (5, 5, 3, 4, 2, 6)
    x6 = np.arange(1, np.prod(sizes6) + 1, dtype=np.float32).reshape(sizes6, order="F")
    i6 = F.cpu(F.trainmode(F.InstanceNorm(2, affine=True))(F.gpu(x6)))
    b6 = F.cpu(F.trainmode(F.BatchNorm(12))(F.gpu(x6.reshape((5, 5, 3, 4, 12, 1), order="F")))).reshape(sizes6, order="F")
    np.testing.assert_allclose(i6, b6, atol=2e-5)


# --------------------------------------------------------------------------------- Embedding ---
def test_embedding_layer(F):
    """Doctest values of src/layers/basic.jl:752-776 and the gradient (scatter-add with repeated indices)."""
    W = np.zeros((4, 26), np.float32)
    W[np.arange(4), np.arange(4)] = 22.0
    emb = F.Embedding(W)
    np.testing.assert_array_equal(F.cpu(emb(2)), [0, 22, 0, 0])
    idx = np.array([3, 1, 20, 14, 4, 15, 7])
    np.testing.assert_array_equal(F.cpu(emb(idx)), O.embedding_fwd(W, idx))
    assert emb(np.ones((10, 1, 12), int)).size == (4, 10, 1, 12)
    with pytest.raises(IndexError):
        emb(np.array([27]))
    with pytest.raises(F.ArgumentError):
        F.Embedding((5, 2), padding_idx=6)
    e2 = F.Embedding((5, 2), padding_idx=1)
    assert e2.weight.size == (2, 5) and (F.cpu(e2(1)) == 0).all() and (F.cpu(e2.weight)[:, 0] == 0).all()
    rng = np.random.default_rng(0)
    Wr = rng.normal(size=(48, 100)).astype(np.float32)
    idx = rng.integers(1, 101, size=(33, 7))
    idx[0, :3] = 5
    er = F.Embedding(Wr, padding_idx=5)
    idg = F.gpu(idx.astype(np.int32))
    val, (g,) = F.withgradient(lambda m: F.sum_abs2(m(idg)), er)
    y = O.embedding_fwd(Wr.astype(np.float64), idx, padding_idx=5)
    close(val, (y * y).sum())
    close(F.cpu(g["weight"]), O.embedding_bwd(Wr.astype(np.float64), idx, 2 * y, padding_idx=5), name="dW")
    assert (F.cpu(g["weight"])[:, 4] == 0).all()


# ----------------------------------------------------------------------------------- Dropout ---
def test_dropout_mask_is_bit_exact_and_layer_semantics(F):
    """The mask is integer work (a counter-based generator): bit-exact against the oracle's restatement; scaling by
    1 / (1 - p); identity in test mode; the backward pass applies the same mask (test/layers/normalisation.jl:4-50)."""
    n = 100003
    x = np.random.default_rng(1).normal(size=n).astype(np.float32)
    tx, ty = dev(x), dempty(n)
    for p, seed, off in [(0.3, 7, 0), (0.5, 2 ** 40 + 3, 11), (0.0, 1, 0), (1.0, 1, 0)]:
        call(F, "fb_dropout", P(tx), P(ty), n, p, seed, off)
        keep = O.dropout_mask(n, p, seed, off)
        got = host(ty, (n,))
        assert ((got != 0) == (keep & (x != 0))).all()
        if p < 1:
            np.testing.assert_allclose(got, O.dropout_fwd(x, p, keep), rtol=1e-6)
    st = F.lib.raw().fb_dropout(F.context().handle, stream(), P(tx), P(ty), n, 1.5, 0, 0)
    assert st == -1 and "0 <= p <= 1" in F.lib.last_error()
    d = F.Dropout(0.4, seed=5)
    xg = F.gpu(x)
    assert d(xg) is xg                                   # inactive outside a gradient call
    assert F.testmode(F.Dropout(0.4))(xg) is xg
    dd = F.trainmode(F.Dropout(0.4, seed=5))
    y1, y2 = F.cpu(dd(xg)), F.cpu(dd(xg))
    assert (y1 != y2).any()                              # successive calls draw different masks
    assert abs((y1 != 0).mean() - 0.6) < 0.01
    with pytest.raises(F.ArgumentError):
        F.Dropout(1.2)
    # gradient: Chain(Dense, Dropout) - the weight gradient sees the same mask as the forward pass
    rng = np.random.default_rng(3)
    W, xin = O.glorot_uniform(rng, 16, 8), rng.normal(size=(8, 5)).astype(np.float32)
    drop = F.Dropout(0.5, seed=9)
    model = F.Chain(F.Dense(W, False), drop)
    xing = F.gpu(xin)
    val, (g,) = F.withgradient(lambda m: F.sum_abs2(m(xing)), model)
    keep = O.dropout_mask(16 * 5, 0.5, 9, 0).reshape((16, 5), order="F")
    h = W.astype(np.float64) @ xin
    yref = O.dropout_fwd(h, 0.5, keep)
    close(val, (yref * yref).sum())
    close(F.cpu(g["layers"][0]["weight"]), (2 * yref * keep / 0.5) @ xin.T.astype(np.float64), name="dW through dropout")


# ------------------------------------------------------------------------- RNNCell / GRUv3Cell ---
@pytest.mark.parametrize("I,H,T,B", [(3, 4, 5, 2), (16, 32, 7, 3), (64, 128, 12, 70), (20, 130, 4, 5)])
@pytest.mark.parametrize("act,bias,state", [("tanh", True, False), ("relu", False, True)])
def test_rnn_fwd_bwd(F, I, H, T, B, act, bias, state):
    rng = np.random.default_rng(I + H + T + B)
    Wi, Wh = O.glorot_uniform(rng, H, I), O.glorot_uniform(rng, H, H)
    b = (rng.normal(size=H) * 0.1).astype(np.float32) if bias else None
    x = rng.normal(size=(I, T, B)).astype(np.float32)
    h0 = rng.normal(size=(H, B)).astype(np.float32) if state else None
    tWi, tWh, tb, tx, th0 = dev(Wi), dev(Wh), dev(b) if bias else None, dev(x), dev(h0) if state else None
    out, hT = dempty(H, T, B), dempty(H, B)
    call(F, "fb_rnn_fwd", ACT[act], P(tWi), P(tWh), P(tb), P(tx), P(th0), P(out), P(hT), I, H, T, B)
    Wi64, Wh64, b64, x64, h064 = f64(Wi, Wh, b, x, h0)
    oref, href = O.rnn_scan_fwd(Wi64, Wh64, b64, x64, act, h064)
    close(host(out, (H, T, B)), oref, name="out")
    close(host(hT, (H, B)), href, name="hT")
    dout = O.sum_abs2_bwd(oref)
    tdout = dev(dout, np.float32)
    cache = torch.empty(F.lib.raw().fb_rnn_cache_bytes(I, H, T, B) // 4, dtype=torch.float32, device="cuda")
    dWi, dWh, db, dx = dempty(H, I), dempty(H, H), dempty(H), dempty(I, T, B)
    call(F, "fb_rnn_bwd", ACT[act], P(tWi), P(tWh), P(tx), P(th0), P(out), P(cache), P(tdout), None, P(dWi), P(dWh),
         P(db) if bias else None, P(dx), I, H, T, B)
    rWi, rWh, rb, rx = O.rnn_scan_bwd(Wi64, Wh64, b64, x64, dout, act, h064)
    if act == "relu":
        pytest.skip("relu masks of pre-activations within rounding of 0 make the BPTT comparison ill-posed; forward checked")
    close(host(dWi, (H, I)), rWi, name="dWi", rtol=2e-4, atol_scale=2e-4)
    close(host(dWh, (H, H)), rWh, name="dWh", rtol=2e-4, atol_scale=2e-4)
    close(host(dx, (I, T, B)), rx, name="dx", rtol=2e-4, atol_scale=2e-4)
    if bias:
        close(host(db, (H,)), rb, name="db", rtol=2e-4, atol_scale=2e-4)


@pytest.mark.parametrize("I,H,T,B", [(3, 4, 5, 2), (16, 32, 7, 3), (64, 128, 12, 70), (20, 130, 4, 5)])
@pytest.mark.parametrize("bias", [True, False])
def test_gruv3_fwd_bwd(F, I, H, T, B, bias):
    rng = np.random.default_rng(I + H + T + B + 2)
    Wi, Wh, Whh = O.glorot_uniform(rng, 3 * H, I), O.glorot_uniform(rng, 3 * H, H), O.glorot_uniform(rng, H, H)
    b = (rng.normal(size=3 * H) * 0.1).astype(np.float32) if bias else None
    x = rng.normal(size=(I, T, B)).astype(np.float32)
    tWi, tWh, tWhh, tb, tx = dev(Wi), dev(Wh), dev(Whh), dev(b) if bias else None, dev(x)
    cache = torch.empty(F.lib.raw().fb_gruv3_cache_bytes(I, H, T, B) // 4, dtype=torch.float32, device="cuda")
    out, hT = dempty(H, T, B), dempty(H, B)
    call(F, "fb_gruv3_fwd", P(tWi), P(tWh), P(tb), P(tWhh), P(tx), None, P(out), P(hT), P(cache), I, H, T, B)
    Wi64, Wh64, b64, Whh64, x64 = f64(Wi, Wh, b, Whh, x)
    oref, href = O.gruv3_scan_fwd(Wi64, Wh64, b64, Whh64, x64)
    close(host(out, (H, T, B)), oref, name="out")
    close(host(hT, (H, B)), href, name="hT")
    out2 = dempty(H, T, B)
    call(F, "fb_gruv3_fwd", P(tWi), P(tWh), P(tb), P(tWhh), P(tx), None, P(out2), None, None, I, H, T, B)
    assert torch.equal(out, out2)
    dout = O.sum_abs2_bwd(oref)
    tdout = dev(dout, np.float32)
    dWi, dWh, db, dWhh, dx = dempty(3 * H, I), dempty(3 * H, H), dempty(3 * H), dempty(H, H), dempty(I, T, B)
    call(F, "fb_gruv3_bwd", P(tWi), P(tWh), P(tWhh), P(tx), None, P(out), P(cache), P(tdout), None, P(dWi), P(dWh),
         P(db) if bias else None, P(dWhh), P(dx), I, H, T, B)
    rWi, rWh, rb, rWhh, rx = O.gruv3_scan_bwd(Wi64, Wh64, b64, Whh64, x64, dout)
    close(host(dWi, (3 * H, I)), rWi, name="dWi", rtol=2e-4, atol_scale=2e-4)
    close(host(dWh, (3 * H, H)), rWh, name="dWh", rtol=2e-4, atol_scale=2e-4)
    close(host(dWhh, (H, H)), rWhh, name="dWh_h", rtol=2e-4, atol_scale=2e-4)
    close(host(dx, (I, T, B)), rx, name="dx", rtol=2e-4, atol_scale=2e-4)
    if bias:
        close(host(db, (3 * H,)), rb, name="db", rtol=2e-4, atol_scale=2e-4)


def test_recurrence_wrappers_of_the_family(F):
    """test/layers/recurrent.jl:24-70, 270-330: zero initial state, state shapes, Recurrence(cell) == RNN(...)."""
    F.seed(4)
    x = F.gpu(np.random.default_rng(0).normal(size=(3, 4, 2)).astype(np.float32))
    cell = F.RNNCell((3, 5))
    assert cell.Wi.size == (5, 3) and cell.Wh.size == (5, 5) and cell.bias.size == (5,) and cell.σ == "tanh"
    y = F.Recurrence(cell)(x)
    assert y.size == (5, 4, 2)
    y2, h = F.Recurrence(cell, return_state=True)(x, cell.initialstates())
    assert h.size == (5, 2) and torch.equal(y.t, y2.t)
    np.testing.assert_allclose(F.cpu(h), F.cpu(y)[:, -1, :], rtol=0, atol=0)
    g3 = F.GRUv3Cell((3, 5))
    assert g3.Wi.size == (15, 3) and g3.Wh.size == (15, 5) and g3.Wh_h.size == (5, 5)
    m = F.GRUv3((3, 5))
    assert len(F.trainables(m)) == 4 and m(x).size == (5, 4, 2)
    val, (g,) = F.withgradient(lambda mm: F.sum_abs2(mm(x)), m)
    assert set(g["cell"]) == {"Wi", "Wh", "b", "Wh_h̃"} and g["cell"]["Wh_h̃"].size == (5, 5)
    with pytest.raises(F.lib.FluxB200Error):
        F.RNNCell((3, 5), sigma="gelu")


# ------------------------------------------------------------------------ checkpoint round trip ---
def test_state_loadmodel_and_checkpoint_round_trip(F, tmp_path):
    """src/loading.jl:90-189 and its doctests; test/loading.jl: structure / size mismatches, false <-> zero bias."""
    F.seed(0)
    m1 = F.Chain(F.Dense((1, 2), "tanh", init=lambda o, i: np.ones((o, i), np.float32)), F.Dense((2, 1), init=lambda o, i: np.ones((o, i), np.float32)))
    s = F.state(m1)
    assert set(s) == {"layers"} and set(s["layers"][0]) == {"weight", "bias", "σ"}
    assert (s["layers"][0]["weight"] == 1).all() and (s["layers"][0]["bias"] == 0).all() and s["layers"][0]["σ"] == "tanh"
    m2 = F.Chain(F.Dense((1, 2), "tanh"), F.Dense((2, 1), bias=False))
    F.loadmodel(m2, s)                                     # zero bias into bias=false is allowed
    assert (F.cpu(m2.layers[0].weight) == 1).all() and m2.layers[1].bias is False
    bn = F.BatchNorm(3)
    sb = F.state(bn)
    assert set(sb) >= {"β", "γ", "μ", "σ2", "ε", "momentum", "affine", "track_stats", "active", "chs"} and sb["active"] is None
    with pytest.raises(F.DimensionMismatch):
        F.loadmodel(F.Chain(F.Dense((1, 3)), F.Dense((3, 1))), s)
    with pytest.raises(F.ArgumentError):
        F.loadmodel(F.Chain(F.Dense((1, 2))), s)
    nz = F.Chain(F.Dense(np.ones((2, 1), np.float32), np.ones(2, np.float32)))
    with pytest.raises(ValueError):
        F.loadmodel(F.Chain(F.Dense((1, 2), bias=False)), nz)   # non-zero bias cannot go into an inactive one
    # model + optimiser round trip through one file, then training continues identically
    rng = np.random.default_rng(1)
    mk = lambda: F.Chain(F.LayerNorm(8), F.Dense(O.glorot_uniform(np.random.default_rng(2), 6, 8), True, "gelu"), F.BatchNorm(6),
                         F.Dense(O.glorot_uniform(np.random.default_rng(3), 4, 6)))
    a = mk()
    x, lab = F.gpu(rng.normal(size=(8, 16)).astype(np.float32)), F.onehotbatch(rng.integers(1, 5, size=16), 4)
    loss = lambda m, xx, yy: F.logitcrossentropy(m(xx), yy)
    oa = F.setup(F.Adam(1e-2), a)
    for _ in range(3):
        F.trainstep(loss, a, (x, lab), oa)
    path = str(tmp_path / "ckpt.npz")
    F.save_checkpoint(path, a, oa)
    b = mk()
    ob = F.setup(F.Adam(1e-2), b)
    F.load_checkpoint(path, b, ob)
    for pa, pb in zip(F.trainables(a), F.trainables(b)):
        assert torch.equal(pa.t, pb.t)
    assert torch.equal(a.layers[2].μ.t, b.layers[2].μ.t) and torch.equal(a.layers[2].σ2.t, b.layers[2].σ2.t)   # non-trainable state
    la = [F.trainstep(loss, a, (x, lab), oa) for _ in range(2)]
    lb = [F.trainstep(loss, b, (x, lab), ob) for _ in range(2)]
    assert la == lb
    for pa, pb in zip(F.trainables(a), F.trainables(b)):
        assert torch.equal(pa.t, pb.t)


# ----------------------------------------------------------------------------- device iterator ---
def test_dataloader_device_iterator(F):
    """test/ext_cuda/cuda.jl:177-204: iterating `DataLoader |> gpu` yields device arrays with the same contents."""
    X = np.random.default_rng(0).normal(size=(5, 3, 22)).astype(np.float32)
    Y = np.arange(22, dtype=np.int64)
    dl = F.DataLoader((X, Y), batchsize=4)
    assert len(dl) == 6
    seen = 0
    for (xb, yb), (xh, yh) in zip(F.DeviceIterator(dl), dl):
        assert isinstance(xb, F.B200Array) and xb.size == xh.shape and yb.size == yh.shape
        np.testing.assert_array_equal(F.cpu(xb), xh)
        np.testing.assert_array_equal(F.cpu(yb), yh)
        seen += xh.shape[-1]
    assert seen == 22
    assert len(F.DataLoader(X, batchsize=4, partial=False)) == 5
    sh = F.DataLoader(X, batchsize=22, shuffle=True, rng=np.random.default_rng(1))
    (b,) = list(F.DeviceIterator(sh))
    assert b.size == (5, 3, 22) and np.allclose(np.sort(F.cpu(b).sum(axis=(0, 1))), np.sort(X.sum(axis=(0, 1))), atol=1e-5)
