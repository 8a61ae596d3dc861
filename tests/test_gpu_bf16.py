"""GPU parity of the BFloat16 path (Flux.bf16): bf16-storage matmul and Dense forward / backward on the tensor cores
against the float64 oracle evaluated on the SAME bf16-rounded inputs; tolerance 2e-2 (a bf16 ulp is 2^-8 = 3.9e-3)."""
import ctypes as C

import numpy as np
import pytest
import torch

import flux_oracle as O
from util import P, stream

pytestmark = pytest.mark.gpu
ACT = {"identity": 0, "relu": 1, "tanh": 2, "sigmoid": 3, "gelu_tanh": 4, "gelu_erf": 5}
TOL = 2e-2


@pytest.fixture(scope="module")
def fb():
    from fluxb200 import lib
    h = C.c_void_p()
    lib.call("fb_ctx_create", 0, C.byref(h))

    class FB:
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


def bf(a):
    """Julia-shaped float array -> (flat CUDA bf16 tensor in column-major order, the rounded values as float64)."""
    t = torch.from_numpy(np.ascontiguousarray(np.asarray(a, np.float32).reshape(-1, order="F"))).cuda().to(torch.bfloat16)
    return t, t.float().cpu().numpy().astype(np.float64).reshape(np.shape(a), order="F")


def back(t, shape):
    return t.float().cpu().numpy().astype(np.float64).reshape(shape, order="F")


def bempty(*shape):
    return torch.empty(int(np.prod(shape)), dtype=torch.bfloat16, device="cuda")


def close(got, ref, name="", tol=TOL):
    scale = float(np.max(np.abs(ref)))
    np.testing.assert_allclose(got, ref, rtol=tol, atol=tol * max(scale, 1e-30), err_msg=name)


@pytest.mark.parametrize("ta,tb", [(0, 0), (1, 0), (0, 1), (1, 1)])
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (256, 384, 192), (200, 136, 104), (512, 768, 1000), (1024, 520, 72), (8, 16, 24)])
def test_gemm_bf16_all_layouts(fb, ta, tb, m, n, k):
    """Both tile variants (one CTA 128 x 128, CTA pair 256 x 256), the four operand layouts, ragged edges, 2-d and 3-d
    tensor maps, bf16 and fp32 results, accumulate."""
    rng = np.random.default_rng(m * 7 + n * 3 + k + ta * 2 + tb)
    tA, A = bf(rng.normal(size=(k, m) if ta else (m, k)))
    tB, B = bf(rng.normal(size=(n, k) if tb else (k, n)))
    ref = (A.T if ta else A) @ (B.T if tb else B)
    tC = bempty(m, n)
    fb.call("fb_gemm_bf16", ta, tb, m, n, k, P(tA), A.shape[0], P(tB), B.shape[0], P(tC), m, 0, 0)
    close(back(tC, (m, n)), ref, name=f"bf16 gemm ta={ta} tb={tb}")
    tF = torch.empty(m * n, dtype=torch.float32, device="cuda")
    fb.call("fb_gemm_bf16", ta, tb, m, n, k, P(tA), A.shape[0], P(tB), B.shape[0], P(tF), m, 0, 1)
    # fp32 output: only the inputs are rounded, the result is exact up to accumulation order
    np.testing.assert_allclose(back(tF, (m, n)), ref, rtol=1e-4, atol=1e-4 * np.abs(ref).max(), err_msg="fp32 result")
    fb.call("fb_gemm_bf16", ta, tb, m, n, k, P(tA), A.shape[0], P(tB), B.shape[0], P(tF), m, 1, 1)
    np.testing.assert_allclose(back(tF, (m, n)), 2 * ref, rtol=1e-4, atol=2e-4 * np.abs(ref).max(), err_msg="accumulate")


def test_gemm_bf16_several_waves_of_pair_tiles(fb):
    """2048 x 4096 x 512: 128 two-CTA tiles on 74 SM pairs (the persistent loop, both accumulator buffers in turn)."""
    rng = np.random.default_rng(1)
    m, n, k = 4096, 2048, 512
    tA, A = bf(rng.normal(size=(m, k)))
    tB, B = bf(rng.normal(size=(k, n)))
    tC = bempty(m, n)
    fb.call("fb_gemm_bf16", 0, 0, m, n, k, P(tA), m, P(tB), k, P(tC), m, 0, 0)
    close(back(tC, (m, n)), A @ B)


def test_gemm_bf16_rejects_unaligned_shapes(fb):
    t = bempty(64)
    st, msg = fb.status("fb_gemm_bf16", 0, 0, 6, 6, 6, P(t), 6, P(t), 6, P(t), 6, 0, 0)
    assert st == -7 and "multiples of 8" in msg
    st, msg = fb.status("fb_gemm_bf16", 0, 0, 8, 8, 8, None, 8, P(t), 8, P(t), 8, 0, 0)
    assert st == -1


@pytest.mark.parametrize("act", ["identity", "relu", "gelu_tanh", "tanh"])
@pytest.mark.parametrize("out_dim,in_dim,n", [(128, 64, 256), (512, 784 + 0, 1024), (1000, 256, 96), (1024, 1024, 2048)])
def test_dense_bf16_fwd_bwd(fb, act, out_dim, in_dim, n):
    if act == "tanh" and (out_dim, in_dim, n) != (128, 64, 256):
        pytest.skip("remaining activations are covered on one shape")
    rng = np.random.default_rng(out_dim + in_dim + n)
    tW, W = bf(O.glorot_uniform(rng, out_dim, in_dim))
    tb, b = bf(rng.normal(size=out_dim) * 0.1)
    tx, x = bf(rng.normal(size=(in_dim, n)))
    tdy, dy = bf(rng.normal(size=(out_dim, n)))
    y, z, delta = bempty(out_dim, n), bempty(out_dim, n), bempty(out_dim, n)
    dW, db, dx = bempty(out_dim, in_dim), bempty(out_dim), bempty(in_dim, n)
    fb.call("fb_dense_fwd_bf16", ACT[act], P(tW), P(tb), P(tx), P(y), P(z), out_dim, in_dim, n)
    yref, zref = O.dense_fwd(W, b, x, act, return_preact=True)
    close(back(z, (out_dim, n)), zref, name="z")
    close(back(y, (out_dim, n)), yref, name="y")
    fb.call("fb_dense_bwd_bf16", ACT[act], P(tW), P(tx), P(y), P(z), P(tdy), P(delta), P(dW), P(db), P(dx), out_dim, in_dim, n)
    # the device takes act' at the bf16-rounded pre-activation (gelu) or output (relu / tanh) it stored
    zq, yq = back(z, (out_dim, n)), back(y, (out_dim, n))
    if act in ("gelu_tanh",):
        d = dy * O.act_grad(act, zq)
    elif act == "relu":
        d = dy * (yq > 0)
    elif act == "tanh":
        d = dy * (1 - yq * yq)
    else:
        d = dy
    close(back(dW, (out_dim, in_dim)), d @ x.T, name="dW")
    close(back(db, (out_dim,)), d.sum(1), name="db")
    close(back(dx, (in_dim, n)), W.T @ d, name="dx")


# ------------------------------------------------------------------- host mirror: Flux.bf16(model) ---
def test_bf16_multiheadattention_forward_and_gradients():
    """bf16(MultiHeadAttention) (the bf16 variant of the attention benchmark configuration): projections with
    BFloat16 storage on the bf16 GEMM, attention core in Float32 on the converted activations; outputs and weight
    gradients within 2e-2 of the float64 oracle evaluated on the same rounded parameters and input."""
    import fluxb200 as F
    rng = np.random.default_rng(5)
    E, S, B, H = 128, 96, 2, 2
    Ws = [O.glorot_uniform(rng, E, E) for _ in range(4)]
    x = rng.normal(size=(E, S, B)).astype(np.float32)
    mha = F.bf16(F.MultiHeadAttention(*[w.copy() for w in Ws], nheads=H))
    assert mha.q_proj.weight.t.dtype == torch.bfloat16 and mha.q_proj.weight.t.element_size() == 2
    xb = F.bf16(F.gpu(x))
    y, _ = mha(xb, mask=F.make_causal_mask())
    assert y.t.dtype == torch.bfloat16
    Wr = [O.bf16_round(w).astype(np.float64) for w in Ws]
    xr = O.bf16_round(x).astype(np.float64)
    mask = O.make_causal_mask(S)
    yref, _ = O.mha_fwd(*Wr, xr, nheads=H, mask=mask)
    close(F.cpu(y), yref, name="y")
    val, (g,) = F.withgradient(lambda m: F.sum_abs2(m(xb, mask=F.make_causal_mask())[0]), mha)
    dWq, dWk, dWv, dWo, _ = O.mha_bwd(*Wr, xr, O.sum_abs2_bwd(yref), nheads=H, mask=mask)
    for name, ref in (("q_proj", dWq), ("k_proj", dWk), ("v_proj", dWv), ("out_proj", dWo)):
        got = g[name]["weight"]
        assert got.t.dtype == torch.bfloat16
        # the intermediate activations are rounded to bf16 between the stages: a few ulps accumulate
        close(F.cpu(got), ref, name=f"d{name}", tol=4e-2)
    assert F.context().device_error() == 0


def test_bf16_model_trains_through_float32_master_weights():
    """Adam on a bf16 model: the step (eta = 1e-3 times a normalised gradient) is far below a bf16 ulp of most weights;
    the Float32 master copy keeps it, the bf16 parameter is the master rounded (bit-exact), and the loss goes down."""
    import fluxb200 as F
    rng = np.random.default_rng(6)
    model = F.bf16(F.Chain(F.Dense(O.glorot_uniform(rng, 64, 32), True, "relu"), F.Dense(O.glorot_uniform(rng, 8, 64))))
    x = F.bf16(F.gpu(rng.normal(size=(32, 48)).astype(np.float32)))
    y = F.onehotbatch(rng.integers(1, 9, size=48), 8)
    opt = F.setup(F.Adam(1e-3), model)
    loss = lambda m, a, b: F.logitcrossentropy(m(a), b)
    losses = [F.trainstep(loss, model, (x, y), opt) for _ in range(30)]
    assert losses[-1] < losses[0] - 0.05
    for p in F.trainables(model):
        leaf = opt.leaves[id(p)]
        assert leaf.master is not None and p.t.dtype == torch.bfloat16
        master = leaf.master.t.cpu().numpy()
        assert (O.to_bf16_bits(master) == p.t.view(torch.int16).cpu().numpy().view(np.uint16)).all()
    with pytest.raises(F.lib.FluxB200Error):
        F.GraphedTrainStep(loss, model, opt, (x, y))
