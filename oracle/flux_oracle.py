"""CPU restatement of the forward + backward hot path of Flux.jl's own layers.

TEST INFRASTRUCTURE ONLY.  This module is the checker that the CUDA library is
compared against; nothing in the shipped package imports it.  It is a numpy
restatement (dtype-generic: float64 for parity checks, float32 for the timed
CPU baseline) that follows the reference sources function by function.  Every
function cites the reference file:line it restates.

Array convention: every array has the *Julia* shape of the reference (e.g. a
Dense weight is ``(out, in)``, a batch of inputs is ``(in, N)``, a sequence is
``(features, seq_len, batch)``, images are WHCN).  Memory order is irrelevant
here; the device library's layout is handled by the host package.

Parity pin status
-----------------
Pinned against the reference's own known-answer tests (see tests/golden and
tests/test_oracle_golden.py): Dense ones-init answers, BatchNorm forward /
running statistics / inference values, logitcrossentropy values, bf16
rounding, nfan / glorot variance, causal-mask zero pattern, the
DistributedDataContainer shard sizes and the allreduce closed forms.

"parity unpinned" (no number in the reference fixes them; the arithmetic lives
in NNlib / Optimisers / Zygote, which are not vendored in the reference and
cannot run here because no Julia toolchain exists on this machine):
LayerNorm numerics (restated as biased variance with eps added to the
variance, NEWS.md:17), the gelu flavour (tanh approximation by default, erf
as a switch), sigmoid_fast / tanh_fast (restated exactly), the attention head
split / scale / mask fill, Adam's epsilon placement, and LSTM / GRU outputs.
Those backward passes are verified here by float64 central finite differences
(the method of the reference's test/test_module.jl:111-182).
"""
from __future__ import annotations

import math
import numpy as np

# --------------------------------------------------------------------------
# activations (NNlib, called from src/layers/basic.jl:199 via bias_act!)
# --------------------------------------------------------------------------
ACTS = ("identity", "relu", "tanh", "sigmoid", "gelu_tanh", "gelu_erf")

_SQRT_2_OVER_PI = math.sqrt(2.0 / math.pi)


def _erf(x):
    # vectorised erf without scipy dependency issues: use math.erf elementwise
    from scipy.special import erf  # scipy is present in the image
    return erf(x)


def act(name: str, z):
    """sigma.(z) for the activation names the library's enum carries."""
    if name == "identity":
        return z
    if name == "relu":
        return np.maximum(z, 0)
    if name == "tanh":
        return np.tanh(z)
    if name == "sigmoid":
        return 1.0 / (1.0 + np.exp(-z))
    if name == "gelu_tanh":
        # NNlib.gelu (tanh approximation): 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))
        return 0.5 * z * (1.0 + np.tanh(_SQRT_2_OVER_PI * (z + 0.044715 * z ** 3)))
    if name == "gelu_erf":
        return 0.5 * z * (1.0 + _erf(z / math.sqrt(2.0)))
    raise ValueError(name)


def act_grad(name: str, z):
    """d sigma / dz evaluated at the pre-activation z."""
    if name == "identity":
        return np.ones_like(z)
    if name == "relu":
        return (z > 0).astype(z.dtype)
    if name == "tanh":
        t = np.tanh(z)
        return 1.0 - t * t
    if name == "sigmoid":
        s = 1.0 / (1.0 + np.exp(-z))
        return s * (1.0 - s)
    if name == "gelu_tanh":
        u = _SQRT_2_OVER_PI * (z + 0.044715 * z ** 3)
        t = np.tanh(u)
        du = _SQRT_2_OVER_PI * (1.0 + 3 * 0.044715 * z * z)
        return 0.5 * (1.0 + t) + 0.5 * z * (1.0 - t * t) * du
    if name == "gelu_erf":
        pdf = np.exp(-0.5 * z * z) / math.sqrt(2.0 * math.pi)
        return 0.5 * (1.0 + _erf(z / math.sqrt(2.0))) + z * pdf
    raise ValueError(name)


# --------------------------------------------------------------------------
# initialisers (src/utils.jl:27-31, 81-86, 537-543)
# --------------------------------------------------------------------------
def nfan(*dims):
    """src/utils.jl:27-31: (fan_in, fan_out)."""
    if len(dims) == 1 and isinstance(dims[0], tuple):
        dims = dims[0]
    if len(dims) == 0:
        return 1, 1
    if len(dims) == 1:
        return 1, dims[0]
    if len(dims) == 2:
        return dims[1], dims[0]
    rf = int(np.prod(dims[:-2]))
    return rf * dims[-2], rf * dims[-1]


def glorot_uniform(rng: np.random.Generator, *dims, gain=1.0):
    """src/utils.jl:81-86: (rand(Float32, dims) - 0.5) * gain * sqrt(24 / (fan_in + fan_out)).

    The Julia RNG stream itself is not reproducible without Julia; the
    distribution is.  Weights are always passed explicitly to the layers.
    """
    scale = np.float32(gain) * np.sqrt(np.float32(24.0) / np.float32(sum(nfan(*dims))))
    return ((rng.random(dims, dtype=np.float32) - np.float32(0.5)) * scale).astype(np.float32)


def to_bf16_bits(x):
    """src/functor.jl:161-166: round-to-nearest-even in the integer domain, NaN -> 0x7fc0."""
    f = np.asarray(x, dtype=np.float32)
    u = f.view(np.uint32).astype(np.uint64)
    bits = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint32) & 0xFFFF
    bits = np.where(np.isnan(f), 0x7FC0, bits)
    return bits.astype(np.uint16)


def bf16_bits_to_f32(bits):
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def bf16_round(x):
    """Float32 value of bf16(x), same rounding as to_bf16_bits."""
    return bf16_bits_to_f32(to_bf16_bits(x)).reshape(np.shape(x))


# --------------------------------------------------------------------------
# Dense (src/layers/basic.jl:196-205) and its reverse
# --------------------------------------------------------------------------
def dense_fwd(W, b, x, sigma="identity", return_preact=False):
    """y = sigma.(W*x .+ b); N-d inputs are flattened to (in, prod(rest)) (basic.jl:202-205).

    b is an array of length out, or None / False for bias=false.
    """
    if x.shape[0] != W.shape[1]:
        # basic.jl:217-223 _size_check -> DimensionMismatch
        raise ValueError(f"DimensionMismatch: layer expects size(input, 1) == {W.shape[1]}, got {x.shape}")
    x2 = x.reshape(x.shape[0], -1)
    z = W @ x2
    if b is not None and b is not False:
        z = z + np.asarray(b).reshape(-1, 1)
    y = act(sigma, z)
    out_shape = (W.shape[0],) + tuple(x.shape[1:])
    if return_preact:
        return y.reshape(out_shape), z.reshape(out_shape)
    return y.reshape(out_shape)


def dense_bwd(W, b, x, dy, sigma="identity"):
    """Reverse of dense_fwd: delta = dy .* sigma'(z); dW = delta x'; db = sum_N delta; dx = W' delta.

    Tangent field names in the reference are (weight, bias, sigma=nothing) (src/gradient.jl:112).
    """
    x2 = x.reshape(x.shape[0], -1)
    z = W @ x2
    has_b = b is not None and b is not False
    if has_b:
        z = z + np.asarray(b).reshape(-1, 1)
    delta = dy.reshape(W.shape[0], -1) * act_grad(sigma, z)
    dW = delta @ x2.T
    db = delta.sum(axis=1) if has_b else None
    dx = (W.T @ delta).reshape(x.shape)
    return dW, db, dx


# --------------------------------------------------------------------------
# LayerNorm (src/layers/normalise.jl:203-210 -> NNlib.normalise; Scale basic.jl:284-287)
# --------------------------------------------------------------------------
def layernorm_fwd(x, gamma, beta, eps=1e-5, sigma="identity", nd=1, return_stats=False):
    """Normalise over the first `nd` dims (biased variance, eps added to the variance),
    then sigma.(gamma .* xhat .+ beta).  gamma/beta None for affine=false."""
    axes = tuple(range(nd))
    mu = x.mean(axis=axes, keepdims=True)
    var = ((x - mu) ** 2).mean(axis=axes, keepdims=True)
    rstd = 1.0 / np.sqrt(var + x.dtype.type(eps))
    xhat = (x - mu) * rstd
    z = xhat
    if gamma is not None:
        gshape = gamma.shape + (1,) * (x.ndim - gamma.ndim)
        z = gamma.reshape(gshape) * xhat + beta.reshape(gshape)
    y = act(sigma, z)
    if return_stats:
        return y, mu, rstd
    return y


def layernorm_bwd(x, gamma, beta, dy, eps=1e-5, sigma="identity", nd=1):
    """dx = rstd (g - mean(g) - xhat mean(g xhat)), g = dz gamma; dgamma = sum dz xhat; dbeta = sum dz."""
    axes = tuple(range(nd))
    mu = x.mean(axis=axes, keepdims=True)
    var = ((x - mu) ** 2).mean(axis=axes, keepdims=True)
    rstd = 1.0 / np.sqrt(var + x.dtype.type(eps))
    xhat = (x - mu) * rstd
    if gamma is not None:
        gshape = gamma.shape + (1,) * (x.ndim - gamma.ndim)
        g_ = gamma.reshape(gshape)
        z = g_ * xhat + beta.reshape(gshape)
    else:
        g_ = 1.0
        z = xhat
    dz = dy * act_grad(sigma, z)
    g = dz * g_
    dx = rstd * (g - g.mean(axis=axes, keepdims=True) - xhat * (g * xhat).mean(axis=axes, keepdims=True))
    if gamma is None:
        return dx, None, None
    red = tuple(range(nd, x.ndim))
    dgamma = (dz * xhat).sum(axis=red)
    dbeta = dz.sum(axis=red)
    return dx, dgamma, dbeta


# --------------------------------------------------------------------------
# BatchNorm (src/layers/normalise.jl:292-304 -> NNlib.batchnorm)
# --------------------------------------------------------------------------
def _bn_axes(x):
    cdim = x.ndim - 2  # channel dim is N-1 (1-based) == ndim-2 (0-based)
    axes = tuple(i for i in range(x.ndim) if i != cdim)
    shp = [1] * x.ndim
    shp[cdim] = x.shape[cdim]
    return cdim, axes, tuple(shp)


def batchnorm_fwd_train(x, gamma, beta, run_mean, run_var, momentum=0.1, eps=1e-5,
                        sigma="identity", track_stats=True):
    """Training-mode BatchNorm.  Returns (y, new_running_mean, new_running_var).

    Per-channel batch mean and *biased* variance over every dim but N-1; running
    stats: mu <- (1-m) mu + m mu_B ; var <- (1-m) var + m var_B * n/(n-1)
    (pinned by test/layers/normalisation.jl:150-156).  n == 1 is an error
    (normalise.jl:295-300).
    """
    cdim, axes, shp = _bn_axes(x)
    n = x.size // x.shape[cdim]
    if n == 1:
        raise ValueError("ArgumentError: BatchNorm expected more than 1 value per channel when training")
    mu = x.mean(axis=axes)
    var = ((x - mu.reshape(shp)) ** 2).mean(axis=axes)
    rstd = 1.0 / np.sqrt(var + x.dtype.type(eps))
    xhat = (x - mu.reshape(shp)) * rstd.reshape(shp)
    z = xhat
    if gamma is not None:
        z = gamma.reshape(shp) * xhat + beta.reshape(shp)
    y = act(sigma, z)
    if track_stats and run_mean is not None:
        m = x.dtype.type(momentum)
        new_mean = (1 - m) * run_mean + m * mu
        new_var = (1 - m) * run_var + m * var * (x.dtype.type(n) / x.dtype.type(n - 1))
    else:
        new_mean, new_var = run_mean, run_var
    return y, new_mean, new_var


def batchnorm_fwd_infer(x, gamma, beta, run_mean, run_var, eps=1e-5, sigma="identity"):
    """Inference-mode BatchNorm: uses the running statistics (normalisation.jl test :158-159)."""
    cdim, axes, shp = _bn_axes(x)
    xhat = (x - run_mean.reshape(shp)) / np.sqrt(run_var.reshape(shp) + x.dtype.type(eps))
    z = xhat
    if gamma is not None:
        z = gamma.reshape(shp) * xhat + beta.reshape(shp)
    return act(sigma, z)


def batchnorm_bwd(x, gamma, beta, dy, eps=1e-5, sigma="identity"):
    """Reverse of the training-mode forward: (dx, dgamma, dbeta)."""
    cdim, axes, shp = _bn_axes(x)
    mu = x.mean(axis=axes)
    var = ((x - mu.reshape(shp)) ** 2).mean(axis=axes)
    rstd = (1.0 / np.sqrt(var + x.dtype.type(eps))).reshape(shp)
    xhat = (x - mu.reshape(shp)) * rstd
    if gamma is not None:
        g_ = gamma.reshape(shp)
        z = g_ * xhat + beta.reshape(shp)
    else:
        g_ = 1.0
        z = xhat
    dz = dy * act_grad(sigma, z)
    dgamma = (dz * xhat).sum(axis=axes)
    dbeta = dz.sum(axis=axes)
    g = dz * g_
    dx = rstd * (g - g.mean(axis=axes, keepdims=True) - xhat * (g * xhat).mean(axis=axes, keepdims=True))
    if gamma is None:
        return dx, None, None
    return dx, dgamma, dbeta


# --------------------------------------------------------------------------
# GroupNorm / InstanceNorm (normalise.jl:388-393, 486-489 -> NNlib.groupnorm / instancenorm)
# --------------------------------------------------------------------------
def _group_view(x, G):
    """x (..., C, N) -> (S, C/G, G, N) with S the product of the leading dims: what NNlib.groupnorm reshapes to."""
    C, N = x.shape[-2], x.shape[-1]
    S = x.size // (C * N)
    # Julia memory order has the first index fastest and channel c = g * (C/G) + k (k fastest): in numpy's C-order
    # view of the Julia-shaped array that is a split of the channel axis into (G, C/G)
    return x.reshape(S, G, C // G, N), S


def groupnorm_fwd(x, gamma, beta, G, eps=1e-5, sigma="identity", return_stats=False):
    """(gn::GroupNorm)(x) (normalise.jl:486-489): per (group, sample) mean and biased variance over the spatial dims
    and the C/G channels of the group, per-channel affine, activation.  Frozen outputs of the reference's test
    (test/layers/normalisation.jl:410, 431) pin the grouping of consecutive channels and the biased variance."""
    C = x.shape[-2]
    if C % G:
        raise ValueError(f"The number of groups ({G}) must divide the number of channels ({C})")
    xv, S = _group_view(x, G)
    mu = xv.mean(axis=(0, 2), keepdims=True)
    var = ((xv - mu) ** 2).mean(axis=(0, 2), keepdims=True)
    rstd = 1.0 / np.sqrt(var + x.dtype.type(eps))
    xhat = ((xv - mu) * rstd).reshape(x.shape)
    z = xhat
    if gamma is not None:
        shp = [1] * x.ndim
        shp[-2] = C
        z = gamma.reshape(shp) * xhat + beta.reshape(shp)
    y = act(sigma, z)
    if return_stats:
        return y, mu.reshape(G, -1), rstd.reshape(G, -1)
    return y


def groupnorm_bwd(x, gamma, beta, dy, G, eps=1e-5, sigma="identity"):
    """Reverse of groupnorm_fwd: (dx, dgamma, dbeta)."""
    C = x.shape[-2]
    xv, S = _group_view(x, G)
    mu = xv.mean(axis=(0, 2), keepdims=True)
    var = ((xv - mu) ** 2).mean(axis=(0, 2), keepdims=True)
    rstd = 1.0 / np.sqrt(var + x.dtype.type(eps))
    xhat = ((xv - mu) * rstd).reshape(x.shape)
    shp = [1] * x.ndim
    shp[-2] = C
    if gamma is not None:
        g_ = gamma.reshape(shp)
        z = g_ * xhat + beta.reshape(shp)
    else:
        g_, z = 1.0, xhat
    dz = dy * act_grad(sigma, z)
    axes = tuple(i for i in range(x.ndim) if i != x.ndim - 2)
    dgamma, dbeta = (dz * xhat).sum(axis=axes), dz.sum(axis=axes)
    g = (dz * g_).reshape(xv.shape)
    xh = xhat.reshape(xv.shape)
    dx = (rstd * (g - g.mean(axis=(0, 2), keepdims=True) - xh * (g * xh).mean(axis=(0, 2), keepdims=True))).reshape(x.shape)
    if gamma is None:
        return dx, None, None
    return dx, dgamma, dbeta


def instancenorm_fwd_train(x, gamma, beta, run_mean, run_var, momentum=0.1, eps=1e-5, sigma="identity", track_stats=False):
    """(l::InstanceNorm)(x) in training (normalise.jl:388-393): GroupNorm with one channel per group; with
    track_stats the running statistics take the batch mean of the per-instance statistics, the variance corrected
    by n/(n-1) with n the number of spatial positions (test/layers/normalisation.jl:262-275).
    Returns (y, new_running_mean, new_running_var)."""
    C, N = x.shape[-2], x.shape[-1]
    y = groupnorm_fwd(x, gamma, beta, C, eps, sigma)
    if not track_stats or run_mean is None:
        return y, run_mean, run_var
    S = x.size // (C * N)
    xv = x.reshape(S, C, N)
    mu = xv.mean(axis=0)                       # (C, N)
    var = ((xv - mu) ** 2).mean(axis=0)
    m = x.dtype.type(momentum)
    corr = x.dtype.type(S / (S - 1)) if S > 1 else x.dtype.type(1)
    return y, (1 - m) * run_mean + m * mu.mean(axis=1), (1 - m) * run_var + m * corr * var.mean(axis=1)


# --------------------------------------------------------------------------
# Embedding (basic.jl:794-800) and Dropout (normalise.jl:83 -> NNlib.dropout)
# --------------------------------------------------------------------------
def embedding_fwd(W, idx, padding_idx=None):
    """(m::Embedding)(x): columns W[:, idx] for 1-based integer indices of any shape; padding columns are zero."""
    idx = np.asarray(idx)
    if idx.min() < 1 or idx.max() > W.shape[1]:
        raise IndexError("BoundsError: embedding index outside 1:vocabulary")
    y = W[:, idx.reshape(-1) - 1]
    if padding_idx is not None:
        y = y * (idx.reshape(1, -1) != padding_idx)
    return y.reshape((W.shape[0],) + idx.shape)


def embedding_bwd(W, idx, dy, padding_idx=None):
    """Reverse of embedding_fwd: scatter-add of dy's columns (the rrule of NNlib.gather)."""
    idx = np.asarray(idx).reshape(-1)
    d = dy.reshape(W.shape[0], -1)
    dW = np.zeros_like(W)
    keep = np.ones(idx.shape, bool) if padding_idx is None else idx != padding_idx
    np.add.at(dW.T, idx[keep] - 1, d[:, keep].T)
    return dW


def philox4x32_10(counter, seed):
    """Philox4x32-10 (Salmon, Moraes, Dror, Shaw 2011) for uint64 counters and one uint64 key; returns (n, 4) uint32.
    The dropout mask of the device library is defined in terms of this generator, so it is restated here bit for bit."""
    counter = np.asarray(counter, dtype=np.uint64)
    c = [(counter & np.uint64(0xFFFFFFFF)).astype(np.uint64), (counter >> np.uint64(32)).astype(np.uint64),
         np.zeros_like(counter), np.zeros_like(counter)]
    k0, k1 = np.uint64(seed & 0xFFFFFFFF), np.uint64((seed >> 32) & 0xFFFFFFFF)
    M0, M1, MASK = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57), np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0, p1 = M0 * c[0], M1 * c[2]
        c = [((p1 >> np.uint64(32)) ^ c[1] ^ k0) & MASK, p1 & MASK, ((p0 >> np.uint64(32)) ^ c[3] ^ k1) & MASK, p0 & MASK]
        k0 = (k0 + np.uint64(0x9E3779B9)) & MASK
        k1 = (k1 + np.uint64(0xBB67AE85)) & MASK
    return np.stack(c, axis=-1).astype(np.uint32)


def dropout_mask(count, p, seed, offset=0):
    """keep[i] for i in 0:count: word i % 4 of Philox(counter = offset + i // 4, key = seed); keep iff
    (word >> 8) * 2^-24 >= p."""
    quads = (count + 3) // 4
    words = philox4x32_10(np.arange(quads, dtype=np.uint64) + np.uint64(offset), seed).reshape(-1)[:count]
    u = (words >> np.uint32(8)).astype(np.float32) * np.float32(1.0 / 16777216.0)
    return u >= np.float32(p)


def dropout_fwd(x, p, mask):
    """NNlib.dropout with a given keep-mask: x .* mask ./ (1 - p) (Flux's Dropout, normalise.jl:83)."""
    return x * mask.reshape(x.shape) / x.dtype.type(1 - p)


# --------------------------------------------------------------------------
# Recurrence: scan (recurrent.jl:1-8), LSTMCell (:411-419), GRUCell (:614-628)
# --------------------------------------------------------------------------
def _sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def lstm_scan_fwd(Wi, Wh, b, x, h0=None, c0=None, return_cache=False):
    """Recurrence(LSTMCell)(x): x is (in, T, B); returns out (H, T, B) and final (h, c).

    g = Wi x_t + Wh h + b; rows split i, f, g~, o (recurrent.jl:415);
    c' = sig(f) c + sig(i) tanh(g~); h' = sig(o) tanh(c').  Zero initial state
    vectors broadcast over the batch (recurrent.jl:391-393).
    """
    H = Wh.shape[1]
    I, T, B = x.shape
    dt = x.dtype
    h = np.zeros((H, B), dt) if h0 is None else np.broadcast_to(h0.reshape(H, -1), (H, B)).astype(dt)
    c = np.zeros((H, B), dt) if c0 is None else np.broadcast_to(c0.reshape(H, -1), (H, B)).astype(dt)
    bb = 0 if (b is None or b is False) else b.reshape(-1, 1)
    out = np.empty((H, T, B), dt)
    cache = []
    for t in range(T):
        g = Wi @ x[:, t, :] + Wh @ h + bb
        i_, f_, g_, o_ = (_sigmoid(g[0:H]), _sigmoid(g[H:2 * H]), np.tanh(g[2 * H:3 * H]), _sigmoid(g[3 * H:4 * H]))
        c_new = f_ * c + i_ * g_
        tc = np.tanh(c_new)
        h_new = o_ * tc
        if return_cache:
            cache.append((h, c, i_, f_, g_, o_, tc))
        h, c = h_new, c_new
        out[:, t, :] = h
    if return_cache:
        return out, (h, c), cache
    return out, (h, c)


def lstm_scan_bwd(Wi, Wh, b, x, dout, dhT=None, dcT=None):
    """BPTT through lstm_scan_fwd with zero initial state.  Returns dWi, dWh, db, dx."""
    H = Wh.shape[1]
    I, T, B = x.shape
    out, _, cache = lstm_scan_fwd(Wi, Wh, b, x, return_cache=True)
    dWi = np.zeros_like(Wi)
    dWh = np.zeros_like(Wh)
    db = np.zeros(4 * H, x.dtype)
    dx = np.zeros_like(x)
    dh = np.zeros((H, B), x.dtype) if dhT is None else dhT.copy()
    dc = np.zeros((H, B), x.dtype) if dcT is None else dcT.copy()
    for t in range(T - 1, -1, -1):
        h_prev, c_prev, i_, f_, g_, o_, tc = cache[t]
        dh = dh + dout[:, t, :]
        do = dh * tc
        dc = dc + dh * o_ * (1 - tc * tc)
        di = dc * g_
        dg = dc * i_
        df = dc * c_prev
        dgates = np.concatenate([di * i_ * (1 - i_), df * f_ * (1 - f_), dg * (1 - g_ * g_), do * o_ * (1 - o_)], axis=0)
        dWi += dgates @ x[:, t, :].T
        dWh += dgates @ h_prev.T
        db += dgates.sum(axis=1)
        dx[:, t, :] = Wi.T @ dgates
        dh = Wh.T @ dgates
        dc = dc * f_
    if b is None or b is False:
        db = None
    return dWi, dWh, db, dx


def gru_scan_fwd(Wi, Wh, b, x, h0=None, return_cache=False):
    """Recurrence(GRUCell)(x) (recurrent.jl:614-628): r, z, h~ rows; r multiplies Wh3 h, bias outside."""
    H = Wh.shape[1]
    I, T, B = x.shape
    dt = x.dtype
    h = np.zeros((H, B), dt) if h0 is None else np.broadcast_to(h0.reshape(H, -1), (H, B)).astype(dt)
    bb = np.zeros((3 * H, 1), dt) if (b is None or b is False) else b.reshape(-1, 1)
    out = np.empty((H, T, B), dt)
    cache = []
    for t in range(T):
        gx = Wi @ x[:, t, :]
        gh = Wh @ h
        r = _sigmoid(gx[0:H] + gh[0:H] + bb[0:H])
        z = _sigmoid(gx[H:2 * H] + gh[H:2 * H] + bb[H:2 * H])
        hc = np.tanh(gx[2 * H:] + r * gh[2 * H:] + bb[2 * H:])
        h_new = (1 - z) * hc + z * h
        if return_cache:
            cache.append((h, r, z, hc, gh[2 * H:]))
        h = h_new
        out[:, t, :] = h
    if return_cache:
        return out, h, cache
    return out, h


def gru_scan_bwd(Wi, Wh, b, x, dout, dhT=None):
    """BPTT through gru_scan_fwd with zero initial state.  Returns dWi, dWh, db, dx."""
    H = Wh.shape[1]
    I, T, B = x.shape
    out, _, cache = gru_scan_fwd(Wi, Wh, b, x, return_cache=True)
    dWi = np.zeros_like(Wi)
    dWh = np.zeros_like(Wh)
    db = np.zeros(3 * H, x.dtype)
    dx = np.zeros_like(x)
    dh = np.zeros((H, B), x.dtype) if dhT is None else dhT.copy()
    for t in range(T - 1, -1, -1):
        h_prev, r, z, hc, gh3 = cache[t]
        dh = dh + dout[:, t, :]
        dhc = dh * (1 - z)
        dz = dh * (h_prev - hc)
        dh_prev = dh * z
        da3 = dhc * (1 - hc * hc)          # pre-activation of h~
        dr = da3 * gh3
        da1 = dr * r * (1 - r)
        da2 = dz * z * (1 - z)
        dgx = np.concatenate([da1, da2, da3], axis=0)
        dgh = np.concatenate([da1, da2, da3 * r], axis=0)
        dWi += dgx @ x[:, t, :].T
        dWh += dgh @ h_prev.T
        db += dgx.sum(axis=1)
        dx[:, t, :] = Wi.T @ dgx
        dh = dh_prev + Wh.T @ dgh
    if b is None or b is False:
        db = None
    return dWi, dWh, db, dx


def rnn_scan_fwd(Wi, Wh, b, x, sigma="tanh", h0=None):
    """Recurrence(RNNCell)(x) (recurrent.jl:193-198): h' = sigma.(Wi x + Wh h + b); returns (out, hT)."""
    H = Wh.shape[1]
    I, T, B = x.shape
    dt = x.dtype
    h = np.zeros((H, B), dt) if h0 is None else np.broadcast_to(h0.reshape(H, -1), (H, B)).astype(dt)
    bb = np.zeros((H, 1), dt) if (b is None or b is False) else b.reshape(-1, 1)
    out = np.empty((H, T, B), dt)
    for t in range(T):
        h = act(sigma, Wi @ x[:, t, :] + Wh @ h + bb)
        out[:, t, :] = h
    return out, h


def rnn_scan_bwd(Wi, Wh, b, x, dout, sigma="tanh", h0=None, dhT=None):
    """BPTT through rnn_scan_fwd.  Returns dWi, dWh, db, dx."""
    H = Wh.shape[1]
    I, T, B = x.shape
    dt = x.dtype
    out, _ = rnn_scan_fwd(Wi, Wh, b, x, sigma, h0)
    h_init = np.zeros((H, B), dt) if h0 is None else np.broadcast_to(h0.reshape(H, -1), (H, B)).astype(dt)
    bb = np.zeros((H, 1), dt) if (b is None or b is False) else b.reshape(-1, 1)
    dWi, dWh, db, dx = np.zeros_like(Wi), np.zeros_like(Wh), np.zeros(H, dt), np.zeros_like(x)
    dh = np.zeros((H, B), dt) if dhT is None else dhT.copy()
    for t in range(T - 1, -1, -1):
        h_prev = h_init if t == 0 else out[:, t - 1, :]
        z = Wi @ x[:, t, :] + Wh @ h_prev + bb
        dpre = (dh + dout[:, t, :]) * act_grad(sigma, z)
        dWi += dpre @ x[:, t, :].T
        dWh += dpre @ h_prev.T
        db += dpre.sum(axis=1)
        dx[:, t, :] = Wi.T @ dpre
        dh = Wh.T @ dpre
    if b is None or b is False:
        db = None
    return dWi, dWh, db, dx


def gruv3_scan_fwd(Wi, Wh, b, Wh_h, x, h0=None, return_cache=False):
    """Recurrence(GRUv3Cell)(x) (recurrent.jl:795-809): r, z use the first two row blocks of Wi, Wh, b;
    h~ = tanh(gx3 + Wh_h (r .* h) + b3); the third row block of Wh is not read."""
    H = Wh.shape[1]
    I, T, B = x.shape
    dt = x.dtype
    h = np.zeros((H, B), dt) if h0 is None else np.broadcast_to(h0.reshape(H, -1), (H, B)).astype(dt)
    bb = np.zeros((3 * H, 1), dt) if (b is None or b is False) else b.reshape(-1, 1)
    out = np.empty((H, T, B), dt)
    cache = []
    for t in range(T):
        gx = Wi @ x[:, t, :]
        gh = Wh @ h
        r = _sigmoid(gx[0:H] + gh[0:H] + bb[0:H])
        z = _sigmoid(gx[H:2 * H] + gh[H:2 * H] + bb[H:2 * H])
        hc = np.tanh(gx[2 * H:] + Wh_h @ (r * h) + bb[2 * H:])
        h_new = (1 - z) * hc + z * h
        if return_cache:
            cache.append((h, r, z, hc))
        h = h_new
        out[:, t, :] = h
    if return_cache:
        return out, h, cache
    return out, h


def gruv3_scan_bwd(Wi, Wh, b, Wh_h, x, dout, dhT=None):
    """BPTT through gruv3_scan_fwd with zero initial state.  Returns dWi, dWh, db, dWh_h, dx."""
    H = Wh.shape[1]
    I, T, B = x.shape
    out, _, cache = gruv3_scan_fwd(Wi, Wh, b, Wh_h, x, return_cache=True)
    dWi, dWh, dWhh = np.zeros_like(Wi), np.zeros_like(Wh), np.zeros_like(Wh_h)
    db = np.zeros(3 * H, x.dtype)
    dx = np.zeros_like(x)
    dh = np.zeros((H, B), x.dtype) if dhT is None else dhT.copy()
    for t in range(T - 1, -1, -1):
        h_prev, r, z, hc = cache[t]
        dh = dh + dout[:, t, :]
        da3 = dh * (1 - z) * (1 - hc * hc)
        da2 = dh * (h_prev - hc) * z * (1 - z)
        drh = Wh_h.T @ da3
        da1 = drh * h_prev * r * (1 - r)
        dgx = np.concatenate([da1, da2, da3], axis=0)
        dWi += dgx @ x[:, t, :].T
        dWh[0:2 * H] += dgx[0:2 * H] @ h_prev.T
        dWhh += da3 @ (r * h_prev).T
        db += dgx.sum(axis=1)
        dx[:, t, :] = Wi.T @ dgx
        dh = dh * z + drh * r + Wh[0:2 * H].T @ dgx[0:2 * H]
    if b is None or b is False:
        db = None
    return dWi, dWh, db, dWhh, dx


# --------------------------------------------------------------------------
# MultiHeadAttention (src/layers/attention.jl:120-133 -> NNlib.dot_product_attention)
# --------------------------------------------------------------------------
def make_causal_mask(length):
    """NNlib.make_causal_mask: mask[j, i] (kv index j, query index i) true iff j <= i
    (pinned by test/layers/attention.jl:38-43: alpha[2,1,:,:] == 0, alpha == triu(alpha))."""
    return np.triu(np.ones((length, length), dtype=bool))


def _contract_c(a, b):
    """out[j, i, h, n] = sum_c a[h, c, j, n] * b[h, c, i, n] (one matrix product per head and batch entry)."""
    return np.matmul(a.transpose(3, 0, 2, 1), b.transpose(3, 0, 1, 2)).transpose(2, 3, 1, 0)


def _apply_ji(a, w):
    """out[h, c, i, n] = sum_j a[h, c, j, n] * w[j, i, h, n] (one matrix product per head and batch entry)."""
    return np.matmul(a.transpose(3, 0, 1, 2), w.transpose(3, 2, 0, 1)).transpose(1, 2, 3, 0)


def dot_product_attention(q, k, v, bias=None, nheads=1, mask=None, return_cache=False, drop=None):
    """q (E, Lq, B), k (E, Lk, B), v (Ev, Lk, B) -> x (Ev, Lq, B), alpha (Lk, Lq, h, B).

    Head h is the contiguous feature block h*d:(h+1)*d of the embed axis; scores
    k'q / sqrt(d); additive bias; boolean mask (true = keep, masked logits -> -inf);
    softmax over the kv axis; `fdrop` on the weights (attention.jl:91, 128; here `drop` = keep-mask / (1 - p) of
    alpha's shape); x = v alpha.  The returned alpha is the one after dropout, as in NNlib.
    """
    E, Lq, B = q.shape
    Ev, Lk, _ = v.shape
    d = E // nheads
    dv = Ev // nheads
    qh = q.reshape(nheads, d, Lq, B)      # Julia reshape(q, d, h, Lq, B) has d fastest; numpy C-order of (E,..) splits E as (h, d)
    kh = k.reshape(nheads, d, Lk, B)
    vh = v.reshape(nheads, dv, Lk, B)
    scale = q.dtype.type(1.0 / math.sqrt(d))
    # logits[j, i, h, b] = sum_c k[h,c,j,b] q[h,c,i,b] * scale
    logits = _contract_c(kh, qh) * scale
    if bias is not None:
        logits = logits + np.broadcast_to(bias.reshape(bias.shape + (1,) * (4 - bias.ndim)), logits.shape)
    if mask is not None:
        m = np.broadcast_to(mask.reshape(mask.shape + (1,) * (4 - mask.ndim)), logits.shape)
        logits = np.where(m, logits, -np.inf)
    mx = logits.max(axis=0, keepdims=True)
    e = np.exp(logits - mx)
    alpha0 = e / e.sum(axis=0, keepdims=True)
    alpha = alpha0 if drop is None else alpha0 * drop
    xh = _apply_ji(vh, alpha)
    x = xh.reshape(Ev, Lq, B)
    if return_cache:
        return x, alpha, (qh, kh, vh, scale, alpha0)
    return x, alpha


def dot_product_attention_bwd(q, k, v, dx, bias=None, nheads=1, mask=None, dalpha=None, drop=None):
    """Reverse of dot_product_attention: dV = dO alpha', dalpha = V' dO (+ the cotangent of the returned weights),
    through the dropout factor, dS = alpha0 .* (dalpha - sum(alpha0 .* dalpha)), dQ = K dS scale, dK = Q dS' scale."""
    E, Lq, B = q.shape
    Ev, Lk, _ = v.shape
    x, alpha, (qh, kh, vh, scale, alpha0) = dot_product_attention(q, k, v, bias, nheads, mask, return_cache=True, drop=drop)
    d = E // nheads
    dv = Ev // nheads
    dxh = dx.reshape(nheads, dv, Lq, B)
    dvh = _apply_ji(dxh, alpha.transpose(1, 0, 2, 3))
    da = _contract_c(vh, dxh)
    if dalpha is not None:
        da = da + dalpha
    if drop is not None:
        da = da * drop
    ds = alpha0 * (da - (alpha0 * da).sum(axis=0, keepdims=True))
    dqh = _apply_ji(kh, ds) * scale
    dkh = _apply_ji(qh, ds.transpose(1, 0, 2, 3)) * scale
    return dqh.reshape(E, Lq, B), dkh.reshape(E, Lk, B), dvh.reshape(Ev, Lk, B)


def mha_fwd(Wq, Wk, Wv, Wo, q_in, k_in=None, v_in=None, nheads=8, mask=None, bias=None,
            bq=None, bk=None, bv=None, bo=None):
    """MultiHeadAttention call (attention.jl:120-133): three Dense projections, attention, output Dense."""
    k_in = q_in if k_in is None else k_in
    v_in = k_in if v_in is None else v_in
    q = dense_fwd(Wq, bq, q_in)
    k = dense_fwd(Wk, bk, k_in)
    v = dense_fwd(Wv, bv, v_in)
    x, alpha = dot_product_attention(q, k, v, bias, nheads, mask)
    y = dense_fwd(Wo, bo, x)
    return y, alpha


def mha_bwd(Wq, Wk, Wv, Wo, x_in, dy, nheads=8, mask=None):
    """Reverse of self-attention mha_fwd(x_in) w.r.t. the four weights and the input
    (loss uses the first output only, as `first o mha` in test/test_module.jl:63)."""
    q = dense_fwd(Wq, None, x_in)
    k = dense_fwd(Wk, None, x_in)
    v = dense_fwd(Wv, None, x_in)
    x, alpha = dot_product_attention(q, k, v, None, nheads, mask)
    dWo, _, dxa = dense_bwd(Wo, None, x, dy)
    dq, dk, dv = dot_product_attention_bwd(q, k, v, dxa, None, nheads, mask)
    dWq, _, dx1 = dense_bwd(Wq, None, x_in, dq)
    dWk, _, dx2 = dense_bwd(Wk, None, x_in, dk)
    dWv, _, dx3 = dense_bwd(Wv, None, x_in, dv)
    return dWq, dWk, dWv, dWo, dx1 + dx2 + dx3


# --------------------------------------------------------------------------
# losses (src/losses/functions.jl:270-273) and sum(abs2, y)
# --------------------------------------------------------------------------
def logsoftmax(z, axis=0):
    mx = z.max(axis=axis, keepdims=True)
    s = z - mx
    return s - np.log(np.exp(s).sum(axis=axis, keepdims=True))


def onehotbatch(labels, nclasses, dtype=np.float32):
    """OneHotArrays.onehotbatch(labels, 1:nclasses): labels are 1-based."""
    labels = np.asarray(labels)
    y = np.zeros((nclasses, labels.size), dtype)
    y[labels - 1, np.arange(labels.size)] = 1
    return y


def logitcrossentropy(yhat, y):
    """mean(.-sum(y .* logsoftmax(yhat; dims=1); dims=1)) (functions.jl:270-273)."""
    if yhat.shape != y.shape:
        raise ValueError("DimensionMismatch: loss function expects size(yhat) == size(y)")
    return (-(y * logsoftmax(yhat, 0)).sum(axis=0)).mean()


def logitcrossentropy_bwd(yhat, y, dloss=1.0):
    """d loss / d yhat = (softmax(yhat) .* sum(y, dims=1) .- y) / N."""
    n = yhat[0].size
    p = np.exp(logsoftmax(yhat, 0))
    return (p * y.sum(axis=0, keepdims=True) - y) * (dloss / n)


def sum_abs2(y):
    return (y * y).sum()


def sum_abs2_bwd(y, dloss=1.0):
    return 2 * dloss * y


# --------------------------------------------------------------------------
# Adam (in-tree statement: src/optimise/optimisers.jl:171-184; state (m, v, beta^t))
# --------------------------------------------------------------------------
def adam_init(x):
    return [np.zeros_like(x), np.zeros_like(x), (0.9, 0.999)]


def adam_apply(state, x, g, eta=1e-3, beta=(0.9, 0.999), eps=1e-8):
    """One Adam update, in place on `state` and returning the new parameter.

    m = b1 m + (1-b1) g ; v = b2 v + (1-b2) g^2 ;
    x <- x - m/(1-b1^t) / (sqrt(v/(1-b2^t)) + eps) * eta ; b^t *= b.
    Scalars are taken in the parameter's eltype, as Optimisers.jl does.
    """
    T = x.dtype.type
    m, v, bt = state
    b1, b2 = T(beta[0]), T(beta[1])
    bt1, bt2 = T(bt[0]), T(bt[1])
    m[...] = b1 * m + (T(1) - b1) * g
    v[...] = b2 * v + (T(1) - b2) * g * g
    dx = m / (T(1) - bt1) / (np.sqrt(v / (T(1) - bt2)) + T(eps)) * T(eta)
    state[2] = (float(bt1 * b1), float(bt2 * b2))
    return x - dx


# --------------------------------------------------------------------------
# DistributedUtils (src/distributed/public_api.jl)
# --------------------------------------------------------------------------
def distributed_shard_indices(total_size, total_workers, local_rank):
    """public_api.jl:262-272: contiguous ceil(n/N) 0-based index ranges, shorter last shard."""
    size_per_worker = int(math.ceil(total_size / total_workers))
    parts = [range(s, min(s + size_per_worker, total_size)) for s in range(0, total_size, size_per_worker)]
    if local_rank >= len(parts):
        raise IndexError("BoundsError: no partition for this rank")
    return np.arange(parts[local_rank].start, parts[local_rank].stop)


def allreduce(bufs, op="avg"):
    """public_api.jl:134-150 / FluxMPINCCLExt.jl:61-66: every rank ends with sum (or mean) of all ranks' buffers."""
    s = np.sum(np.stack(bufs, 0), axis=0)
    if op == "avg":
        s = s / len(bufs)
    elif op != "+":
        raise ValueError(op)
    return [s.copy() for _ in bufs]


def bcast(bufs, root=0):
    """public_api.jl:102-116: every rank ends with root's buffer."""
    return [bufs[root].copy() for _ in bufs]


def reduce(bufs, op="+", root=0):
    """public_api.jl:166-183: root ends with the reduction; other ranks keep their buffers."""
    s = np.sum(np.stack(bufs, 0), axis=0)
    if op == "avg":
        s = s / len(bufs)
    out = [b.copy() for b in bufs]
    out[root] = s
    return out


# --------------------------------------------------------------------------
# whole-model helpers used by parity tests and the CPU baseline
# --------------------------------------------------------------------------
def mlp_chain_fwd_bwd(layers, x, y_onehot):
    """Chain(Dense...) + logitcrossentropy: returns loss and per-layer (dW, db) plus dx.

    `layers` is a list of (W, b, sigma).  Mirrors Zygote's reverse sweep over
    basic.jl:65-72 / :196-200.
    """
    acts = [x]
    for (W, b, s) in layers:
        acts.append(dense_fwd(W, b, acts[-1], s))
    loss = logitcrossentropy(acts[-1], y_onehot)
    d = logitcrossentropy_bwd(acts[-1], y_onehot)
    grads = []
    for (W, b, s), xin in zip(reversed(layers), reversed(acts[:-1])):
        dW, db, d = dense_bwd(W, b, xin, d, s)
        grads.append((dW, db))
    grads.reverse()
    return loss, grads, d


def dp_mlp_fwd_bwd(blocks, head, x, y_onehot, gelu="gelu_tanh", eps=1e-5):
    """Config-5 model: blocks of LayerNorm(D) -> Dense(D=>D, gelu), then Dense(D=>C); logitcrossentropy.

    blocks: list of dicts {gamma, beta, W, b}; head: {W, b}.  Returns loss and a
    gradient structure of the same shape.
    """
    h = x
    saved = []
    for blk in blocks:
        hn = layernorm_fwd(h, blk["gamma"], blk["beta"], eps)
        hd = dense_fwd(blk["W"], blk["b"], hn, gelu)
        saved.append((h, hn))
        h = hd
    logits = dense_fwd(head["W"], head["b"], h)
    loss = logitcrossentropy(logits, y_onehot)
    d = logitcrossentropy_bwd(logits, y_onehot)
    dWh, dbh, d = dense_bwd(head["W"], head["b"], h, d)
    ghead = {"W": dWh, "b": dbh}
    gblocks = []
    for blk, (hin, hn) in zip(reversed(blocks), reversed(saved)):
        dW, db, dhn = dense_bwd(blk["W"], blk["b"], hn, d, gelu)
        dxin, dgamma, dbeta = layernorm_bwd(hin, blk["gamma"], blk["beta"], dhn, eps)
        gblocks.append({"gamma": dgamma, "beta": dbeta, "W": dW, "b": db})
        d = dxin
    gblocks.reverse()
    return loss, gblocks, ghead


def finite_difference(f, x, h=1e-6):
    """Central finite-difference gradient of scalar f at float64 x (used by the oracle's own tests,
    following the reference's test/test_module.jl:100 approach)."""
    x = np.array(x, dtype=np.float64)
    g = np.zeros_like(x)
    it = np.nditer(x, flags=["multi_index"])
    while not it.finished:
        idx = it.multi_index
        old = x[idx]
        x[idx] = old + h
        fp = f(x)
        x[idx] = old - h
        fm = f(x)
        x[idx] = old
        g[idx] = (fp - fm) / (2 * h)
        it.iternext()
    return g
