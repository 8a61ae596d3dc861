"""Host-side mirror of Flux's layers for B200 arrays: same names, fields, argument meaning and errors.

Each call operator does what the Julia extension's method does: size checks on the host, one call
into libfluxb200.so, and (under `withgradient`) a recorded pullback that calls the matching
backward entry point.  Reference: src/layers/basic.jl (Chain :49-81, Dense :179-205),
normalise.jl (LayerNorm :186-210, BatchNorm :259-307), recurrent.jl (scan :1-8, Recurrence :61-81,
LSTMCell :383-419, GRUCell :586-628, LSTM :491-524, GRU :685-718), attention.jl (:68-133).
"""
from __future__ import annotations

import numpy as np
import torch

from . import lib
from .core import B200Array, Tape, context, empty, gpu, is_bf16, to_bf16, to_f32, zeros
from .init import glorot_uniform


class DimensionMismatch(ValueError):
    pass


class ArgumentError(ValueError):
    pass


def _act_name(sigma) -> str:
    if sigma is None:
        return "identity"
    if callable(sigma) and hasattr(sigma, "__name__"):
        sigma = sigma.__name__
    if sigma not in lib.ACT:
        raise lib.FluxB200Error(-7, f"activation {sigma!r} has no B200 kernel (known: {sorted(lib.ACT)})")
    return sigma


def _ptr(a):
    return a.ptr if a is not None else None


def _wait_params(*params):
    """A gradient sink that defers the parameter all-gather to the next step's forward pass must have delivered a
    layer's parameters before the layer reads them."""
    sink = Tape.grad_sink
    if sink is not None and getattr(sink, "gathering", False):
        for p in params:
            if isinstance(p, B200Array):
                sink.wait_param(p)


def _size_check(layer, x: B200Array, d: int, n: int):
    """basic.jl:217-223 (d is 1-based)."""
    if not (0 < d <= x.ndim):
        raise DimensionMismatch(f"layer {layer} expects ndims(input) >= {d}, but got {x}")
    if x.size[d - 1] != n:
        raise DimensionMismatch(f"layer {layer} expects size(input, {d}) == {n}, but got {x}")


class Layer:
    """Base: `_fields` names the child fields (arrays, layers, scalars) in Flux's order;
    `_trainable` the trainable subset (Flux's `@layer ... trainable=`)."""

    _fields: tuple = ()
    _trainable = None

    def _fmap(self, f):
        import copy
        new = copy.copy(self)
        for name in self._fields:
            v = getattr(self, name)
            if isinstance(v, (B200Array, np.ndarray, tuple, list, dict)) or hasattr(v, "_fmap"):
                setattr(new, name, f(v))
        return new

    def trainable_fields(self):
        return self._fields if self._trainable is None else self._trainable


def trainables(obj) -> list:
    """Flux.trainables: the trainable arrays in traversal order."""
    out = []
    if isinstance(obj, B200Array):
        out.append(obj)
    elif isinstance(obj, (tuple, list)):
        for v in obj:
            out.extend(trainables(v))
    elif isinstance(obj, Layer):
        for name in obj.trainable_fields():
            out.extend(trainables(getattr(obj, name)))
    return out


# ------------------------------------------------------------------------------------ Chain ---
class Chain(Layer):
    _fields = ("layers",)

    def __init__(self, *layers):
        self.layers = tuple(layers)

    def __call__(self, x):
        for l in self.layers:
            x = l(x)
        return x

    def __getitem__(self, i):
        return self.layers[i]

    def __repr__(self):
        return "Chain(" + ", ".join(map(repr, self.layers)) + ")"


def _round_bf16(a: B200Array) -> B200Array:
    """In place: every element becomes Float32(BFloat16(element)) (round to nearest even, NaN -> canonical NaN)."""
    ctx = context()
    lib.call("fb_round_bf16", ctx.handle, ctx.stream, a.ptr, a.ptr, a.numel())
    return a


def bf16(m):
    """Flux.bf16 (src/functor.jl:274, 137-183): the opt-in low-precision path.  For an array: BFloat16 storage (2 bytes
    per element, round to nearest even).  For a model: the weights and biases of its Dense layers move to BFloat16
    storage and those layers run on the bf16 tensor-core GEMM (Float32 accumulation, BFloat16 activations and
    gradients); the parameters of the other layers are rounded to BFloat16 values and keep Float32 storage, since
    their kernels compute in Float32 (as the reference keeps normalisation statistics in Float32,
    normalise.jl:513-519).  Arrays that cross between the two are converted on the way."""
    if isinstance(m, B200Array):
        return to_bf16(m)
    for layer in _walk(m):
        if isinstance(layer, BatchNorm):
            continue
        if isinstance(layer, Dense):
            layer.precision = "bf16"
            layer.weight = to_bf16(layer.weight)
            if layer.bias is not False:
                layer.bias = to_bf16(layer.bias)
            continue
        for name in layer.trainable_fields():
            v = getattr(layer, name, None)
            if isinstance(v, B200Array) and v.t.dtype == torch.float32:
                _round_bf16(v)
    return m


def f32(m):
    """Flux.f32 (src/functor.jl:137-148): back to Float32 storage and the Float32 kernels."""
    if isinstance(m, B200Array):
        return to_f32(m)
    for layer in _walk(m):
        if isinstance(layer, Dense) and layer.precision == "bf16":
            layer.precision = "default"
            layer.weight = to_f32(layer.weight)
            if layer.bias is not False:
                layer.bias = to_f32(layer.bias)
    return m


# ------------------------------------------------------------------------------------ Dense ---
class Dense(Layer):
    """Dense(W, bias, sigma): y = sigma.(W*x .+ b) (basic.jl:179-205). `bias=False` means no bias.

    `Dense((in, out), sigma, bias=True, init=glorot_uniform)` is Flux's `Dense(in => out, σ; init, bias)`
    (basic.jl:189-192): the weight is `init(out, in)`."""

    _fields = ("weight", "bias", "σ")
    _trainable = ("weight", "bias")

    def __init__(self, weight, bias=True, sigma="identity", precision="default", init=glorot_uniform):
        if isinstance(weight, (tuple, list)) and len(weight) == 2 and all(isinstance(v, (int, np.integer)) for v in weight):
            if isinstance(bias, str):      # Dense((in, out), "relu")
                bias, sigma = True, bias
            in_dim, out_dim = int(weight[0]), int(weight[1])
            weight = init(out_dim, in_dim)
        self.weight = gpu(weight) if isinstance(weight, np.ndarray) else weight
        if self.weight.ndim != 2:
            raise TypeError("MethodError: Dense weight must be a matrix")
        out = self.weight.size[0]
        if bias is True:
            bias = zeros((out,))
        elif bias is False or bias is None:
            bias = False
        else:
            bias = gpu(bias) if isinstance(bias, np.ndarray) else bias
            if bias.size != (out,):
                raise DimensionMismatch(f"expected bias of size ({out},), got size {bias.size}")
        self.bias = bias
        self.σ = _act_name(sigma)
        self.precision = precision

    def __repr__(self):
        return f"Dense({self.weight.size[1]} => {self.weight.size[0]}, {self.σ})"

    def __call__(self, x: B200Array) -> B200Array:
        if not isinstance(x, B200Array):
            raise TypeError("MethodError: Dense expects an array")
        out_dim, in_dim = self.weight.size
        _size_check(self, x, 1, in_dim)
        n = x.numel() // in_dim
        ctx = context()
        _wait_params(self.weight, self.bias)
        if is_bf16(self.weight):
            return self._call_bf16(to_bf16(x), out_dim, in_dim, n)
        x = to_f32(x)
        act, prec = lib.ACT[self.σ], lib.PREC[self.precision]
        b = self.bias if self.bias is not False else None
        recording = Tape.active
        y = empty((out_dim,) + x.size[1:])
        z = empty(y.size) if (recording and self.σ in ("gelu", "gelu_tanh", "gelu_erf")) else None
        lib.call("fb_dense_fwd", ctx.handle, ctx.stream, act, prec, self.weight.ptr, _ptr(b), x.ptr, y.ptr, _ptr(z),
                 out_dim, in_dim, n)
        if recording:
            W = self.weight

            def pullback(gs, x=x, y=y, z=z):
                dy = gs[0]
                need_dx = Tape.needs(x)
                sink = Tape.grad_sink
                dW = (sink.buffer_for(W) if sink else None) or empty(W.size)
                db = ((sink.buffer_for(b) if sink else None) or empty(b.size)) if b is not None else None
                dx = empty(x.size) if need_dx else None
                delta = empty(y.size) if act != 0 else None
                if sink is not None and need_dx and hasattr(sink, "ready"):
                    # dW (and db) first, reported to the gradient sink at once so that their exchange overlaps the dX product
                    lib.call("fb_dense_bwd", ctx.handle, ctx.stream, act, prec, W.ptr, x.ptr, y.ptr, _ptr(z), dy.ptr,
                             _ptr(delta), dW.ptr, _ptr(db), None, out_dim, in_dim, n)
                    sink.ready(W, early=True)
                    d = delta if act != 0 else dy
                    lib.call("fb_gemm_f32", ctx.handle, ctx.stream, 1, 0, in_dim, n, out_dim, W.ptr, out_dim, d.ptr, out_dim, dx.ptr, in_dim,
                             0, prec)
                else:
                    lib.call("fb_dense_bwd", ctx.handle, ctx.stream, act, prec, W.ptr, x.ptr, y.ptr, _ptr(z), dy.ptr,
                             _ptr(delta), dW.ptr, _ptr(db), _ptr(dx), out_dim, in_dim, n)
                res = [(W, dW)]
                if b is not None:
                    res.append((b, db))
                if need_dx:
                    res.append((x, dx))
                return res

            Tape.record(y, [x, W, b], pullback)
        return y


def _dense_call_bf16(self, x, out_dim, in_dim, n):
    """The Dense call for BFloat16 storage: one fused tensor-core GEMM (bias, activation, pre-activation) forward,
    fb_dense_bwd_bf16 in the pullback; every array involved is bf16."""
    ctx = context()
    act = lib.ACT[self.σ]
    W = self.weight
    b = self.bias if self.bias is not False else None
    recording = Tape.active
    bf = torch.bfloat16
    y = empty((out_dim,) + x.size[1:], bf)
    z = empty(y.size, bf) if (recording and self.σ in ("gelu", "gelu_tanh", "gelu_erf")) else None
    lib.call("fb_dense_fwd_bf16", ctx.handle, ctx.stream, act, W.ptr, _ptr(b), x.ptr, y.ptr, _ptr(z), out_dim, in_dim, n)
    if recording:
        def pullback(gs, x=x, y=y, z=z):
            dy = to_bf16(gs[0])
            need_dx = Tape.needs(x)
            dW = empty(W.size, bf)
            db = empty(b.size, bf) if b is not None else None
            dx = empty(x.size, bf) if need_dx else None
            delta = empty(y.size, bf) if act != 0 else None
            lib.call("fb_dense_bwd_bf16", ctx.handle, ctx.stream, act, W.ptr, x.ptr, y.ptr, _ptr(z), dy.ptr, _ptr(delta), dW.ptr,
                     _ptr(db), _ptr(dx), out_dim, in_dim, n)
            res = [(W, dW)]
            if b is not None:
                res.append((b, db))
            if need_dx:
                res.append((x, dx))
            return res

        Tape.record(y, [x, W, b], pullback)
    return y


Dense._call_bf16 = _dense_call_bf16


# -------------------------------------------------------------------------------- LayerNorm ---
class LayerNorm(Layer):
    """LayerNorm(size..., λ; affine=true, eps=1f-5) (normalise.jl:186-210); `diag` is the Scale."""

    _fields = ("λ", "diag", "ε", "size", "affine")
    _trainable = ("diag",)

    class _Scale(Layer):
        _fields = ("scale", "bias", "σ")
        _trainable = ("scale", "bias")

        def __init__(self, size, sigma):
            self.scale = gpu(np.ones(size, np.float32))
            self.bias = gpu(np.zeros(size, np.float32))
            self.σ = sigma

    def __init__(self, *size, sigma="identity", affine=True, eps=1e-5):
        if len(size) == 1 and isinstance(size[0], (tuple, list)):
            size = tuple(size[0])
        self.size = tuple(int(s) for s in size)
        self.λ = _act_name(sigma)
        self.affine = bool(affine)
        self.ε = float(eps)
        self.diag = LayerNorm._Scale(self.size, self.λ) if affine else None

    def __repr__(self):
        return f"LayerNorm({', '.join(map(str, self.size))})"

    def __call__(self, x: B200Array) -> B200Array:
        x = to_f32(x)
        if self.affine:
            _wait_params(self.diag.scale, self.diag.bias)
            for d, s in enumerate(self.size):
                _size_check(self, x, d + 1, s)
        d = int(np.prod(self.size))
        if x.numel() % d != 0 or x.size[:len(self.size)] != self.size:
            raise DimensionMismatch(f"layer {self} expects leading dims {self.size}, got {x}")
        n = x.numel() // d
        ctx = context()
        act = lib.ACT[self.λ]
        g = self.diag.scale if self.affine else None
        b = self.diag.bias if self.affine else None
        y, mean, rstd = empty(x.size), empty((n,)), empty((n,))
        lib.call("fb_layernorm_fwd", ctx.handle, ctx.stream, x.ptr, _ptr(g), _ptr(b), y.ptr, mean.ptr, rstd.ptr, d, n,
                 self.ε, act)
        if Tape.active:
            def pullback(gs, x=x):
                dy = gs[0]
                sink = Tape.grad_sink
                dx = empty(x.size)
                dg = ((sink.buffer_for(g) if sink else None) or empty(g.size)) if g is not None else None
                dbeta = ((sink.buffer_for(b) if sink else None) or empty(b.size)) if b is not None else None
                lib.call("fb_layernorm_bwd", ctx.handle, ctx.stream, x.ptr, _ptr(g), _ptr(b), mean.ptr, rstd.ptr, dy.ptr,
                         dx.ptr, _ptr(dg), _ptr(dbeta), d, n, act)
                res = [(x, dx)] if Tape.needs(x) else []
                if g is not None:
                    res += [(g, dg), (b, dbeta)]
                return res

            Tape.record(y, [x, g, b], pullback)
        return y


# -------------------------------------------------------------------------------- BatchNorm ---
class BatchNorm(Layer):
    """BatchNorm(chs, λ; affine, track_stats, eps=1f-5, momentum=0.1f0) (normalise.jl:259-307).

    `active=None` means automatic: training under `withgradient`, inference otherwise (`_isactive`)."""

    _fields = ("λ", "β", "γ", "μ", "σ2", "ε", "momentum", "affine", "track_stats", "active", "chs")
    _trainable = ("β", "γ")

    def __init__(self, chs: int, sigma="identity", affine=True, track_stats=True, active=None, eps=1e-5, momentum=0.1):
        self.chs = int(chs)
        self.λ = _act_name(sigma)
        self.affine, self.track_stats, self.active = bool(affine), bool(track_stats), active
        self.ε, self.momentum = float(eps), float(momentum)
        self.β = gpu(np.zeros(chs, np.float32)) if affine else None
        self.γ = gpu(np.ones(chs, np.float32)) if affine else None
        self.μ = gpu(np.zeros(chs, np.float32)) if track_stats else None
        self.σ2 = gpu(np.ones(chs, np.float32)) if track_stats else None

    def __repr__(self):
        return f"BatchNorm({self.chs}, {self.λ})"

    def _isactive(self):
        return Tape.active if self.active is None else bool(self.active)

    def __call__(self, x: B200Array) -> B200Array:
        x = to_f32(x)
        N = x.ndim
        if N < 2:
            raise DimensionMismatch(f"layer {self} expects ndims(input) >= 2, but got {x}")
        _size_check(self, x, N - 1, self.chs)
        training = self._isactive()
        s = int(np.prod(x.size[:N - 2], dtype=np.int64)) if N > 2 else 1
        c, n = self.chs, x.size[-1]
        if training and s * n == 1:
            raise ArgumentError(
                f"BatchNorm expected more than 1 value per channel when training, got input of size {x.size}. "
                "The batch variance of a single value is undefined; use a larger batch or call `testmode!` for inference.")
        ctx = context()
        act = lib.ACT[self.λ]
        y = empty(x.size)
        if not training and self.track_stats:
            lib.call("fb_batchnorm_fwd_infer", ctx.handle, ctx.stream, x.ptr, _ptr(self.γ), _ptr(self.β), self.μ.ptr,
                     self.σ2.ptr, y.ptr, s, c, n, self.ε, act)
            return y
        mean, rstd = empty((c,)), empty((c,))
        lib.call("fb_batchnorm_fwd_train", ctx.handle, ctx.stream, x.ptr, _ptr(self.γ), _ptr(self.β), _ptr(self.μ),
                 _ptr(self.σ2), y.ptr, mean.ptr, rstd.ptr, s, c, n, self.ε, self.momentum, act,
                 1 if (training and self.track_stats) else 0)
        if Tape.active:
            g, b = self.γ, self.β

            def pullback(gs, x=x):
                dy = gs[0]
                dx = empty(x.size)
                dg = empty((c,)) if g is not None else None
                dbeta = empty((c,)) if b is not None else None
                lib.call("fb_batchnorm_bwd", ctx.handle, ctx.stream, x.ptr, _ptr(g), _ptr(b), mean.ptr, rstd.ptr, dy.ptr,
                         dx.ptr, _ptr(dg), _ptr(dbeta), s, c, n, act)
                res = [(x, dx)] if Tape.needs(x) else []
                if g is not None:
                    res += [(g, dg), (b, dbeta)]
                return res

            Tape.record(y, [x, g, b], pullback)
        return y


def testmode(m, mode=True):
    """Flux.testmode! (functor.jl:30-54): walks the model and sets `.active`."""
    for layer in _walk(m):
        if hasattr(layer, "active"):
            layer.active = None if mode is None else (not mode)
    return m


def trainmode(m):
    return testmode(m, False)


def _walk(m):
    if isinstance(m, Layer):
        yield m
        for name in m._fields:
            yield from _walk(getattr(m, name, None))
    elif isinstance(m, (tuple, list)):
        for v in m:
            yield from _walk(v)


# ---------------------------------------------------------------------------------- recurrent ---
class LSTMCell(Layer):
    """LSTMCell(Wi, Wh, bias): Wi (4H, in), Wh (4H, H), b (4H) with gate rows i, f, g, o (recurrent.jl:383-419)."""

    _fields = ("Wi", "Wh", "bias")
    NG = 4

    def __init__(self, Wi, Wh=None, bias=True, init_kernel=glorot_uniform, init_recurrent_kernel=glorot_uniform):
        if isinstance(Wi, (tuple, list)) and len(Wi) == 2 and all(isinstance(v, (int, np.integer)) for v in Wi):
            in_dim, out = int(Wi[0]), int(Wi[1])     # LSTMCell(in => out) (recurrent.jl:395-407)
            Wi, Wh = init_kernel(out * 4, in_dim), init_recurrent_kernel(out * 4, out)
        self.Wi, self.Wh = gpu(Wi), gpu(Wh)
        rows = self.Wi.size[0]
        if bias is True:
            bias = zeros((rows,))
        elif bias is False or bias is None:
            bias = False
        else:
            bias = gpu(bias)
        self.bias = bias

    @property
    def hidden(self):
        return self.Wh.size[1]

    def initialstates(self):
        H = self.hidden
        return zeros((H,)), zeros((H,))


class GRUCell(Layer):
    """GRUCell(Wi, Wh, b): rows r, z, h~ (recurrent.jl:586-628)."""

    _fields = ("Wi", "Wh", "b")
    NG = 3

    def __init__(self, Wi, Wh=None, b=True, init_kernel=glorot_uniform, init_recurrent_kernel=glorot_uniform):
        if isinstance(Wi, (tuple, list)) and len(Wi) == 2 and all(isinstance(v, (int, np.integer)) for v in Wi):
            in_dim, out = int(Wi[0]), int(Wi[1])     # GRUCell(in => out) (recurrent.jl:596-607)
            Wi, Wh = init_kernel(out * 3, in_dim), init_recurrent_kernel(out * 3, out)
        self.Wi, self.Wh = gpu(Wi), gpu(Wh)
        rows = self.Wi.size[0]
        if b is True:
            b = zeros((rows,))
        elif b is False or b is None:
            b = False
        else:
            b = gpu(b)
        self.b = b

    @property
    def hidden(self):
        return self.Wh.size[1]

    def initialstates(self):
        return zeros((self.hidden,))


def _broadcast_state(s: B200Array | None, H: int, B: int):
    """A length-H state vector is broadcast over the batch (recurrent.jl:391-393); None = zeros."""
    if s is None:
        return None
    if s.size == (H, B):
        return s
    if s.size == (H,):
        return B200Array(s.t.repeat(B).contiguous(), (H, B))   # memory [B][H]
    raise DimensionMismatch(f"state of size {s.size} does not match hidden size {H} and batch {B}")


class Recurrence(Layer):
    """Recurrence(cell; return_state=false): applies `scan(cell, x, state)` over x[in, T, B] (recurrent.jl:1-8, 61-81)."""

    _fields = ("cell",)

    def __init__(self, cell, return_state=False):
        self.cell = cell
        self.return_state = bool(return_state)

    def __call__(self, x: B200Array, state=None):
        cell = self.cell
        x = to_f32(x)
        if not isinstance(cell, (LSTMCell, GRUCell)):
            return _scan_family(self, x, state)
        in_dim = cell.Wi.size[1]
        _size_check(cell, x, 1, in_dim)
        if x.ndim == 2:
            x3 = x.reshape(x.size[0], x.size[1], 1)
        elif x.ndim == 3:
            x3 = x
        else:
            raise DimensionMismatch(f"Recurrence expects a 2-d or 3-d input, got {x}")
        _, T, B = x3.size
        H = cell.hidden
        ctx = context()
        recording = Tape.active
        is_lstm = isinstance(cell, LSTMCell)
        bias = (cell.bias if is_lstm else cell.b)
        bias = bias if bias is not False else None
        out = empty((H, T, B))
        hT = empty((H, B))
        if is_lstm:
            h0, c0 = (None, None) if state is None else state
            h0, c0 = _broadcast_state(h0, H, B), _broadcast_state(c0, H, B)
            cT = empty((H, B))
            cache = None
            if recording:
                nbytes = lib.raw().fb_lstm_cache_bytes(in_dim, H, T, B)
                cache = torch.empty(max(nbytes // 4, 1), dtype=torch.float32, device=x.t.device)
            lib.call("fb_lstm_fwd", ctx.handle, ctx.stream, cell.Wi.ptr, cell.Wh.ptr, _ptr(bias), x3.ptr, _ptr(h0), _ptr(c0),
                     out.ptr, hT.ptr, cT.ptr, cache.data_ptr() if cache is not None else None, in_dim, H, T, B)
            final = (hT, cT)
        else:
            h0 = _broadcast_state(state, H, B)
            cache = None
            if recording:
                nbytes = lib.raw().fb_gru_cache_bytes(in_dim, H, T, B)
                cache = torch.empty(max(nbytes // 4, 1), dtype=torch.float32, device=x.t.device)
            lib.call("fb_gru_fwd", ctx.handle, ctx.stream, cell.Wi.ptr, cell.Wh.ptr, _ptr(bias), x3.ptr, _ptr(h0), out.ptr,
                     hT.ptr, cache.data_ptr() if cache is not None else None, in_dim, H, T, B)
            final = hT
        if recording:
            def pullback(gs, x3=x3):
                dout = gs[0] if gs[0] is not None else zeros(out.size)
                dWi, dWh = empty(cell.Wi.size), empty(cell.Wh.size)
                db = empty(bias.size) if bias is not None else None
                dx = empty(x3.size) if Tape.needs(x3) else None
                if is_lstm:
                    dhT, dcT = gs[1], gs[2]
                    lib.call("fb_lstm_bwd", ctx.handle, ctx.stream, cell.Wi.ptr, cell.Wh.ptr, x3.ptr, _ptr(h0), _ptr(c0),
                             out.ptr, cache.data_ptr(), dout.ptr, _ptr(dhT), _ptr(dcT), dWi.ptr, dWh.ptr, _ptr(db),
                             _ptr(dx), in_dim, H, T, B)
                else:
                    dhT = gs[1]
                    lib.call("fb_gru_bwd", ctx.handle, ctx.stream, cell.Wi.ptr, cell.Wh.ptr, x3.ptr, _ptr(h0), out.ptr,
                             cache.data_ptr(), dout.ptr, _ptr(dhT), dWi.ptr, dWh.ptr, _ptr(db), _ptr(dx), in_dim, H, T, B)
                res = [(cell.Wi, dWi), (cell.Wh, dWh)]
                if bias is not None:
                    res.append((bias, db))
                if dx is not None:
                    res.append((x3, dx))
                return res

            outs = [out, hT, cT] if is_lstm else [out, hT]
            Tape.record(outs, [x3, cell.Wi, cell.Wh, bias], pullback)
        y = out if x.ndim == 3 else out.reshape(H, T)
        if self.return_state:
            return y, final
        return y


def LSTM(Wi, Wh=None, bias=True, return_state=False, **init):
    """LSTM(in => out) == Recurrence(LSTMCell(in => out)) (recurrent.jl:491-524); `LSTM((in, out))` or explicit arrays."""
    return Recurrence(LSTMCell(Wi, Wh, bias, **init), return_state=return_state)


def GRU(Wi, Wh=None, b=True, return_state=False, **init):
    """GRU(in => out) == Recurrence(GRUCell(in => out)) (recurrent.jl:685-718); `GRU((in, out))` or explicit arrays."""
    return Recurrence(GRUCell(Wi, Wh, b, **init), return_state=return_state)


# ---------------------------------------------------------------------------------- attention ---
class CausalMask:
    """What NNlib.make_causal_mask(x) stands for: key j visible to query i iff j <= i.  Passed as `mask=`."""


def make_causal_mask(x=None):
    return CausalMask()


class AttnScores:
    """The second return value of MultiHeadAttention: alpha[kv, q, heads, batch] (after dropout, as NNlib returns it),
    materialised on first use (attention.jl:128-132 returns it eagerly; here it costs nothing unless it is read).
    Materialising it under `withgradient` makes it an output of the attention call on the tape, so a loss may use it."""

    def __init__(self, q, k, lse, mask, causal, nheads, dims, extras, entry=None):
        self._args = (q, k, lse, mask, causal, nheads, dims)
        self._extras = extras          # (bias, stride_h, stride_b, p, seed, offset)
        self._entry = entry            # the tape entry of the attention call (its output list grows by alpha)
        self._val = None
        self.size = dims

    def materialize(self) -> B200Array:
        if self._val is None:
            q, k, lse, mask, causal, nheads, (Lk, Lq, H, B) = self._args
            bias, sh, sb, p, seed, off = self._extras
            ctx = context()
            a = empty((Lk, Lq, H, B))
            lib.call("fb_attn_scores_ex", ctx.handle, ctx.stream, q.ptr, k.ptr, _ptr(mask), _ptr(bias), sh, sb, p, seed, off, lse.ptr,
                     a.ptr, q.size[0], Lq, Lk, B, nheads, 1 if causal else 0)
            self._val = a
            if Tape.active and self._entry is not None:
                self._entry[0].append(a)
                Tape.tracked.add(id(a))
        return self._val


def _attention_bias(bias, Lk, Lq, H, B):
    """bias broadcastable to (kv_len, q_len, nheads, batch) (attention.jl:40-44) -> (device array, head stride, batch stride)."""
    if bias is None:
        return None, 0, 0
    if isinstance(bias, np.ndarray):
        bias = gpu(bias.astype(np.float32))
    bias = to_f32(bias)
    size = tuple(bias.size) + (1,) * (4 - bias.ndim)
    if len(size) != 4 or size[0] != Lk or size[1] != Lq or size[2] not in (1, H) or size[3] not in (1, B):
        raise DimensionMismatch(f"bias of size {bias.size} is not broadcastable to (kv_len, q_len, nheads, batch) = ({Lk}, {Lq}, {H}, {B})")
    sh = Lk * Lq if size[2] == H and H > 1 else 0
    sb = Lk * Lq * size[2] if size[3] == B and B > 1 else 0
    return bias, sh, sb


def dot_product_attention(q: B200Array, k: B200Array, v: B200Array, bias=None, nheads=1, mask=None, fdrop=None):
    """NNlib.dot_product_attention(q, k, v, bias; nheads, mask, fdrop) -> (x, alpha) for 3-d B200 arrays.  `fdrop` is a
    Dropout layer acting on the attention weights (MultiHeadAttention's `attn_drop`)."""
    low = is_bf16(q)
    q, k, v = to_f32(q), to_f32(k), to_f32(v)
    E, Lq, B = q.size
    Ev, Lk, _ = v.size
    if k.size != (E, Lk, B):
        raise DimensionMismatch(f"key of size {k.size} does not match query {q.size} / value {v.size}")
    if E % nheads or Ev % nheads:
        raise ArgumentError(f"qk_dim = {E} and v_dim = {Ev} should be divisible by nheads = {nheads}")
    causal = isinstance(mask, CausalMask)
    m = None
    if mask is not None and not causal:
        m = gpu(np.asarray(mask, dtype=np.uint8)) if isinstance(mask, np.ndarray) else mask
        if m.size != (Lk, Lq):
            raise DimensionMismatch(f"mask of size {m.size} must be (kv_len, q_len) = ({Lk}, {Lq})")
    bias_a, sh, sb = _attention_bias(bias, Lk, Lq, nheads, B)
    p, seed, off = 0.0, 0, 0
    if fdrop is not None and fdrop.p > 0 and fdrop._isactive():
        p, seed, off = fdrop.p, fdrop.seed, fdrop.next_offset(Lk * Lq * nheads * B)
    extras = (bias_a, sh, sb, p, seed, off)
    ctx = context()
    o, lse = empty((Ev, Lq, B)), empty((Lq, nheads, B))
    lib.call("fb_attn_fwd_ex", ctx.handle, ctx.stream, q.ptr, k.ptr, v.ptr, _ptr(m), _ptr(bias_a), sh, sb, p, seed, off, o.ptr, lse.ptr,
             E, Ev, Lq, Lk, B, nheads, 1 if causal else 0)
    entry = None
    if Tape.active:
        def pullback(gs):
            do = gs[0] if gs[0] is not None else zeros(o.size)
            dalpha = gs[1] if len(gs) > 1 else None
            dq, dk, dv = empty(q.size), empty(k.size), empty(v.size)
            lib.call("fb_attn_bwd_ex", ctx.handle, ctx.stream, q.ptr, k.ptr, v.ptr, _ptr(m), _ptr(bias_a), sh, sb, p, seed, off, o.ptr,
                     lse.ptr, do.ptr, _ptr(dalpha), dq.ptr, dk.ptr, dv.ptr, E, Ev, Lq, Lk, B, nheads, 1 if causal else 0)
            return [(q, dq), (k, dk), (v, dv)]

        Tape.record(o, [q, k, v], pullback)
        entry = Tape.entries[-1]
    scores = AttnScores(q, k, lse, m, causal, nheads, (Lk, Lq, nheads, B), extras, entry)
    return (to_bf16(o) if low else o), scores


class MultiHeadAttention(Layer):
    """MultiHeadAttention(dims; nheads, bias=false) = 3 input Dense + attention + output Dense (attention.jl:68-133)."""

    _fields = ("nheads", "q_proj", "k_proj", "v_proj", "attn_drop", "out_proj")
    _trainable = ("q_proj", "k_proj", "v_proj", "out_proj")

    def __init__(self, Wq, Wk=None, Wv=None, Wo=None, nheads=8, biases=None, precision="default", bias=False,
                 init=glorot_uniform, dropout_prob=0.0):
        bq = bk = bv = bo = False
        if biases is not None:
            bq, bk, bv, bo = biases
        if Wk is None:
            # MultiHeadAttention(dims; nheads, bias, init) (attention.jl:79-94): dims is an Int or
            # (in, (qkv, out)) with in = Int | (q_in, k_in, v_in) and qkv = Int | (qk, v)  (normalize_mha_dims :97-112)
            d = Wq
            if isinstance(d, (int, np.integer)):
                q_in = k_in = v_in = qk = vd = out = int(d)
            else:
                inp, (qkv, out) = d
                q_in, k_in, v_in = (inp, inp, inp) if isinstance(inp, (int, np.integer)) else inp
                qk, vd = (qkv, qkv) if isinstance(qkv, (int, np.integer)) else qkv
            if qk % nheads:
                raise ArgumentError(f"qk_dim = {qk} should be divisible by nheads = {nheads}")
            if vd % nheads:
                raise ArgumentError(f"v_dim = {vd} should be divisible by nheads = {nheads}")
            Wq, Wk, Wv, Wo = init(qk, q_in), init(qk, k_in), init(vd, v_in), init(out, vd)
            bq = bk = bv = bo = bool(bias)
        self.nheads = int(nheads)
        self.q_proj = Dense(Wq, bq, precision=precision)
        self.k_proj = Dense(Wk, bk, precision=precision)
        self.v_proj = Dense(Wv, bv, precision=precision)
        self.out_proj = Dense(Wo, bo, precision=precision)
        self.attn_drop = Dropout(float(dropout_prob))
        qk, vd = self.q_proj.weight.size[0], self.v_proj.weight.size[0]
        if qk % nheads:
            raise ArgumentError(f"qk_dim = {qk} should be divisible by nheads = {nheads}")
        if vd % nheads:
            raise ArgumentError(f"v_dim = {vd} should be divisible by nheads = {nheads}")

    def __call__(self, q_in, k_in=None, v_in=None, bias=None, mask=None):
        k_in = q_in if k_in is None else k_in
        v_in = k_in if v_in is None else v_in
        for a in (q_in, k_in, v_in):
            if a.ndim != 3:
                raise TypeError("MethodError: MultiHeadAttention expects 3-d arrays (features, len, batch)")
        q = self.q_proj(q_in)
        k = self.k_proj(k_in)
        v = self.v_proj(v_in)
        x, alpha = dot_product_attention(q, k, v, bias, nheads=self.nheads, mask=mask, fdrop=self.attn_drop)
        return self.out_proj(x), alpha


# ------------------------------------------------------------- the rest of the layer family ---
class GroupNorm(Layer):
    """GroupNorm(chs, G, λ; affine=true, eps=1f-5) (normalise.jl:440-489): every group of chs/G consecutive channels of a
    sample is normalised with its own mean and biased variance; per-channel scale γ and bias β."""

    _fields = ("G", "λ", "β", "γ", "μ", "σ2", "ε", "momentum", "affine", "track_stats", "active", "chs")
    _trainable = ("β", "γ")

    def __init__(self, chs: int, G: int, sigma="identity", affine=True, active=None, eps=1e-5, momentum=0.1):
        if chs % G != 0:
            raise ArgumentError(f"The number of groups ({G}) must divide the number of channels ({chs})")
        self.chs, self.G = int(chs), int(G)
        self.λ = _act_name(sigma)
        self.affine, self.track_stats, self.active = bool(affine), False, active
        self.ε, self.momentum = float(eps), float(momentum)
        self.β = gpu(np.zeros(chs, np.float32)) if affine else None
        self.γ = gpu(np.ones(chs, np.float32)) if affine else None
        self.μ = self.σ2 = None

    def __repr__(self):
        return f"GroupNorm({self.chs}, {self.G}, {self.λ})"

    def _groups(self):
        return self.G

    def __call__(self, x: B200Array) -> B200Array:
        N = x.ndim
        if N < 2:
            raise DimensionMismatch(f"layer {self} expects ndims(input) >= 2, but got {x}")
        _size_check(self, x, N - 1, self.chs)
        s = int(np.prod(x.size[:N - 2], dtype=np.int64)) if N > 2 else 1
        c, n, G = self.chs, x.size[-1], self._groups()
        ctx = context()
        act = lib.ACT[self.λ]
        y, mean, rstd = empty(x.size), empty((n * G,)), empty((n * G,))
        lib.call("fb_groupnorm_fwd", ctx.handle, ctx.stream, x.ptr, _ptr(self.γ), _ptr(self.β), y.ptr, mean.ptr, rstd.ptr,
                 s, c, n, G, self.ε, act)
        self._after_forward(mean, rstd, s, c, n)
        if Tape.active:
            g, b = self.γ, self.β

            def pullback(gs, x=x):
                dy = gs[0]
                dx = empty(x.size)
                dg = empty((c,)) if g is not None else None
                dbeta = empty((c,)) if b is not None else None
                lib.call("fb_groupnorm_bwd", ctx.handle, ctx.stream, x.ptr, _ptr(g), _ptr(b), mean.ptr, rstd.ptr, dy.ptr, dx.ptr,
                         _ptr(dg), _ptr(dbeta), s, c, n, G, act)
                res = [(x, dx)] if Tape.needs(x) else []
                if g is not None:
                    res += [(g, dg), (b, dbeta)]
                return res

            Tape.record(y, [x, g, b], pullback)
        return y

    def _after_forward(self, mean, rstd, s, c, n):
        pass


class InstanceNorm(GroupNorm):
    """InstanceNorm(chs, λ; affine=false, track_stats=false, eps=1f-5, momentum=0.1f0) (normalise.jl:330-393): every
    (channel, sample) slice is normalised on its own; with track_stats the running statistics are updated while
    training and used for inference."""

    def __init__(self, chs: int, sigma="identity", affine=False, track_stats=False, active=None, eps=1e-5, momentum=0.1):
        super().__init__(chs, chs, sigma, affine=affine, active=active, eps=eps, momentum=momentum)
        self.track_stats = bool(track_stats)
        self.μ = gpu(np.zeros(chs, np.float32)) if track_stats else None
        self.σ2 = gpu(np.ones(chs, np.float32)) if track_stats else None

    def __repr__(self):
        return f"InstanceNorm({self.chs}, {self.λ})"

    def _isactive(self):
        return Tape.active if self.active is None else bool(self.active)

    def __call__(self, x: B200Array) -> B200Array:
        if self.track_stats and not self._isactive():
            N = x.ndim
            _size_check(self, x, N - 1, self.chs)
            s = int(np.prod(x.size[:N - 2], dtype=np.int64)) if N > 2 else 1
            ctx = context()
            y = empty(x.size)
            lib.call("fb_batchnorm_fwd_infer", ctx.handle, ctx.stream, x.ptr, _ptr(self.γ), _ptr(self.β), self.μ.ptr, self.σ2.ptr,
                     y.ptr, s, self.chs, x.size[-1], self.ε, lib.ACT[self.λ])
            return y
        return super().__call__(x)

    def _after_forward(self, mean, rstd, s, c, n):
        if self.track_stats and self._isactive():
            ctx = context()
            lib.call("fb_instancenorm_update_stats", ctx.handle, ctx.stream, mean.ptr, rstd.ptr, self.μ.ptr, self.σ2.ptr, s, c, n,
                     self.ε, self.momentum)


class Embedding(Layer):
    """Embedding(in => out; init=randn32, padding_idx=nothing) (basic.jl:778-800): a lookup table whose columns are
    selected by 1-based integer indices of any shape; the padding column is zero and receives no gradient."""

    _fields = ("weight", "padding_idx")
    _trainable = ("weight",)

    def __init__(self, weight, padding_idx=None, init=None):
        if isinstance(weight, (tuple, list)) and len(weight) == 2 and all(isinstance(v, (int, np.integer)) for v in weight):
            from .init import randn32
            vocab, out = int(weight[0]), int(weight[1])
            weight = (init or randn32)(out, vocab)
            if padding_idx is not None:
                if not (1 <= padding_idx <= vocab):
                    raise ArgumentError(f"padding_idx={padding_idx} must be in 1:{vocab}")
                weight[:, padding_idx - 1] = 0
        self.weight = gpu(weight) if isinstance(weight, np.ndarray) else weight
        self.padding_idx = None if padding_idx is None else int(padding_idx)

    def __repr__(self):
        return f"Embedding({self.weight.size[1]} => {self.weight.size[0]})"

    def __call__(self, idx) -> B200Array:
        if isinstance(idx, (int, np.integer)):
            idx = np.array([idx], np.int32)
            scalar = True
        else:
            scalar = False
        if isinstance(idx, np.ndarray):
            if idx.size and (idx.min() < 1 or idx.max() > self.weight.size[1]):
                raise IndexError(f"BoundsError: attempt to access {self.weight.size[1]}-column embedding at index outside 1:{self.weight.size[1]}")
            idx = gpu(idx.astype(np.int32))
        out_dim, vocab = self.weight.size
        n = idx.numel()
        ctx = context()
        pad = self.padding_idx or 0
        y = empty((out_dim,) + (() if scalar else idx.size))
        lib.call("fb_embedding_fwd", ctx.handle, ctx.stream, self.weight.ptr, idx.ptr, y.ptr, out_dim, vocab, n, pad)
        if Tape.needs(self.weight):
            W = self.weight

            def pullback(gs):
                dW = empty(W.size)
                lib.call("fb_embedding_bwd", ctx.handle, ctx.stream, gs[0].ptr, idx.ptr, dW.ptr, out_dim, vocab, n, pad)
                return [(W, dW)]

            Tape.record(y, [W], pullback)
        return y


class Dropout(Layer):
    """Dropout(p; active=nothing, seed) (normalise.jl:54-92): while active, every element is zeroed with probability p and
    the rest scaled by 1 / (1 - p); inactive (test mode, or outside `withgradient` when active is None) it is the
    identity.  The mask is a counter-based function of (seed, call number, element index), so the backward pass
    regenerates it instead of storing it."""

    _fields = ("p", "active", "seed")
    _trainable = ()

    def __init__(self, p: float, active=None, seed: int = 0):
        if not (0 <= p <= 1):
            raise ArgumentError(f"Dropout expects 0 ≤ p ≤ 1, got p = {p}")
        self.p, self.active, self.seed = float(p), active, int(seed)
        self.calls = 0

    def _isactive(self):
        return Tape.active if self.active is None else bool(self.active)

    def next_offset(self, count: int) -> int:
        """Counter offset of this call's mask; successive calls take disjoint counter ranges."""
        off = self.calls
        self.calls += (count + 3) // 4
        return off

    def __call__(self, x: B200Array) -> B200Array:
        if not self._isactive() or self.p == 0.0:
            return x
        ctx = context()
        y = empty(x.size)
        off = self.next_offset(x.numel())
        lib.call("fb_dropout", ctx.handle, ctx.stream, x.ptr, y.ptr, x.numel(), self.p, self.seed, off)
        if Tape.needs(x):
            def pullback(gs):
                dx = empty(x.size)
                lib.call("fb_dropout", ctx.handle, ctx.stream, gs[0].ptr, dx.ptr, x.numel(), self.p, self.seed, off)
                return [(x, dx)]

            Tape.record(y, [x], pullback)
        return y


class RNNCell(Layer):
    """RNNCell(in => out, σ = tanh) (recurrent.jl:140-198): h' = σ.(Wi x + Wh h + b)."""

    _fields = ("σ", "Wi", "Wh", "bias")
    _trainable = ("Wi", "Wh", "bias")
    NG = 1

    def __init__(self, Wi, Wh=None, bias=True, sigma="tanh", init_kernel=glorot_uniform, init_recurrent_kernel=glorot_uniform):
        if isinstance(Wi, (tuple, list)) and len(Wi) == 2 and all(isinstance(v, (int, np.integer)) for v in Wi):
            in_dim, out = int(Wi[0]), int(Wi[1])
            Wi, Wh = init_kernel(out, in_dim), init_recurrent_kernel(out, out)
        self.Wi, self.Wh = gpu(Wi), gpu(Wh)
        self.σ = _act_name(sigma)
        if self.σ not in ("identity", "relu", "tanh", "sigmoid"):
            raise lib.FluxB200Error(-7, f"RNNCell activation {self.σ!r} has no B200 kernel (identity, relu, tanh, sigmoid)")
        rows = self.Wi.size[0]
        self.bias = zeros((rows,)) if bias is True else (False if bias in (False, None) else gpu(bias))

    @property
    def hidden(self):
        return self.Wh.size[1]

    def initialstates(self):
        return zeros((self.hidden,))


class GRUv3Cell(Layer):
    """GRUv3Cell(in => out) (recurrent.jl:765-809): like GRUCell, but the candidate state uses a separate matrix
    Wh_h̃ applied to r .* h."""

    _fields = ("Wi", "Wh", "b", "Wh_h̃")
    NG = 3

    def __init__(self, Wi, Wh=None, b=True, Wh_h=None, init_kernel=glorot_uniform, init_recurrent_kernel=glorot_uniform):
        if isinstance(Wi, (tuple, list)) and len(Wi) == 2 and all(isinstance(v, (int, np.integer)) for v in Wi):
            in_dim, out = int(Wi[0]), int(Wi[1])
            Wi, Wh, Wh_h = init_kernel(out * 3, in_dim), init_recurrent_kernel(out * 3, out), init_recurrent_kernel(out, out)
        self.Wi, self.Wh = gpu(Wi), gpu(Wh)
        setattr(self, "Wh_h̃", gpu(Wh_h))
        rows = self.Wi.size[0]
        self.b = zeros((rows,)) if b is True else (False if b in (False, None) else gpu(b))

    @property
    def Wh_h(self):
        return getattr(self, "Wh_h̃")

    @property
    def hidden(self):
        return self.Wh.size[1]

    def initialstates(self):
        return zeros((self.hidden,))


def _scan_family(rec, x: B200Array, state=None):
    """scan(cell, x, state) for RNNCell and GRUv3Cell (recurrent.jl:1-8)."""
    cell = rec.cell
    in_dim = cell.Wi.size[1]
    _size_check(cell, x, 1, in_dim)
    if x.ndim == 2:
        x3 = x.reshape(x.size[0], x.size[1], 1)
    elif x.ndim == 3:
        x3 = x
    else:
        raise DimensionMismatch(f"Recurrence expects a 2-d or 3-d input, got {x}")
    _, T, B = x3.size
    H = cell.hidden
    ctx = context()
    is_rnn = isinstance(cell, RNNCell)
    bias = cell.bias if is_rnn else cell.b
    bias = bias if bias is not False else None
    h0 = _broadcast_state(state, H, B)
    out, hT = empty((H, T, B)), empty((H, B))
    recording = Tape.active
    cache = None
    if is_rnn:
        act = lib.ACT[cell.σ]
        lib.call("fb_rnn_fwd", ctx.handle, ctx.stream, act, cell.Wi.ptr, cell.Wh.ptr, _ptr(bias), x3.ptr, _ptr(h0), out.ptr, hT.ptr,
                 in_dim, H, T, B)
    else:
        if recording:
            cache = torch.empty(max(lib.raw().fb_gruv3_cache_bytes(in_dim, H, T, B) // 4, 1), dtype=torch.float32, device=x.t.device)
        lib.call("fb_gruv3_fwd", ctx.handle, ctx.stream, cell.Wi.ptr, cell.Wh.ptr, _ptr(bias), cell.Wh_h.ptr, x3.ptr, _ptr(h0), out.ptr,
                 hT.ptr, cache.data_ptr() if cache is not None else None, in_dim, H, T, B)
    if recording:
        def pullback(gs, x3=x3):
            dout = gs[0] if gs[0] is not None else zeros(out.size)
            dhT = gs[1]
            dWi, dWh = empty(cell.Wi.size), empty(cell.Wh.size)
            db = empty(bias.size) if bias is not None else None
            dx = empty(x3.size) if Tape.needs(x3) else None
            if is_rnn:
                scratch = torch.empty(max(lib.raw().fb_rnn_cache_bytes(in_dim, H, T, B) // 4, 1), dtype=torch.float32, device=x.t.device)
                lib.call("fb_rnn_bwd", ctx.handle, ctx.stream, act, cell.Wi.ptr, cell.Wh.ptr, x3.ptr, _ptr(h0), out.ptr,
                         scratch.data_ptr(), dout.ptr, _ptr(dhT), dWi.ptr, dWh.ptr, _ptr(db), _ptr(dx), in_dim, H, T, B)
                res = [(cell.Wi, dWi), (cell.Wh, dWh)]
            else:
                dWhh = empty(cell.Wh_h.size)
                lib.call("fb_gruv3_bwd", ctx.handle, ctx.stream, cell.Wi.ptr, cell.Wh.ptr, cell.Wh_h.ptr, x3.ptr, _ptr(h0), out.ptr,
                         cache.data_ptr(), dout.ptr, _ptr(dhT), dWi.ptr, dWh.ptr, _ptr(db), dWhh.ptr, _ptr(dx), in_dim, H, T, B)
                res = [(cell.Wi, dWi), (cell.Wh, dWh), (cell.Wh_h, dWhh)]
            if bias is not None:
                res.append((bias, db))
            if dx is not None:
                res.append((x3, dx))
            return res

        ins = [x3, cell.Wi, cell.Wh, bias] + ([] if is_rnn else [cell.Wh_h])
        Tape.record([out, hT], ins, pullback)
    y = out if x.ndim == 3 else out.reshape(H, T)
    if rec.return_state:
        return y, hT
    return y


def RNN(Wi, Wh=None, bias=True, sigma="tanh", return_state=False, **init):
    """RNN(in => out, σ) == Recurrence(RNNCell(in => out, σ)) (recurrent.jl:262-300)."""
    return Recurrence(RNNCell(Wi, Wh, bias, sigma, **init), return_state=return_state)


def GRUv3(Wi, Wh=None, b=True, Wh_h=None, return_state=False, **init):
    """GRUv3(in => out) == Recurrence(GRUv3Cell(in => out)) (recurrent.jl:860-900)."""
    return Recurrence(GRUv3Cell(Wi, Wh, b, Wh_h, **init), return_state=return_state)
