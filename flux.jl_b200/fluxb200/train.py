"""Losses, `withgradient`, the Adam rule and the training step for B200 arrays.

Mirrors src/losses/functions.jl:270-273 (logitcrossentropy), src/gradient.jl:214-233
(withgradient), src/train.jl (`setup` :142-150, `trainstep!` :323-339 / `_eager_step!` :375-379,
`train!` :198-253) and the Adam rule whose arithmetic the reference states in
src/optimise/optimisers.jl:171-184.
"""
from __future__ import annotations

import ctypes as C
import math

import numpy as np
import torch

from . import lib
from .core import B200Array, Tape, accumulate, context, empty, gpu, to_bf16, to_f32, zeros
from .layers import DimensionMismatch, Layer, trainables


class DomainError(ArithmeticError):
    pass


# ------------------------------------------------------------------------------------- losses ---
def logitcrossentropy(yhat: B200Array, y, dims=1, agg="mean") -> B200Array:
    """Flux.logitcrossentropy(ŷ, y): mean over the batch of -sum(y .* logsoftmax(ŷ; dims=1); dims=1).

    `y` is either a dense target array of the same size as ŷ or a `OneHotLabels` (1-based integer labels,
    what `onehotbatch(labels, 1:C)` stands for)."""
    if dims != 1 or agg != "mean":
        raise lib.FluxB200Error(-7, "logitcrossentropy on B200 arrays supports dims=1, agg=mean")
    yhat = to_f32(yhat)
    c = yhat.size[0]
    n = yhat.numel() // c
    ctx = context()
    loss = empty(())
    recording = Tape.needs(yhat)
    dyhat = empty(yhat.size) if recording else None
    if isinstance(y, OneHotLabels):
        if y.nclasses != c or y.labels.numel() != n:
            raise DimensionMismatch(f"loss function expects size(ŷ) = {yhat.size} to match size(y) = {(y.nclasses, y.labels.numel())}")
        lib.call("fb_logitcrossentropy_labels", ctx.handle, ctx.stream, yhat.ptr, y.labels.ptr, loss.ptr,
                 dyhat.ptr if dyhat else None, c, n, 1.0)
    else:
        if y.size != yhat.size:
            raise DimensionMismatch(f"loss function expects size(ŷ) = {yhat.size} to match size(y) = {y.size}")
        lib.call("fb_logitcrossentropy_dense", ctx.handle, ctx.stream, yhat.ptr, y.ptr, loss.ptr,
                 dyhat.ptr if dyhat else None, c, n, 1.0)
    if recording:
        def pullback(gs):
            g = gs[0]   # cotangent of the scalar loss (device scalar); 1 for a top-level loss
            if g is not None and not getattr(g, "_is_one", False):
                s = float(g.t.item())
                lib.call("fb_scale", ctx.handle, ctx.stream, dyhat.ptr, s, dyhat.ptr, dyhat.numel())
            return [(yhat, dyhat)]

        Tape.record(loss, [yhat], pullback)
    return loss


class OneHotLabels:
    """onehotbatch(labels, 1:nclasses) kept as the integer labels (1-based) on the device."""

    def __init__(self, labels, nclasses: int):
        if isinstance(labels, np.ndarray):
            labels = gpu(labels.astype(np.int32))
        self.labels = labels
        self.nclasses = int(nclasses)


def onehotbatch(labels, nclasses):
    return OneHotLabels(np.asarray(labels), nclasses)


def sum_abs2(y: B200Array) -> B200Array:
    """sum(abs2, y); its pullback is the cotangent 2y."""
    y = to_f32(y)
    ctx = context()
    out = empty(())
    lib.call("fb_sumsq", ctx.handle, ctx.stream, y.ptr, y.numel(), out.ptr)
    if Tape.needs(y):
        def pullback(gs):
            g = gs[0]
            s = 2.0 if (g is None or getattr(g, "_is_one", False)) else 2.0 * float(g.t.item())
            dy = empty(y.size)
            lib.call("fb_scale", ctx.handle, ctx.stream, y.ptr, s, dy.ptr, y.numel())
            return [(y, dy)]

        Tape.record(out, [y], pullback)
    return out


def sum_all(y: B200Array) -> B200Array:
    """sum(y); its pullback fills the cotangent."""
    y = to_f32(y)
    ctx = context()
    out = empty(())
    lib.call("fb_sum", ctx.handle, ctx.stream, y.ptr, y.numel(), out.ptr)
    if Tape.needs(y):
        def pullback(gs):
            g = gs[0]
            s = 1.0 if (g is None or getattr(g, "_is_one", False)) else float(g.t.item())
            dy = empty(y.size)
            lib.call("fb_fill", ctx.handle, ctx.stream, dy.ptr, s, y.numel())
            return [(y, dy)]

        Tape.record(out, [y], pullback)
    return out


def add(a: B200Array, b: B200Array) -> B200Array:
    """a + b for two arrays of one size (e.g. two loss terms); the cotangent goes to both."""
    a, b = to_f32(a), to_f32(b)
    if a.size != b.size:
        raise DimensionMismatch(f"dimensions must match: a has dims {a.size}, b has dims {b.size}")
    ctx = context()
    out = B200Array(a.t.clone(), a.size)
    lib.call("fb_axpy", ctx.handle, ctx.stream, 1.0, b.ptr, out.ptr, out.numel())
    if Tape.needs(a, b):
        Tape.record(out, [a, b], lambda gs: [(a, gs[0]), (b, gs[0])])
    return out


def scale(c: float, a: B200Array) -> B200Array:
    """c * a for a Python scalar c."""
    ctx = context()
    out = empty(a.size)
    lib.call("fb_scale", ctx.handle, ctx.stream, a.ptr, float(c), out.ptr, a.numel())
    if Tape.needs(a):
        def pullback(gs):
            g = gs[0]
            da = empty(a.size)
            if getattr(g, "_is_one", False):
                lib.call("fb_fill", ctx.handle, ctx.stream, da.ptr, float(c), a.numel())
            else:
                lib.call("fb_scale", ctx.handle, ctx.stream, g.ptr, float(c), da.ptr, a.numel())
            return [(a, da)]

        Tape.record(out, [a], pullback)
    return out


# ----------------------------------------------------------------------------------- gradient ---
def _grad_tree(obj, grads: dict):
    """Gradient with the model's structure: dict of field name -> subtree / array / None
    (src/gradient.jl:112: `(layers = ((weight = ..., bias = ..., σ = nothing), ...),)`)."""
    if isinstance(obj, B200Array):
        return grads.get(id(obj))
    if isinstance(obj, (tuple, list)):
        return tuple(_grad_tree(v, grads) for v in obj)
    if isinstance(obj, Layer):
        return {name: _grad_tree(getattr(obj, name), grads) for name in obj._fields}
    return None


def _withgradient_device(f, model, grad_sink=None):
    """Forward + reverse sweep without any device -> host read: returns (loss B200Array, aux, grad_tree)."""
    assert not Tape.active, "nested withgradient is not supported"
    Tape.reset()
    Tape.active = True
    Tape.grad_sink = grad_sink
    params = trainables(model)
    for p in params:
        Tape.track(p)
    try:
        out = f(model)
        aux = None
        loss = out
        if isinstance(out, tuple):
            loss, aux = out[0], out[1:]
        if not isinstance(loss, B200Array) or loss.numel() != 1:
            raise TypeError("withgradient: the function must return a scalar B200Array")
        if grad_sink is not None and hasattr(grad_sink, "set_loss"):
            grad_sink.set_loss(loss)
        if grad_sink is not None and hasattr(grad_sink, "expect_uses"):
            # a parameter used by several recorded calls receives several contributions (Zygote's `accum`)
            pid = {id(p) for p in params}
            counts: dict = {}
            for _, inputs, _ in Tape.entries:
                for a in inputs:
                    if a is not None and id(a) in pid:
                        counts[id(a)] = counts.get(id(a), 0) + 1
            grad_sink.expect_uses(counts)
        grads: dict = {}
        keep: dict = {}
        grads[id(loss)] = _One(B200Array(torch.ones(1, device=loss.t.device), ()))
        keep[id(loss)] = loss
        # gradient averaging runs beside the reverse sweep: leave it the SMs it needs
        reserve = int(getattr(grad_sink, "reserved_sms", 0) or 0)
        if reserve:
            context().set_reserved_sms(reserve)
        for outs, inputs, pullback in reversed(Tape.entries):
            gs = [grads.get(id(o)) for o in outs]
            if all(g is None for g in gs):
                continue
            for arr, g in pullback(gs):
                if arr is None or g is None:
                    continue
                accumulate(grads, keep, arr, g)
                if grad_sink is not None:
                    grad_sink.ready(arr)
        tree = _grad_tree(model, grads)
    finally:
        if int(getattr(grad_sink, "reserved_sms", 0) or 0):
            context().set_reserved_sms(0)
        Tape.active = False
        Tape.grad_sink = None
        Tape.reset()
    return loss, aux, tree


def withgradient(f, model, grad_sink=None):
    """Flux.withgradient(m -> loss, model): returns (loss_value, (grad_tree,)).

    `f(model)` must return a scalar B200Array (or a tuple whose first element is one, like Zygote's
    auxiliary-output form).  The loss value comes back as a Python float (one device -> host read,
    the same sync `_eager_step!` pays at src/train.jl:377).
    """
    loss, aux, tree = _withgradient_device(f, model, grad_sink)
    val = float(loss.t.item())
    if aux is not None:
        return (val,) + tuple(aux), (tree,)
    return val, (tree,)


class _One(B200Array):
    """Cotangent 1 of the top-level loss."""

    __slots__ = ("_is_one",)

    def __init__(self, a: B200Array):
        super().__init__(a.t, a.size)
        self._is_one = True


def gradient(f, model):
    return withgradient(f, model)[1]


# --------------------------------------------------------------------------------------- Adam ---
class Adam:
    """Optimisers.Adam(η = 0.001, β = (0.9, 0.999), ϵ = 1e-8)."""

    def __init__(self, eta=1e-3, beta=(0.9, 0.999), epsilon=1e-8):
        self.eta, self.beta, self.epsilon = float(eta), (float(beta[0]), float(beta[1])), float(epsilon)


class Descent:
    """Optimisers.Descent(η): x .-= η .* dx (used by the reference's train tests)."""

    def __init__(self, eta=0.1):
        self.eta = float(eta)


class Leaf:
    """Optimisers.Leaf(rule, state): state = (m, v, (β1ᵗ, β2ᵗ)) for Adam."""

    def __init__(self, rule, param: B200Array):
        self.rule = rule
        # a BFloat16 parameter is updated through a Float32 master copy (the step eta * m / sqrt(v) is usually below
        # half a bf16 ulp of the weight, so updating the bf16 value directly would lose it)
        self.master = to_f32(param) if param.t.dtype == torch.bfloat16 else None
        if isinstance(rule, Adam):
            self.state = [zeros(param.size), zeros(param.size), (rule.beta[0], rule.beta[1])]
        else:
            self.state = None


class OptState:
    def __init__(self, rule, model):
        self.rule = rule
        self.params = trainables(model)
        if len({id(p) for p in self.params}) != len(self.params):
            pass  # tied weights share one leaf
        self.leaves = {}
        for p in self.params:
            if id(p) not in self.leaves:
                self.leaves[id(p)] = Leaf(rule, p)


def setup(rule, model) -> OptState:
    """Flux.setup(rule, model) (src/train.jl:142-150): one Leaf per trainable array."""
    inner = rule.opt if isinstance(rule, DistributedOptimizerBase) else rule
    if not isinstance(inner, (Adam, Descent)):
        raise lib.FluxB200Error(-7, f"optimiser rule {type(inner).__name__} has no B200 kernel")
    st = OptState(inner, model)
    st.outer = rule
    return st


class DistributedOptimizerBase:
    """Marker base so `setup` can unwrap DistributedUtils.DistributedOptimizer without a circular import."""
    opt = None
    buckets = None

    def all_finite(self, loss_value: float) -> bool:
        return math.isfinite(loss_value)


def _flat_grads(model, tree, out: dict):
    if isinstance(model, B200Array):
        if tree is not None:
            out[id(model)] = tree
    elif isinstance(model, (tuple, list)):
        for m, t in zip(model, tree):
            _flat_grads(m, t, out)
    elif isinstance(model, Layer) and tree is not None:
        for name in model.trainable_fields():
            _flat_grads(getattr(model, name), tree.get(name), out)


def update(opt_state: OptState, model, grad_tree):
    """Optimisers.update!(opt_state, model, grads) (src/train.jl:425): in-place, multi-tensor."""
    gmap: dict = {}
    _flat_grads(model, grad_tree, gmap)
    outer = getattr(opt_state, "outer", None)
    if isinstance(outer, DistributedOptimizerBase):
        outer.average_gradients(opt_state, gmap)
    ctx = context()
    rule = opt_state.rule
    ps = [p for p in opt_state.params if id(p) in gmap]
    seen = set()
    ps = [p for p in ps if not (id(p) in seen or seen.add(id(p)))]
    if not ps:
        return opt_state, model
    # BFloat16 parameters: the rule runs on the Float32 master copy with the gradient widened to Float32; the
    # parameter is the master rounded back
    low = [p for p in ps if opt_state.leaves[id(p)].master is not None]
    wmap = {id(p): (opt_state.leaves[id(p)].master if opt_state.leaves[id(p)].master is not None else p) for p in ps}
    gmap = {k: to_f32(g) for k, g in gmap.items()}
    if isinstance(rule, Descent):
        for p in ps:
            lib.call("fb_axpy", ctx.handle, ctx.stream, -rule.eta, gmap[id(p)].ptr, wmap[id(p)].ptr, p.numel())
        _write_back(low, wmap)
        return opt_state, model
    # leaves share (β1ᵗ, β2ᵗ) when they have seen the same number of steps: group by that pair
    groups: dict = {}
    for p in ps:
        groups.setdefault(opt_state.leaves[id(p)].state[2], []).append(p)
    for (b1t, b2t), plist in groups.items():
        k = len(plist)
        arr_t = C.c_void_p * k
        w = arr_t(*[wmap[id(p)].t.data_ptr() for p in plist])
        g = arr_t(*[gmap[id(p)].t.data_ptr() for p in plist])
        m = arr_t(*[opt_state.leaves[id(p)].state[0].t.data_ptr() for p in plist])
        v = arr_t(*[opt_state.leaves[id(p)].state[1].t.data_ptr() for p in plist])
        cnt = (C.c_int64 * k)(*[p.numel() for p in plist])
        lib.call("fb_adam_step", ctx.handle, ctx.stream, k, w, g, m, v, cnt, rule.eta, rule.beta[0], rule.beta[1],
                 rule.epsilon, b1t, b2t, 1.0)
        f32 = np.float32
        nb = (float(f32(b1t) * f32(rule.beta[0])), float(f32(b2t) * f32(rule.beta[1])))
        for p in plist:
            opt_state.leaves[id(p)].state[2] = nb
    _write_back(low, wmap)
    return opt_state, model


def _write_back(low, wmap):
    ctx = context()
    for p in low:
        lib.call("fb_cast_f32_bf16", ctx.handle, ctx.stream, wmap[id(p)].ptr, p.ptr, p.numel())


def trainstep(loss, model, batch, opt_state):
    """Flux.trainstep!(loss, model, batch, opt_state) (src/train.jl:323-339, 375-379): returns the
    pre-update loss; a non-finite loss skips the update."""
    if not isinstance(batch, tuple):
        batch = (batch,)
    outer = getattr(opt_state, "outer", None)
    sink = getattr(outer, "buckets", None)
    if hasattr(outer, "check_async_error"):
        outer.check_async_error()
    if sink is not None:
        sink.begin_step()
    l, gs = withgradient(lambda m: loss(m, *batch), model, grad_sink=sink)
    lv = l[0] if isinstance(l, tuple) else l
    finite = outer.all_finite(lv) if isinstance(outer, DistributedOptimizerBase) else math.isfinite(lv)
    if finite:
        update(opt_state, model, gs[0])
    elif sink is not None:
        sink.finish()   # the collectives already started must be matched on every worker
    _raise_on_device_error()
    return l


def _raise_on_device_error():
    """A kernel whose bounded wait ran out records a code in the context's device error word and leaves its work
    undone; later persistent launches return early while the word is set.  Reading the word clears it."""
    code = context().device_error()
    if code != 0:
        raise lib.FluxB200Error(-6, f"a kernel gave up waiting (device error code {code}); the results of this step are invalid")


def train(loss, model, data, opt_state):
    """Flux.train!(loss, model, data, opt_state) (src/train.jl:198-253): stops with DomainError on a
    non-finite loss, as the reference does."""
    from .layers import trainmode
    trainmode(model)
    for i, batch in enumerate(data):
        l = trainstep(loss, model, batch, opt_state)
        lv = l[0] if isinstance(l, tuple) else l
        if not math.isfinite(lv):
            raise DomainError(f"Loss is {lv} on data item {i + 1}, stopping training")


# ------------------------------------------------------------------ one-launch train step ---
def _clone_static(b):
    if isinstance(b, B200Array):
        return B200Array(b.t.clone(), b.size)
    if isinstance(b, OneHotLabels):
        return OneHotLabels(B200Array(b.labels.t.clone(), b.labels.size), b.nclasses)
    return b


def _copy_into(dst, src):
    if isinstance(dst, B200Array):
        t = src.t if isinstance(src, B200Array) else src
        dst.t.copy_(t, non_blocking=True)
    elif isinstance(dst, OneHotLabels):
        t = src.labels.t if isinstance(src, OneHotLabels) else src
        dst.labels.t.copy_(t, non_blocking=True)


class GraphedGradient:
    """`withgradient(f, model)` for fixed input buffers as ONE CUDA-graph launch (forward + reverse sweep).

    `f(model)` must close over device arrays that are updated in place between calls.  `graph()` replays the captured
    launch sequence and returns the loss array (device scalar) and the gradient tree, whose arrays are the same
    buffers on every call.  BatchNorm running statistics advance on every replay, as they would in eager calls.
    (Recurrent layers run one launch per time step inside a captured step: a cooperative launch cannot be recorded.)"""

    def __init__(self, f, model):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            _withgradient_device(f, model)          # warm-up: grows the scratch arena and torch's pools
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.loss, _, self.tree = _withgradient_device(f, model)

    def __call__(self):
        self.graph.replay()
        return self.loss, self.tree


class GraphedTrainStep:
    """`trainstep!` for a fixed batch shape as ONE CUDA-graph launch: forward, reverse sweep, gradient averaging
    (when `opt_state` wraps a DistributedOptimizer) and the Adam update are captured once and replayed.

    This is the device-specific train-step hook Flux already has a slot for (src/train.jl:335-339; the Reactant
    extension compiles the step per batch shape, ext/FluxReactantExt.jl:147-152).  Semantics follow `_eager_step!`
    (src/train.jl:375-379): the returned loss is the pre-update loss, and a non-finite loss leaves parameters and
    optimiser state untouched (the captured Adam kernels read the loss on the device and skip themselves).

    `step(*batch)` accepts B200 arrays / OneHotLabels, or pinned host tensors of the same sizes (copied into the
    step's static input buffers on the current stream).
    """

    error_poll_every = 16   # the device error word is read back every this many steps (one 4-byte copy)

    def __init__(self, loss, model, opt_state, example_batch, grad_sink=None, shard_optimizer=False, defer_gather=False):
        from .layers import BatchNorm, _walk
        if not isinstance(example_batch, tuple):
            example_batch = (example_batch,)
        rule = opt_state.rule
        if not isinstance(rule, Adam):
            raise lib.FluxB200Error(-7, "GraphedTrainStep supports the Adam rule")
        if any(leaf.master is not None for leaf in opt_state.leaves.values()):
            raise lib.FluxB200Error(-7, "GraphedTrainStep supports Float32 parameters; use trainstep for a bf16 model")
        self.model, self.opt_state, self.sink = model, opt_state, grad_sink
        self.static = tuple(_clone_static(b) for b in example_batch)
        self._stage = self._copy_stream = self._staged_ev = self._consumed_ev = None
        self._has_prefetch = False
        self.params = [p for p in opt_state.params]
        seen = set()
        self.params = [p for p in self.params if not (id(p) in seen or seen.add(id(p)))]
        bts = {opt_state.leaves[id(p)].state[2] for p in self.params}
        if len(bts) != 1:
            raise lib.FluxB200Error(-7, "GraphedTrainStep needs all leaves at the same step count")
        self.bt = torch.tensor(list(bts.pop()), dtype=torch.float32, device=self.params[0].t.device)
        ctx = context()
        fn = lambda m: loss(m, *self.static)
        # warm-up outside the graph: grows the library's scratch arena and torch's pools; running statistics of
        # BatchNorm layers are put back afterwards so that the warm-up leaves no trace
        bns = [l for l in _walk(model) if isinstance(l, BatchNorm) and l.track_stats]
        saved = [(l.μ.t.clone(), l.σ2.t.clone()) for l in bns]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            if grad_sink is not None:
                grad_sink.begin_step()
            _withgradient_device(fn, model, grad_sink)
            if grad_sink is not None:
                grad_sink.finish()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        for l, (mu, var) in zip(bns, saved):
            l.μ.t.copy_(mu)
            l.σ2.t.copy_(var)
        # sharded optimiser: the sink's bucket launches carry reduce-scatter + Adam on this rank's block + all-gather
        self.sharded = bool(shard_optimizer and grad_sink is not None and hasattr(grad_sink, "shard_optimizer")
                            and all(id(p) in grad_sink.views for p in self.params)
                            and grad_sink.shard_optimizer(opt_state, self.bt))
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            if grad_sink is not None:
                grad_sink.begin_step()
                grad_sink.armed = self.sharded
                # deferred gathers need every layer of the model to wait for its parameters: Dense and LayerNorm do
                if self.sharded and defer_gather and getattr(grad_sink, "peer", None) is not None and self._only_waiting_layers(model):
                    grad_sink.defer_gather = True
                    grad_sink.start_gathers()
            try:
                loss_arr, _, tree = _withgradient_device(fn, model, grad_sink)
                gmap: dict = {}
                _flat_grads(model, tree, gmap)
                outer = getattr(opt_state, "outer", None)
                if isinstance(outer, DistributedOptimizerBase):
                    outer.average_gradients(opt_state, gmap)
                elif self.sharded:
                    grad_sink.finish()
            finally:
                if grad_sink is not None:
                    grad_sink.armed = False
            ps = [p for p in self.params if id(p) in gmap]
            c = context()
            if not self.sharded:
                k = len(ps)
                arr_t = C.c_void_p * k
                self._tables = (arr_t(*[p.t.data_ptr() for p in ps]), arr_t(*[gmap[id(p)].t.data_ptr() for p in ps]),
                                arr_t(*[opt_state.leaves[id(p)].state[0].t.data_ptr() for p in ps]),
                                arr_t(*[opt_state.leaves[id(p)].state[1].t.data_ptr() for p in ps]),
                                (C.c_int64 * k)(*[p.numel() for p in ps]))
            # with several workers the guard is the sum of all workers' losses: every rank takes the same decision
            guard = getattr(grad_sink, "guard", None) or loss_arr
            if not self.sharded:
                lib.call("fb_adam_step_dev", c.handle, c.stream, k, *self._tables, rule.eta, rule.beta[0], rule.beta[1],
                         rule.epsilon, C.c_void_p(self.bt.data_ptr()), guard.ptr, 1.0)
            lib.call("fb_adam_advance", c.handle, c.stream, C.c_void_p(self.bt.data_ptr()), rule.beta[0], rule.beta[1],
                     guard.ptr)
            self._keep = (loss_arr, tree, gmap, guard)
        self.loss_arr = loss_arr
        self.guard_arr = guard
        self._updated = ps

    @staticmethod
    def _only_waiting_layers(model):
        from .layers import Chain, Dense, LayerNorm, _walk
        return all(isinstance(l, (Chain, Dense, LayerNorm, LayerNorm._Scale)) for l in _walk(model))

    def sync_params(self):
        """With deferred gathers a rank's parameters are complete only after the next step has started; call this
        before reading them (checkpoint, evaluation) outside a step."""
        if self.sink is not None and hasattr(self.sink, "sync_params"):
            self.sink.sync_params()

    def prefetch(self, *batch):
        """Starts copying the NEXT step's inputs (pinned host tensors, or device arrays) into staging buffers on a copy
        stream, so that the transfer runs beside the step that is executing; `step()` without arguments then uses them."""
        if self._stage is None:
            self._stage = tuple(_clone_static(b) for b in self.static)
            self._copy_stream = torch.cuda.Stream()
            self._staged_ev = torch.cuda.Event()
        if self._consumed_ev is not None:
            self._copy_stream.wait_event(self._consumed_ev)   # the previous batch must have left the staging buffers
        with torch.cuda.stream(self._copy_stream):
            for dst, src in zip(self._stage, batch):
                _copy_into(dst, src)
            self._staged_ev.record(self._copy_stream)
        self._has_prefetch = True

    def __call__(self, *batch, prefetch=None):
        """One train step.  `step(x, y)` copies the batch into the step's static buffers first; `step()` takes the batch
        handed to `prefetch` earlier; `prefetch=(x, y)` starts the transfer of the following batch right after this
        step has been launched (before the loss is read back)."""
        cur = torch.cuda.current_stream()
        if not batch:
            if not self._has_prefetch:
                raise lib.FluxB200Error(-1, "GraphedTrainStep: step() without arguments needs a prefetched batch")
            cur.wait_event(self._staged_ev)
            for dst, src in zip(self.static, self._stage):
                _copy_into(dst, src)
            self._consumed_ev = torch.cuda.Event()
            self._consumed_ev.record(cur)
            self._has_prefetch = False
        else:
            for dst, src in zip(self.static, batch):
                if src is not dst:
                    _copy_into(dst, src)
        self.graph.replay()
        if prefetch is not None:
            self.prefetch(*prefetch)
        lv = float(self.loss_arr.t.item())
        gv = lv if self.guard_arr is self.loss_arr else float(self.guard_arr.t.item())
        self._calls = getattr(self, "_calls", 0) + 1
        if self._calls % self.error_poll_every == 0:
            _raise_on_device_error()
        if math.isfinite(gv):
            rule = self.opt_state.rule
            f32 = np.float32
            for p in self._updated:
                st = self.opt_state.leaves[id(p)].state
                st[2] = (float(f32(st[2][0]) * f32(rule.beta[0])), float(f32(st[2][1]) * f32(rule.beta[1])))
        return lv
