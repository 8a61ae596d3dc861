"""Device context, the B200 array type, `gpu` / `cpu` movement and the reverse-mode tape.

Host-side mirror of the pieces of Flux that sit above the C ABI: a `B200Array` plays the role of
the new device array type the Julia extension dispatches on (column-major, like Julia's `Array`),
`gpu` / `cpu` mirror src/functor.jl:85, 116, and the tape stands in for Zygote: every layer call
records its pullback, `withgradient` replays them in reverse.

PyTorch is used for device memory (caching allocator) and streams only; every kernel that touches
the data is in libfluxb200.so.
"""
from __future__ import annotations

import ctypes as C
import threading

import numpy as np
import torch

from . import lib

_state = threading.local()


class Context:
    """One fb_ctx per (process, device); created lazily by `context()`."""

    def __init__(self, device: int):
        if not torch.cuda.is_available():
            raise lib.FluxB200Error(-4, "no CUDA device: fluxb200 has no CPU fallback")
        self.device = device
        torch.cuda.set_device(device)
        h = C.c_void_p()
        lib.call("fb_ctx_create", device, C.byref(h))
        self.handle = h

    @property
    def stream(self):
        return C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def set_reserved_sms(self, n: int):
        """SMs the persistent GEMM leaves free for communication kernels that run beside it (0 = none)."""
        lib.call("fb_ctx_set_reserved_sms", self.handle, int(n))

    def device_error(self) -> int:
        out = C.c_int32(0)
        lib.call("fb_device_error", self.handle, self.stream, C.byref(out))
        return out.value


def context(device: int | None = None) -> Context:
    ctx = getattr(_state, "ctx", None)
    if ctx is None or (device is not None and ctx.device != device):
        if not torch.cuda.is_available():
            raise lib.FluxB200Error(-4, "no CUDA device: fluxb200 has no CPU fallback")
        ctx = Context(torch.cuda.current_device() if device is None else device)
        _state.ctx = ctx
    return ctx


class B200Array:
    """A dense column-major Float32 (or Int32 / UInt8) array in B200 memory.

    `size` is the Julia shape; the storage is the flat torch tensor `t` whose memory order is
    Julia's (first index fastest).
    """

    __slots__ = ("t", "size", "_node", "__weakref__")

    def __init__(self, t: torch.Tensor, size):
        self.t = t
        self.size = tuple(int(s) for s in size)
        self._node = None
        assert t.is_cuda and t.is_contiguous() and t.numel() == int(np.prod(self.size, dtype=np.int64)), (t.shape, size)

    @property
    def ptr(self):
        return C.c_void_p(self.t.data_ptr())

    @property
    def ndim(self):
        return len(self.size)

    def numel(self):
        return self.t.numel()

    def reshape(self, *size):
        """Julia `reshape`: same memory, new column-major shape (no tape entry needed: identity pullback)."""
        if len(size) == 1 and isinstance(size[0], (tuple, list)):
            size = tuple(size[0])
        total = self.numel()
        size = list(size)
        if -1 in size:
            i = size.index(-1)
            rest = int(np.prod([s for s in size if s != -1], dtype=np.int64))
            size[i] = total // max(rest, 1)
        out = B200Array(self.t, size)
        if Tape.needs(self):
            Tape.record(out, [self], lambda gs, src=self: [(src, B200Array(gs[0].t, src.size))])
        return out

    def __repr__(self):
        return f"B200Array{self.size}"


def empty(size, dtype=torch.float32) -> B200Array:
    n = int(np.prod(size, dtype=np.int64)) if len(size) else 1
    return B200Array(torch.empty(n, dtype=dtype, device=f"cuda:{context().device}"), size)


def zeros(size, dtype=torch.float32) -> B200Array:
    n = int(np.prod(size, dtype=np.int64)) if len(size) else 1
    return B200Array(torch.zeros(n, dtype=dtype, device=f"cuda:{context().device}"), size)


def gpu(x):
    """Moves a numpy array (Julia-shaped) to the B200; maps over tuples / lists / dicts / layers (functor.jl:85)."""
    if isinstance(x, B200Array) or x is None or isinstance(x, (bool, int, float, str)):
        return x
    if isinstance(x, np.ndarray):
        ctx = context()
        if x.dtype == np.float64 or x.dtype == np.float16:
            x = x.astype(np.float32)
        elif x.dtype == np.int64:
            x = x.astype(np.int32)
        elif x.dtype == np.bool_:
            x = x.astype(np.uint8)
        flat = np.ascontiguousarray(x.reshape(-1, order="F"))
        t = torch.from_numpy(flat).to(f"cuda:{ctx.device}")
        return B200Array(t, x.shape)
    if isinstance(x, (tuple, list)):
        return type(x)(gpu(v) for v in x)
    if isinstance(x, dict):
        return {k: gpu(v) for k, v in x.items()}
    if hasattr(x, "_fmap"):
        return x._fmap(gpu)
    raise TypeError(f"gpu: unsupported type {type(x)}")


def cpu(x):
    """Copies back to a Julia-shaped numpy array (functor.jl:116); BFloat16 storage comes back as Float32 values."""
    if isinstance(x, B200Array):
        t = x.t.detach()
        if t.dtype == torch.bfloat16:
            t = t.float()
        return t.cpu().numpy().reshape(x.size, order="F")
    if isinstance(x, (tuple, list)):
        return type(x)(cpu(v) for v in x)
    if isinstance(x, dict):
        return {k: cpu(v) for k, v in x.items()}
    if hasattr(x, "_fmap"):
        return x._fmap(cpu)
    return x


def is_bf16(a) -> bool:
    return isinstance(a, B200Array) and a.t.dtype == torch.bfloat16


def to_bf16(a: B200Array) -> B200Array:
    """Float32 -> BFloat16 storage (round to nearest even, bit-exact with Flux._to_bf16, src/functor.jl:161-166).
    Under `withgradient` the cast is recorded: the cotangent comes back in the input's element type."""
    if a is None or a.t.dtype == torch.bfloat16:
        return a
    ctx = context()
    out = empty(a.size, torch.bfloat16)
    lib.call("fb_cast_f32_bf16", ctx.handle, ctx.stream, a.ptr, out.ptr, a.numel())
    if Tape.needs(a):
        Tape.record(out, [a], lambda gs, src=a: [(src, to_f32(gs[0]))])
    return out


def to_f32(a: B200Array) -> B200Array:
    """BFloat16 -> Float32 storage (exact)."""
    if a is None or a.t.dtype != torch.bfloat16:
        return a
    ctx = context()
    out = empty(a.size)
    lib.call("fb_cast_bf16_f32", ctx.handle, ctx.stream, a.ptr, out.ptr, a.numel())
    if Tape.needs(a):
        Tape.record(out, [a], lambda gs, src=a: [(src, to_bf16(gs[0]))])
    return out


# ------------------------------------------------------------------------------------- tape ---
class Tape:
    """Reverse-mode tape: a list of (output, inputs, pullback) recorded while `Tape.active`."""

    active = False
    entries: list = []
    tracked: set = set()
    grad_sink = None   # optional object with .buffer_for(param) -> B200Array | None and .ready(param)

    @classmethod
    def needs(cls, *arrays) -> bool:
        return cls.active and any(a is not None and (id(a) in cls.tracked) for a in arrays)

    @classmethod
    def track(cls, a: B200Array):
        cls.tracked.add(id(a))

    @classmethod
    def record(cls, out, inputs, pullback):
        """pullback(grad_out) -> list of (input_array, grad_array)."""
        if not cls.active:
            return
        outs = out if isinstance(out, (tuple, list)) else [out]
        for o in outs:
            cls.tracked.add(id(o))
            o._node = True
        cls.entries.append((outs, inputs, pullback))

    @classmethod
    def reset(cls):
        cls.entries = []
        cls.tracked = set()


def accumulate(grads: dict, keep: dict, arr: B200Array, g: B200Array):
    """grads[id(arr)] += g (tangent accumulation, Zygote's `accum`)."""
    k = id(arr)
    keep[k] = arr
    if k in grads:
        if grads[k].t.data_ptr() != g.t.data_ptr():
            ctx = context()
            if grads[k].t.dtype == torch.bfloat16:
                g = to_bf16(g)
                lib.call("fb_axpy_bf16", ctx.handle, ctx.stream, 1.0, g.ptr, grads[k].ptr, g.numel())
            else:
                lib.call("fb_axpy", ctx.handle, ctx.stream, 1.0, to_f32(g).ptr, grads[k].ptr, g.numel())
    else:
        grads[k] = g
