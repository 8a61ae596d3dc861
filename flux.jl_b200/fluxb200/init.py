"""Host-side parameter initialisers, mirroring src/utils.jl: `nfan` (:27-31), `glorot_uniform` (:81-86),
`create_bias` (:537-543), `zeros32` / `ones32` / `rand32` / `randn32` (:497-530).

Parameters are created on the host in Float32 and moved to the B200 by the layer constructors.  The random stream is
numpy's PCG64 (`seed(n)` plays the role of `Random.seed!(n)`); Julia's own generator cannot be reproduced without
Julia, so a model that must match a Flux model bit for bit takes explicit arrays, as `Dense(W, b, σ)` allows.
"""
from __future__ import annotations

import numpy as np

_rng = np.random.default_rng()


def seed(n: int) -> None:
    """Random.seed!(n) for the initialisers of this package."""
    global _rng
    _rng = np.random.default_rng(n)


def default_rng() -> np.random.Generator:
    return _rng


def nfan(*dims):
    """(fan_in, fan_out) of an array of size `dims` (utils.jl:27-31)."""
    if len(dims) == 1 and isinstance(dims[0], (tuple, list)):
        dims = tuple(dims[0])
    if len(dims) == 0:
        return 1, 1
    if len(dims) == 1:
        return 1, dims[0]                 # a vector is treated as an n x 1 matrix
    if len(dims) == 2:
        return dims[1], dims[0]           # Dense kernels: (out, in)
    rf = int(np.prod(dims[:-2]))          # convolution kernels
    return rf * dims[-2], rf * dims[-1]


def _split_rng(args):
    if args and isinstance(args[0], np.random.Generator):
        return args[0], args[1:]
    return _rng, args


def glorot_uniform(*args, gain: float = 1.0):
    """glorot_uniform([rng], dims...; gain = 1): (rand(Float32, dims...) .- 0.5f0) .* gain * sqrt(24 / (fan_in + fan_out))
    (utils.jl:81-84).  With no dims it returns the initialiser bound to that rng / gain (utils.jl:86)."""
    rng, dims = _split_rng(args)
    if not dims:
        return lambda *d, **kw: glorot_uniform(rng, *d, **{"gain": gain, **kw})
    scale = np.float32(gain) * np.float32(np.sqrt(np.float32(24.0) / np.float32(sum(nfan(*dims)))))
    return ((rng.random(dims, dtype=np.float32) - np.float32(0.5)) * scale).astype(np.float32)


def zeros32(*dims):
    return np.zeros(dims, np.float32)


def ones32(*dims):
    return np.ones(dims, np.float32)


def rand32(*args):
    rng, dims = _split_rng(args)
    return rng.random(dims, dtype=np.float32)


def randn32(*args):
    rng, dims = _split_rng(args)
    return rng.standard_normal(dims, dtype=np.float32)


def create_bias(weights, bias, *dims):
    """create_bias(weights, bias, dims...) (utils.jl:537-543): `True` -> zeros, `False` -> False, an array is checked
    against `dims` and converted to Float32."""
    if bias is True:
        return np.zeros(dims, np.float32)
    if bias is False or bias is None:
        return False
    b = np.asarray(bias)
    if tuple(b.shape) != tuple(dims):
        from .layers import DimensionMismatch
        raise DimensionMismatch(f"expected bias of size {tuple(dims)}, got size {tuple(b.shape)}")
    return b.astype(np.float32)
