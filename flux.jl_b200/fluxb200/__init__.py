"""fluxb200 — host-side mirror of Flux.jl's layer API over libfluxb200.so (hand-written sm_100a CUDA).

The names follow Flux: Chain, Dense, LayerNorm, BatchNorm, LSTMCell / GRUCell / Recurrence / LSTM / GRU,
MultiHeadAttention, logitcrossentropy, withgradient, setup, update (`update!`), trainstep
(`trainstep!`), train (`train!`), gpu / cpu, and DistributedUtils.
"""
from . import lib
from .core import B200Array, Tape, context, cpu, empty, gpu, zeros
from .layers import (ArgumentError, AttnScores, BatchNorm, CausalMask, Chain, Dense, DimensionMismatch, GRU, GRUCell,
                     LSTM, LSTMCell, Layer, LayerNorm, MultiHeadAttention, Recurrence, dot_product_attention,
                     make_causal_mask, testmode, trainables, trainmode, bf16, f32)
from .train import (Adam, Descent, DomainError, GraphedGradient, GraphedTrainStep, OneHotLabels, gradient, logitcrossentropy, onehotbatch, setup, scale, sum_abs2, sum_all,
                    train, trainstep, update, withgradient)
from .init import create_bias, glorot_uniform, nfan, ones32, rand32, randn32, seed, zeros32
from . import distributed as DistributedUtils

__all__ = [n for n in dir() if not n.startswith("_")]
