"""fluxb200 — host-side mirror of Flux.jl's layer API over libfluxb200.so (hand-written sm_100a CUDA).

The names follow Flux: Chain, Dense, LayerNorm, BatchNorm, LSTMCell / GRUCell / Recurrence / LSTM / GRU,
MultiHeadAttention, logitcrossentropy, withgradient, setup, update (`update!`), trainstep
(`trainstep!`), train (`train!`), gpu / cpu, and DistributedUtils.
"""
from . import lib
from .core import B200Array, Tape, context, cpu, empty, gpu, zeros
from .layers import (ArgumentError, AttnScores, BatchNorm, CausalMask, Chain, Dense, DimensionMismatch, Dropout, Embedding, GRU,
                     GRUCell, GRUv3, GRUv3Cell, GroupNorm, InstanceNorm, LSTM, LSTMCell, Layer, LayerNorm, MultiHeadAttention,
                     RNN, RNNCell, Recurrence, dot_product_attention, make_causal_mask, testmode, trainables, trainmode, bf16,
                     f32)
from .train import (add, Adam, Descent, DomainError, GraphedGradient, GraphedTrainStep, OneHotLabels, gradient, logitcrossentropy, onehotbatch, setup, scale, sum_abs2, sum_all,
                    train, trainstep, update, withgradient)
from .init import create_bias, glorot_uniform, nfan, ones32, rand32, randn32, seed, zeros32
from .loading import load_checkpoint, load_opt_state, loadmodel, opt_state, save_checkpoint, state
from .data import DataLoader, DeviceIterator
from . import distributed as DistributedUtils

__all__ = [n for n in dir() if not n.startswith("_")]
