"""ctypes binding of libfluxb200.so: one Python prototype per entry point of include/fluxb200.h.

The library is the product; this module only loads it and checks status codes.  There is no
CPU fallback: if the shared library is missing, importing this module raises, and every compute
call fails with FB_ERR_CUDA when no B200 is present.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfluxb200.so")

FB_OK = 0
ERR_NAMES = {-1: "FB_ERR_INVALID_ARG", -2: "FB_ERR_SHAPE", -3: "FB_ERR_ALLOC", -4: "FB_ERR_CUDA",
             -5: "FB_ERR_NCCL", -6: "FB_ERR_TIMEOUT", -7: "FB_ERR_UNSUPPORTED"}

ACT = {"identity": 0, "relu": 1, "tanh": 2, "sigmoid": 3, "gelu_tanh": 4, "gelu": 4, "gelu_erf": 5}
# "bf16": operands hold bf16 values (see fluxb200.bf16); the GEMM is the single TF32 pass, exact for such operands
PREC = {"default": 0, "fp32_simt": 1, "3xtf32": 2, "tf32": 3, "3xtf32_pair": 4, "bf16": 3}
OP = {"+": 0, "sum": 0, "avg": 1}
UNIQUE_ID_BYTES = 128


class FluxB200Error(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"{ERR_NAMES.get(code, code)}: {msg}")
        self.code = code


if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python flux.jl_b200/build.py` (nvcc, sm_100a). "
        "fluxb200 has no CPU fallback.")

_lib = C.CDLL(LIB_PATH)

_p, _i32, _i64, _f = C.c_void_p, C.c_int32, C.c_int64, C.c_float

# name -> (restype, argtypes); mirrors include/fluxb200.h declaration by declaration
PROTOTYPES = {
    "fb_version": (_i32, []),
    "fb_kernel_launches": (_i64, []),
    "fb_ctx_create": (_i32, [_i32, C.POINTER(_p)]),
    "fb_ctx_set_reserved_sms": (_i32, [_p, _i32]),
    "fb_ctx_destroy": (_i32, [_p]),
    "fb_last_error": (C.c_char_p, []),
    "fb_malloc": (_i32, [_p, _i64, C.POINTER(_p)]),
    "fb_free": (_i32, [_p, _p]),
    "fb_memcpy_h2d": (_i32, [_p, _p, _p, _p, _i64]),
    "fb_memcpy_d2h": (_i32, [_p, _p, _p, _p, _i64]),
    "fb_memcpy_d2d": (_i32, [_p, _p, _p, _p, _i64]),
    "fb_memset": (_i32, [_p, _p, _p, _i32, _i64]),
    "fb_sync": (_i32, [_p, _p]),
    "fb_device_error": (_i32, [_p, _p, C.POINTER(_i32)]),
    "fb_selftest_bounded_wait": (_i32, [_p, _p, _i32]),
    "fb_gemm_f32": (_i32, [_p, _p, _i32, _i32, _i64, _i64, _i64, _p, _i64, _p, _i64, _p, _i64, _i32, _i32]),
    "fb_dense_fwd": (_i32, [_p, _p, _i32, _i32, _p, _p, _p, _p, _p, _i64, _i64, _i64]),
    "fb_dense_bwd": (_i32, [_p, _p, _i32, _i32, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64]),
    "fb_gemm_bf16": (_i32, [_p, _p, _i32, _i32, _i64, _i64, _i64, _p, _i64, _p, _i64, _p, _i64, _i32, _i32]),
    "fb_axpy_bf16": (_i32, [_p, _p, _f, _p, _p, _i64]),
    "fb_dense_fwd_bf16": (_i32, [_p, _p, _i32, _p, _p, _p, _p, _p, _i64, _i64, _i64]),
    "fb_dense_bwd_bf16": (_i32, [_p, _p, _i32, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64]),
    "fb_layernorm_fwd": (_i32, [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _f, _i32]),
    "fb_layernorm_bwd": (_i32, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i32]),
    "fb_layernorm_bwd_noalloc": (_i32, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i32]),
    "fb_batchnorm_fwd_train": (_i32, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _f, _f, _i32, _i32]),
    "fb_batchnorm_fwd_infer": (_i32, [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _f, _i32]),
    "fb_batchnorm_bwd": (_i32, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i32]),
    "fb_groupnorm_fwd": (_i32, [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _f, _i32]),
    "fb_groupnorm_bwd": (_i32, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i32]),
    "fb_instancenorm_update_stats": (_i32, [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _f, _f]),
    "fb_embedding_fwd": (_i32, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i32]),
    "fb_embedding_bwd": (_i32, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i32]),
    "fb_dropout": (_i32, [_p, _p, _p, _p, _i64, _f, C.c_uint64, C.c_uint64]),
    "fb_logitcrossentropy_labels": (_i32, [_p, _p, _p, _p, _p, _p, _i64, _i64, _f]),
    "fb_logitcrossentropy_dense": (_i32, [_p, _p, _p, _p, _p, _p, _i64, _i64, _f]),
    "fb_sumsq": (_i32, [_p, _p, _p, _i64, _p]),
    "fb_sum": (_i32, [_p, _p, _p, _i64, _p]),
    "fb_timestamp": (_i32, [_p, _p, _p]),
    "fb_fill": (_i32, [_p, _p, _p, _f, _i64]),
    "fb_scale": (_i32, [_p, _p, _p, _f, _p, _i64]),
    "fb_axpy": (_i32, [_p, _p, _f, _p, _p, _i64]),
    "fb_cast_f32_bf16": (_i32, [_p, _p, _p, _p, _i64]),
    "fb_cast_bf16_f32": (_i32, [_p, _p, _p, _p, _i64]),
    "fb_round_bf16": (_i32, [_p, _p, _p, _p, _i64]),
    "fb_adam_step": (_i32, [_p, _p, _i32, C.POINTER(_p), C.POINTER(_p), C.POINTER(_p), C.POINTER(_p),
                            C.POINTER(_i64), _f, _f, _f, _f, _f, _f, _f]),
    "fb_adam_step_dev": (_i32, [_p, _p, _i32, C.POINTER(_p), C.POINTER(_p), C.POINTER(_p), C.POINTER(_p),
                                C.POINTER(_i64), _f, _f, _f, _f, _p, _p, _f]),
    "fb_adam_block_dev": (_i32, [_p, _p, _p, _p, _p, _p, _i64, _f, _f, _f, _f, _p, _p, _f]),
    "fb_adam_advance": (_i32, [_p, _p, _p, _f, _f, _p]),
    "fb_lstm_cache_bytes": (_i64, [_i64, _i64, _i64, _i64]),
    "fb_gru_cache_bytes": (_i64, [_i64, _i64, _i64, _i64]),
    "fb_lstm_fwd": (_i32, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64]),
    "fb_lstm_bwd": (_i32, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64]),
    "fb_gru_fwd": (_i32, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64]),
    "fb_gru_bwd": (_i32, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64]),
    "fb_rnn_cache_bytes": (_i64, [_i64, _i64, _i64, _i64]),
    "fb_rnn_fwd": (_i32, [_p, _p, _i32, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64]),
    "fb_rnn_bwd": (_i32, [_p, _p, _i32, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64]),
    "fb_gruv3_cache_bytes": (_i64, [_i64, _i64, _i64, _i64]),
    "fb_gruv3_fwd": (_i32, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64]),
    "fb_gruv3_bwd": (_i32, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64]),
    "fb_attn_fwd": (_i32, [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i32, _i32]),
    "fb_attn_bwd": (_i32, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i32, _i32]),
    "fb_attn_scores": (_i32, [_p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i32, _i32]),
    "fb_attn_fwd_ex": (_i32, [_p, _p, _p, _p, _p, _p, _p, _i64, _i64, _f, C.c_uint64, C.c_uint64, _p, _p, _i64, _i64, _i64, _i64, _i64, _i32, _i32]),
    "fb_attn_bwd_ex": (_i32, [_p, _p, _p, _p, _p, _p, _p, _i64, _i64, _f, C.c_uint64, C.c_uint64, _p, _p, _p, _p, _p, _p, _p,
                              _i64, _i64, _i64, _i64, _i64, _i32, _i32]),
    "fb_attn_scores_ex": (_i32, [_p, _p, _p, _p, _p, _p, _i64, _i64, _f, C.c_uint64, C.c_uint64, _p, _p, _i64, _i64, _i64, _i64, _i32, _i32]),
    "fb_comm_get_unique_id": (_i32, [_p]),
    "fb_comm_init_rank": (_i32, [_p, _p, _i32, _i32, C.POINTER(_p)]),
    "fb_comm_destroy": (_i32, [_p]),
    "fb_comm_rank": (_i32, [_p]),
    "fb_comm_size": (_i32, [_p]),
    "fb_allreduce": (_i32, [_p, _p, _p, _p, _i64, _i32]),
    "fb_reduce_scatter": (_i32, [_p, _p, _p, _p, _i64, _i32]),
    "fb_allgather": (_i32, [_p, _p, _p, _p, _i64]),
    "fb_bcast": (_i32, [_p, _p, _p, _p, _i64, _i32]),
    "fb_reduce": (_i32, [_p, _p, _p, _p, _i64, _i32, _i32]),
    "fb_peer_alloc": (_i32, [_p, _i64, C.POINTER(_p), _p]),
    "fb_peer_open": (_i32, [_p, _p, C.POINTER(_p)]),
    "fb_peer_close": (_i32, [_p, _p]),
    "fb_peer_free": (_i32, [_p, _p]),
    "fb_peer_barrier": (_i32, [_p, _p, C.POINTER(_p), _i32, _i32, _p, _i64]),
    "fb_peer_push_blocks": (_i32, [_p, _p, _p, _i64, C.POINTER(_p), _i32, _i32, _i64]),
    "fb_reduce_slots": (_i32, [_p, _p, _i32, C.POINTER(_p), _p, _i64, _f]),
    "fb_bucket_create": (_i32, [_p, _p, _p, _i64, _i32, C.POINTER(_i64), _p, C.POINTER(_p)]),
    "fb_bucket_destroy": (_i32, [_p]),
    "fb_bucket_register": (_i32, [_p, _i64, _i64, C.POINTER(_i32)]),
    "fb_bucket_begin_step": (_i32, [_p]),
    "fb_bucket_mark_ready": (_i32, [_p, _i32, _p]),
    "fb_bucket_wait": (_i32, [_p, _p]),
    "fb_comm_async_error": (_i32, [_p, C.POINTER(_i32)]),
}

for _name, (_res, _args) in PROTOTYPES.items():
    _fn = getattr(_lib, _name)   # AttributeError here means the build is out of date
    _fn.restype = _res
    _fn.argtypes = _args


def raw():
    """The ctypes handle (tests call entry points directly through it)."""
    return _lib


def last_error() -> str:
    return _lib.fb_last_error().decode("utf-8", "replace")


def check(status: int) -> None:
    if status != FB_OK:
        raise FluxB200Error(status, last_error())


PROFILE = None   # optional {"names": set, "events": list}: CUDA events recorded around the named entry points


def call(name: str, *args):
    """Calls an int32-status entry point and raises FluxB200Error on failure."""
    prof = PROFILE
    if prof is not None and name in prof["names"]:
        import torch
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        check(getattr(_lib, name)(*args))
        e1.record()
        prof["events"].append((name, args, e0, e1))
        return
    check(getattr(_lib, name)(*args))
