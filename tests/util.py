"""Helpers shared by the GPU parity tests: Julia-shaped numpy <-> flat device buffers, tolerances."""
import ctypes as C

import numpy as np
import torch

RTOL = 1e-4   # fp32 parity tolerance on outputs and gradients (the reference's test_gradients uses rtol = atol = 1e-4)


def dev(a, dtype=None):
    """Julia-shaped numpy array -> flat CUDA tensor in column-major (Julia) memory order."""
    a = np.asarray(a)
    if dtype is not None:
        a = a.astype(dtype)
    return torch.from_numpy(np.ascontiguousarray(a.reshape(-1, order="F"))).cuda()


def host(t, shape):
    return t.detach().cpu().numpy().reshape(shape, order="F")


def dempty(*shape, dtype=torch.float32):
    n = int(np.prod(shape)) if shape else 1
    return torch.empty(max(n, 1), dtype=dtype, device="cuda")


def P(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def close(got, ref, rtol=RTOL, atol_scale=RTOL, name=""):
    ref = np.asarray(ref, dtype=np.float64)
    got = np.asarray(got, dtype=np.float64)
    scale = float(np.max(np.abs(ref))) if ref.size else 0.0
    np.testing.assert_allclose(got, ref, rtol=rtol, atol=atol_scale * max(scale, 1e-30), err_msg=name)


def stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)
