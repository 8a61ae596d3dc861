"""Batches that arrive on the device: `DataLoader` (MLUtils.DataLoader as re-exported by Flux, src/Flux.jl:40) and the
device iterator that `DataLoader |> gpu` gives (MLDataDevices.DeviceIterator; test/ext_cuda/cuda.jl:177-204).

The device iterator stages every batch through pinned host memory and copies it on its own stream while the previous
batch is being used (two device buffers per array), so the host-to-device transfer runs beside the training step.
"""
from __future__ import annotations

import numpy as np
import torch

from .core import B200Array, context


class DataLoader:
    """DataLoader(data; batchsize=1, shuffle=false, partial=true, rng): `data` is an array or a tuple of arrays whose
    LAST dimension counts the observations (MLUtils' convention); iteration yields arrays (or tuples) of `batchsize`
    observations, the last one shorter when `partial`."""

    def __init__(self, data, batchsize: int = 1, shuffle: bool = False, partial: bool = True, rng=None):
        self.data = data
        self.tuple = isinstance(data, (tuple, list))
        arrs = list(data) if self.tuple else [data]
        n = {a.shape[-1] for a in arrs}
        if len(n) != 1:
            raise ValueError("DimensionMismatch: all data containers must have the same number of observations")
        self.nobs = n.pop()
        if batchsize < 1:
            raise ValueError("ArgumentError: batchsize must be positive")
        self.batchsize, self.shuffle, self.partial = int(batchsize), bool(shuffle), bool(partial)
        self.rng = rng if rng is not None else np.random.default_rng()

    def __len__(self):
        return -(-self.nobs // self.batchsize) if self.partial else self.nobs // self.batchsize

    def __iter__(self):
        order = self.rng.permutation(self.nobs) if self.shuffle else np.arange(self.nobs)
        arrs = list(self.data) if self.tuple else [self.data]
        for i in range(len(self)):
            idx = order[i * self.batchsize:(i + 1) * self.batchsize]
            contiguous = not self.shuffle
            batch = [a[..., idx[0]:idx[-1] + 1] if contiguous else a[..., idx] for a in arrs]
            yield tuple(batch) if self.tuple else batch[0]


def _host_flat(a: np.ndarray) -> np.ndarray:
    if a.dtype == np.float64:
        a = a.astype(np.float32)
    elif a.dtype == np.int64:
        a = a.astype(np.int32)
    elif a.dtype == np.bool_:
        a = a.astype(np.uint8)
    return np.ascontiguousarray(a.reshape(-1, order="F"))


class DeviceIterator:
    """`DataLoader |> gpu`: yields B200 arrays.  Batch k + 1 is copied (pinned staging buffer, dedicated copy stream)
    while the caller works on batch k; a yielded batch stays valid until the batch after the next one is requested."""

    def __init__(self, loader, depth: int = 2):
        self.loader = loader
        self.depth = max(2, int(depth))

    def __len__(self):
        return len(self.loader)

    def __iter__(self):
        ctx = context()
        dev = f"cuda:{ctx.device}"
        copy_stream = torch.cuda.Stream()
        slots = [None] * self.depth     # per slot: list of (pinned host tensor, device tensor) per array
        ready = [None] * self.depth
        released = [None] * self.depth  # event recorded on the consumer's stream when the slot may be overwritten

        def stage(slot, batch):
            arrs = list(batch) if isinstance(batch, tuple) else [batch]
            flats = [_host_flat(np.asarray(a)) for a in arrs]
            bufs = slots[slot]
            if bufs is None or any(b[0].numel() < f.size or b[0].numpy().dtype != f.dtype for b, f in zip(bufs, flats)) or len(bufs) != len(flats):
                bufs = [(torch.empty(f.size, dtype=torch.from_numpy(f).dtype).pin_memory(),
                         torch.empty(f.size, dtype=torch.from_numpy(f).dtype, device=dev)) for f in flats]
                slots[slot] = bufs
            if released[slot] is not None:
                copy_stream.wait_event(released[slot])
            out = []
            with torch.cuda.stream(copy_stream):
                for (pin, devt), f, a in zip(bufs, flats, arrs):
                    pin[:f.size].copy_(torch.from_numpy(f))
                    devt[:f.size].copy_(pin[:f.size], non_blocking=True)
                    out.append(B200Array(devt[:f.size], np.asarray(a).shape))
                ev = torch.cuda.Event()
                ev.record(copy_stream)
            ready[slot] = ev
            return tuple(out) if isinstance(batch, tuple) else out[0]

        it = iter(self.loader)
        pending = []
        k = 0
        for batch in it:
            pending.append((k % self.depth, stage(k % self.depth, batch)))
            k += 1
            if len(pending) == self.depth:
                slot, dev_batch = pending.pop(0)
                torch.cuda.current_stream().wait_event(ready[slot])
                yield dev_batch
                released[slot] = torch.cuda.Event()
                released[slot].record(torch.cuda.current_stream())
        for slot, dev_batch in pending:
            torch.cuda.current_stream().wait_event(ready[slot])
            yield dev_batch
            released[slot] = torch.cuda.Event()
            released[slot].record(torch.cuda.current_stream())
