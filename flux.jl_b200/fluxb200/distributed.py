"""DistributedUtils for B200 arrays: NCCL backend, broadcast / allreduce / reduce, `synchronize`,
`DistributedDataContainer`, `DistributedOptimizer` with bucketed, overlapped gradient averaging.

Mirrors src/distributed/public_api.jl (initialize :45-49, get_distributed_backend :67-71,
local_rank / total_workers :82-93, bcast! :102-116, allreduce! :134-150, reduce! :166-183,
synchronize!! :203-231, DistributedDataContainer :245-272, DistributedOptimizer :286-300) and
ext/FluxMPINCCLExt (NCCL collectives on device buffers).  The reference bootstraps the NCCL unique
id over MPI; here the launcher's rendezvous (torch.distributed store, env:// as torchrun sets it)
carries the 128 id bytes, and every data-path collective runs through fb_allreduce / fb_bcast /
fb_reduce of libfluxb200.so on a dedicated communication stream.
"""
from __future__ import annotations

import ctypes as C
import math
import os

import numpy as np
import torch

from . import lib
from .core import B200Array, context
from .layers import Layer, trainables
from .train import DistributedOptimizerBase, OptState

avg = "avg"
_BACKEND = None


class NCCLBackend:
    """NCCLBackend(comm): one rank of a single-node NCCL communicator."""

    def __init__(self, comm_handle, rank: int, size: int):
        self.comm = comm_handle
        self.rank, self.size = rank, size
        self.stream = torch.cuda.Stream(priority=-1)   # communication stream (high priority)

    def __repr__(self):
        return f"NCCLBackend(rank={self.rank}, size={self.size})"


def shard_indices(total_size: int, total_workers: int, local_rank: int) -> np.ndarray:
    """public_api.jl:262-272: contiguous ceil(n/N) index ranges (0-based here), shorter last shard."""
    per = int(math.ceil(total_size / total_workers))
    starts = list(range(0, total_size, per))
    if local_rank >= len(starts):
        raise IndexError("BoundsError: attempt to access partition of a rank without data")
    s = starts[local_rank]
    return np.arange(s, min(s + per, total_size))


def initialize(backend=NCCLBackend, device: int | None = None):
    """DistributedUtils.initialize(NCCLBackend): joins the process group named by the launcher's
    environment (RANK, WORLD_SIZE, LOCAL_RANK, MASTER_ADDR, MASTER_PORT) and creates the communicator."""
    global _BACKEND
    if _BACKEND is not None:
        return _BACKEND
    rank = int(os.environ.get("RANK", "0"))
    size = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    dev = local if device is None else device
    ctx = context(dev)
    idbuf = (C.c_uint8 * lib.UNIQUE_ID_BYTES)()
    if size > 1:
        import torch.distributed as dist
        if not dist.is_initialized():
            dist.init_process_group(backend="gloo", rank=rank, world_size=size)
        if rank == 0:
            lib.call("fb_comm_get_unique_id", idbuf)
        t = torch.tensor(list(bytes(idbuf)), dtype=torch.uint8)
        dist.broadcast(t, src=0)
        idbuf = (C.c_uint8 * lib.UNIQUE_ID_BYTES)(*t.tolist())
        h = C.c_void_p()
        lib.call("fb_comm_init_rank", ctx.handle, idbuf, size, rank, C.byref(h))
    else:
        # a single worker needs no communicator; one is still created when NCCL is present so that the
        # collectives run the same code path
        h = C.c_void_p()
        try:
            lib.call("fb_comm_get_unique_id", idbuf)
            lib.call("fb_comm_init_rank", ctx.handle, idbuf, 1, 0, C.byref(h))
        except lib.FluxB200Error:
            h = None
    _BACKEND = NCCLBackend(h, rank, size)
    return _BACKEND


def get_distributed_backend(backend=NCCLBackend):
    if _BACKEND is None:
        raise RuntimeError("backend `NCCLBackend` is not initialized; call DistributedUtils.initialize first")
    return _BACKEND


def local_rank(backend) -> int:
    return backend.rank


def total_workers(backend) -> int:
    return backend.size


def _stream_ptr(backend, on_comm_stream: bool):
    s = backend.stream if on_comm_stream else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)


def _local_copy(src: B200Array, dst: B200Array):
    """A one-worker collective is a copy (or nothing when the buffers coincide)."""
    if dst.t.data_ptr() != src.t.data_ptr():
        ctx = context()
        lib.call("fb_memcpy_d2d", ctx.handle, ctx.stream, dst.ptr, src.ptr, 4 * dst.numel())
    return dst


def bcast(backend, sendrecvbuf: B200Array, recvbuf: B200Array | None = None, root: int = 0):
    """bcast!(backend, sendrecvbuf; root) / bcast!(backend, sendbuf, recvbuf; root)."""
    dst = sendrecvbuf if recvbuf is None else recvbuf
    if backend.comm is None:
        return _local_copy(sendrecvbuf, dst)
    lib.call("fb_bcast", backend.comm, _stream_ptr(backend, False), sendrecvbuf.ptr, dst.ptr, dst.numel(), root)
    return dst


def allreduce(backend, sendrecvbuf: B200Array, op_or_recv="+", op=None):
    """allreduce!(backend, sendrecvbuf, op) / allreduce!(backend, sendbuf, recvbuf, op); op is "+" or avg."""
    if isinstance(op_or_recv, B200Array):
        dst, o = op_or_recv, op
    else:
        dst, o = sendrecvbuf, op_or_recv
    if backend.comm is None:
        return _local_copy(sendrecvbuf, dst)
    lib.call("fb_allreduce", backend.comm, _stream_ptr(backend, False), sendrecvbuf.ptr, dst.ptr, dst.numel(), lib.OP[o])
    return dst


def reduce(backend, sendrecvbuf: B200Array, op_or_recv="+", op=None, root: int = 0):
    if isinstance(op_or_recv, B200Array):
        dst, o = op_or_recv, op
    else:
        dst, o = sendrecvbuf, op_or_recv
    if backend.comm is None:
        return _local_copy(sendrecvbuf, dst)
    lib.call("fb_reduce", backend.comm, _stream_ptr(backend, False), sendrecvbuf.ptr, dst.ptr, dst.numel(), lib.OP[o], root)
    return dst


class WorkerLost(lib.FluxB200Error):
    """A worker did not report for a step in time, or reported a different gradient-bucket layout."""

    def __init__(self, msg):
        super().__init__(-6, msg)


class Heartbeat:
    """Host-side failure detection between steps.  Before a step is launched every worker adds itself to a counter
    of that step in the rendezvous store and waits (with a limit) until all have; a worker that died, hung or left
    is noticed here, on the host, instead of inside the next collective, which would wait for it for ever (as it does
    in the reference: NCCL.Allreduce! has no timeout, ext/FluxMPINCCLExt/FluxMPINCCLExt.jl:61-66).

    `store` is any object with torch.distributed.Store's `add(key, n) -> int` (TCPStore, FileStore, HashStore)."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 30.0, poll_s: float = 0.005, prefix: str = "fluxb200/hb"):
        self.store, self.rank, self.world = store, int(rank), int(world)
        self.timeout_s, self.poll_s, self.prefix = float(timeout_s), float(poll_s), prefix
        self.step = 0

    def beat(self):
        """Call once per step on every worker, before the step's first launch.  Raises WorkerLost when fewer than
        `world` workers have reported within the limit."""
        import time
        key = f"{self.prefix}/{self.step}"
        seen = self.store.add(key, 1)
        t0 = time.monotonic()
        while seen < self.world:
            if time.monotonic() - t0 > self.timeout_s:
                raise WorkerLost(f"step {self.step}: only {seen} of {self.world} workers reported within {self.timeout_s:g} s "
                                 f"(seen from rank {self.rank}); not launching the step")
            time.sleep(self.poll_s)
            seen = self.store.add(key, 0)
        self.step += 1


def verify_layout(store, rank: int, world: int, layout, timeout_s: float = 30.0, prefix: str = "fluxb200/layout"):
    """Every worker publishes a digest of its gradient-bucket layout (bucket boundaries and leaf sizes) and compares it
    with the others' before the first collective: a worker built with a different model or bucket size would otherwise
    exchange buffers of different lengths, which NCCL answers with a hang or silent corruption."""
    import hashlib
    import time
    digest = hashlib.sha256(repr(layout).encode()).hexdigest()
    store.set(f"{prefix}/{rank}", digest)
    t0 = time.monotonic()
    for r in range(world):
        key = f"{prefix}/{r}"
        while True:
            try:
                if hasattr(store, "check") and not store.check([key]):
                    raise KeyError(key)
                other = store.get(key)
                break
            except Exception:
                if time.monotonic() - t0 > timeout_s:
                    raise WorkerLost(f"worker {r} did not publish its gradient-bucket layout within {timeout_s:g} s")
                time.sleep(0.005)
        other = other.decode() if isinstance(other, (bytes, bytearray)) else str(other)
        if other != digest:
            raise WorkerLost(f"worker {r} has a different gradient-bucket layout than worker {rank}: the workers were not "
                             "built with the same model / bucket size")


class FluxDistributedModel:
    def __init__(self, model):
        self.model = model


def synchronize(backend, ps, root: int = 0):
    """synchronize!!(backend, ps; root): broadcasts every array leaf (model parameters, optimiser
    moments) from `root`; scalar state (β powers) is broadcast through a one-element buffer."""
    if isinstance(ps, FluxDistributedModel):
        synchronize(backend, ps.model, root)
        return ps.model
    if isinstance(ps, B200Array):
        bcast(backend, ps, root=root)
        return ps
    if isinstance(ps, OptState):
        for leaf in ps.leaves.values():
            if leaf.state is not None:
                bcast(backend, leaf.state[0], root=root)
                bcast(backend, leaf.state[1], root=root)
                t = torch.tensor(leaf.state[2], dtype=torch.float32, device="cuda")
                bcast(backend, B200Array(t, (2,)), root=root)
                v = t.cpu().tolist()
                leaf.state[2] = (float(np.float32(v[0])), float(np.float32(v[1])))
        return ps
    if isinstance(ps, (tuple, list)):
        return type(ps)(synchronize(backend, p, root) for p in ps)
    if isinstance(ps, dict):
        return {k: synchronize(backend, v, root) for k, v in ps.items()}
    if isinstance(ps, Layer):
        for name in ps._fields:
            v = getattr(ps, name, None)
            if isinstance(v, (B200Array, Layer, tuple, list)):
                synchronize(backend, v, root)
        return ps
    return ps


class DistributedDataContainer:
    """DistributedDataContainer(backend, data): this rank's contiguous shard of the observations
    (last array dimension)."""

    def __init__(self, backend, data: np.ndarray):
        self.data = data
        n = data.shape[-1]
        self.idxs = shard_indices(n, backend.size, backend.rank)

    def __len__(self):
        return len(self.idxs)

    def __getitem__(self, i):
        return self.data[..., self.idxs[i]]


class GradBuckets:
    """Flat gradient buffer split into buckets of ~bucket_mb MiB in reverse parameter order (the order
    the backward pass produces gradients), the small leaves together in one last bucket.  Layer pullbacks write
    gradients straight into their slice; when a bucket's last gradient has landed, its exchange starts on the
    communication stream while the backward pass continues: a mean all-reduce, or - in a step captured with the
    sharded optimiser (`shard_optimizer`) - reduce-scatter, Adam on this rank's block and all-gather, over peer memory
    on one node (`_setup_peer_exchange`) or with NCCL."""

    SMALL_LEAF = 1 << 16   # leaves below this many elements share the last bucket

    def __init__(self, backend, params, bucket_mb: float = 64.0, reserved_sms: int | None = None):
        self.backend = backend
        # SMs the persistent GEMMs leave free for the exchange kernels.  Measured at 8 GPUs, per-GPU batch 1024: with
        # the NCCL exchange 0, 16 and 32 reserved SMs give 6.43-6.51, 6.52-6.56 and 6.85 ms per step; with the
        # peer-memory exchange 12 reserved SMs gave 5.95 against 6.12 ms in one run and the default 5.91 in another,
        # so the default reserves none (FLUXB200_SM_RESERVE or the argument overrides).
        if reserved_sms is None:
            reserved_sms = int(os.environ.get("FLUXB200_SM_RESERVE", "0"))
        self.reserved_sms = reserved_sms if backend.size > 1 else 0
        self.params = list(params)
        pad = lambda n: (n + 63) // 64 * 64          # every slice starts on a 256-byte boundary
        total = sum(pad(p.numel()) for p in self.params)
        dev = self.params[0].t.device
        self.flat = torch.zeros(total, dtype=torch.float32, device=dev)
        self.views, self.bucket_of, self.offsets = {}, {}, {}
        self.buckets = []   # [start, end, pending ids, all ids]
        # sharded-optimiser mode (shard_optimizer): parameters / Adam moments re-homed in flat buffers laid out
        # like the gradient buffer; `armed` is set by the step that captured the update kernels
        self.pflat = self.mflat = self.vflat = None
        self.adam = None
        self.armed = False
        self.peer = None             # peer-memory tables of the exchange over NVLink (see _setup_peer_exchange)
        self.defer_gather = False    # parameter gathers at the start of the next step (start_gathers) instead of per bucket
        self.gather_events = None
        self.gathering = False
        self.loss = None
        self.guard = None            # device scalar the update kernels test for finiteness (see set_loss)
        self._guard_buf = None
        self.guard_event = None
        # optional timeline: device time marks (fb_timestamp) placed on both streams; see enable_timeline
        self.marks = None
        self.mark_names = []
        limit = int(bucket_mb * (1 << 20) / 4)
        off = 0
        cur_start, cur_ids = 0, []
        # Weight matrices in the order the reverse sweep produces them, cut into buckets of ~bucket_mb; the small
        # leaves (biases, normalisation scales) together in one last bucket.  A Dense pullback reports its weight
        # gradient as soon as the dW product is enqueued, so a bucket of weights starts its exchange while the dX
        # product and the normalisation layer's reverse pass still run; what is left after the sweep's last kernel is
        # the small bucket only.
        small = lambda q: q.numel() < self.SMALL_LEAF
        order = [q for q in reversed(self.params) if not small(q)]
        n_big = len(order)
        order += [q for q in reversed(self.params) if small(q)]
        for pi, p in enumerate(order):
            if pi == n_big and cur_ids:       # the small leaves start a bucket of their own
                self.buckets.append([cur_start, off, set(), list(cur_ids)])
                cur_start, cur_ids = off, []
            n = p.numel()
            self.views[id(p)] = B200Array(self.flat[off:off + n], p.size)
            self.offsets[id(p)] = off
            cur_ids.append(id(p))
            off += pad(n)
            if off - cur_start >= limit:
                self.buckets.append([cur_start, off, set(), list(cur_ids)])
                cur_start, cur_ids = off, []
        if cur_ids:
            self.buckets.append([cur_start, off, set(), list(cur_ids)])
        for bi, b in enumerate(self.buckets):
            for k in b[3]:
                self.bucket_of[k] = bi
        self.events = [torch.cuda.Event() for _ in self.buckets]
        self.launched = [False] * len(self.buckets)
        self.begin_step()

    def layout(self):
        """What has to agree on every worker: bucket boundaries and the size of every gradient slice, in order."""
        return (tuple((b[0], b[1]) for b in self.buckets), tuple(p.numel() for p in self.params), self.backend.size)

    def enable_timeline(self, slots: int = 256):
        """Time marks on the compute and communication streams (they are captured with the step when it is a
        graph): after a step `timeline()` lists (name, microseconds since the step's first mark)."""
        self.marks = torch.zeros(slots, dtype=torch.int64, device=self.flat.device)
        self.mark_names = []

    def _mark(self, name, stream=None):
        if self.marks is None or len(self.mark_names) >= self.marks.numel():
            return
        st = C.c_void_p(stream.cuda_stream) if stream is not None else context().stream
        lib.call("fb_timestamp", context().handle, st, C.c_void_p(self.marks.data_ptr() + 8 * len(self.mark_names)))
        self.mark_names.append(name)

    def timeline(self):
        if self.marks is None:
            return []
        t = self.marks[:len(self.mark_names)].cpu().tolist()
        t0 = min(t) if t else 0
        return sorted(((n, (v - t0) / 1e3) for n, v in zip(self.mark_names, t)), key=lambda kv: kv[1])

    def begin_step(self):
        for b in self.buckets:
            b[2] = set(b[3])
        self.launched = [False] * len(self.buckets)
        self.early = set()      # parameters a pullback reported itself and has not released yet
        self.holds = {}         # bucket -> early-reported parameters some enqueued kernel may still read
        self.update_pending = set()   # buckets whose gradients are exchanged but whose update waits for a release
        self.gather_waited = set()   # buckets whose deferred parameter gather the forward pass already waits for
        self.handed = set()     # parameters whose slice a pullback of this step already writes
        self.uses = {}          # parameter id -> gradient contributions still to come (set by expect_uses)
        if self.marks is not None:
            self.mark_names = []
            self._mark("step start")

    def buffer_for(self, param):
        """The slice of the flat gradient buffer a pullback may OVERWRITE with this parameter's gradient: handed out
        once per step.  A parameter applied twice in one model (tied weights, a layer called twice) gets None for its
        later contributions, which then go to a temporary that `accumulate` adds to the slice."""
        if param is None:
            return None
        k = id(param)
        if k not in self.views or k in self.handed:
            return None
        self.handed.add(k)
        return self.views[k]

    def expect_uses(self, counts: dict):
        """counts[id(param)] = number of recorded layer calls that will contribute a gradient to the parameter in this
        reverse sweep; `ready` starts a bucket only after the last contribution of each of its parameters."""
        self.uses = dict(counts)

    def ready(self, param, early=False):
        """The gradient of `param` has been enqueued.  A pullback may call this itself with early=True as soon as the
        kernel that writes the gradient is launched although its remaining kernels still READ the parameter; the
        reverse sweep's own call for the same contribution, which comes when the pullback has returned, then only
        releases the parameter.  Between the two calls the bucket's gradient exchange may run, its parameter update
        may not (`_launch` holds it back).  Honoured with the peer-memory exchange only."""
        k = id(param)
        bi = self.bucket_of.get(k)
        if bi is None:
            return
        if early:
            if not (self.armed and self.peer is not None):
                return
            self.early.add(k)
            self.holds[bi] = self.holds.get(bi, 0) + 1
        elif k in self.early:
            self.early.discard(k)
            self.holds[bi] -= 1
            if self.holds[bi] == 0 and bi in self.update_pending:
                self.update_pending.discard(bi)
                self._peer_update(bi)
            return
        left = self.uses.get(k, 1) - 1
        self.uses[k] = left
        if left > 0:
            return
        b = self.buckets[bi]
        b[2].discard(k)
        if not b[2] and not self.launched[bi]:
            self._launch(bi)

    def shard_optimizer(self, opt_state, bt: torch.Tensor) -> bool:
        """Sharded optimiser state: after every bucket's reduce-scatter each rank runs Adam on its 1/N block of
        the bucket and the blocks are put together again by an all-gather, all on the communication stream while
        the backward pass continues (the layers of a finished bucket are not read again in the step).  The result
        equals all-reduce + Adam on every rank; the update costs 1/N of the HBM traffic per rank.

        Parameters and moments are re-homed (values kept) in flat buffers with the gradient buffer's layout; a
        rank's moments are current only inside its own blocks.  `bt` is the device tensor holding (β1ᵗ, β2ᵗ).
        Returns False (and changes nothing) when a bucket does not divide by the number of workers."""
        from .train import Adam
        n = self.backend.size
        rule = opt_state.rule
        if n == 1 or not isinstance(rule, Adam) or any((b[1] - b[0]) % n for b in self.buckets):
            return False
        if self.pflat is None:
            self.mflat, self.vflat = (torch.zeros_like(self.flat) for _ in range(2))
            # parameters live in memory the peers can write when the peer-memory exchange is available
            self.pflat = self._setup_peer_exchange()
            if self.pflat is None:
                self.pflat = torch.zeros_like(self.flat)
            for p in self.params:
                off, cnt = self.offsets[id(p)], p.numel()
                st = opt_state.leaves[id(p)].state
                for flat, arr in ((self.pflat, p), (self.mflat, st[0]), (self.vflat, st[1])):
                    view = flat[off:off + cnt]
                    view.copy_(arr.t)
                    arr.t = view
        self.adam = (rule, bt)
        return True

    def _setup_peer_exchange(self):
        """Allocates a staging area, this rank's parameter buffer and a page of barrier words in memory the other ranks
        map (CUDA IPC) and maps theirs, so that the reduce-scatter and the all-gather of the sharded step run as small
        kernels that store over NVLink (fb_peer_push_blocks, fb_peer_barrier, fb_reduce_slots).  Returns the parameter
        buffer as a tensor, or None when any rank cannot map its peers (or FLUXB200_EXCHANGE=nccl): then the NCCL
        collectives are used."""
        import torch.distributed as dist
        be = self.backend
        self.peer = None
        want = os.environ.get("FLUXB200_EXCHANGE", "peer") == "peer" and be.size <= 16 and dist.is_initialized()
        ctx = context()
        nbytes = 4 * self.flat.numel()
        HB = 64
        NB = 3                              # staging area, parameter buffer, barrier epoch words
        mine, ptrs = [0] * (1 + NB * HB + 16), []
        mine[1 + NB * HB:] = list(torch.cuda.get_device_properties(self.flat.device).uuid.bytes)
        if want:
            try:
                for k in range(NB):
                    ptr, h = C.c_void_p(), (C.c_uint8 * HB)()
                    lib.call("fb_peer_alloc", ctx.handle, nbytes if k < 2 else 4096, C.byref(ptr), h)
                    ptrs.append(ptr.value)
                    mine[1 + k * HB:1 + (k + 1) * HB] = list(bytes(h))
                mine[0] = 1
            except lib.FluxB200Error:
                mine[0] = 0
        gathered = [torch.zeros(1 + NB * HB + 16, dtype=torch.uint8) for _ in range(be.size)]
        dist.all_gather(gathered, torch.tensor(mine, dtype=torch.uint8))
        ok = all(int(g[0]) == 1 for g in gathered)
        # the barrier kernels of the ranks wait for one another: every rank needs a GPU of its own
        ok = ok and len({bytes(g[1 + NB * HB:].tolist()) for g in gathered}) == be.size
        stage, pbuf, flags = [None] * be.size, [None] * be.size, [None] * be.size
        if ok:
            try:
                for r, g in enumerate(gathered):
                    if r == be.rank:
                        stage[r], pbuf[r], flags[r] = ptrs
                        continue
                    for k, table in ((0, stage), (1, pbuf), (2, flags)):
                        h = (C.c_uint8 * HB)(*g[1 + k * HB:1 + (k + 1) * HB].tolist())
                        ptr = C.c_void_p()
                        lib.call("fb_peer_open", ctx.handle, h, C.byref(ptr))
                        table[r] = ptr.value
            except lib.FluxB200Error:
                ok = False
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) != 1:
            for ptr in ptrs:
                lib.call("fb_peer_free", ctx.handle, C.c_void_p(ptr))
            return None

        class _Raw:   # a device buffer owned by the library, seen by torch without a copy
            def __init__(self, ptr, count):
                self.__cuda_array_interface__ = {"shape": (count,), "typestr": "<f4", "data": (ptr, False), "version": 3, "strides": None}

        raw = _Raw(pbuf[be.rank], self.flat.numel())
        ptensor = torch.as_tensor(raw, device=self.flat.device)
        self.peer = {"stage": stage, "pflat": pbuf, "flags": flags, "keep": raw,
                     "epoch": torch.zeros(1, dtype=torch.int32, device=self.flat.device),
                     "timeout_ms": int(os.environ.get("FLUXB200_BARRIER_TIMEOUT_MS", "10000"))}
        dist.barrier()      # every rank has mapped every flag array before the first epoch is posted
        return ptensor

    def start_gathers(self):
        """Deferred all-gather (sharded optimiser over peer memory): the parameter blocks updated in the previous step
        travel to the peers at the START of a step, in the order the forward pass needs them, beside the forward
        pass - instead of beside the reverse sweep, whose exchange then carries the gradients only.  Every layer waits
        for its bucket (`wait_param`) before it reads its parameters.  Between steps the parameters of a rank are
        current only inside its own blocks; `sync_params` brings them together for a reader outside the step."""
        peer = self.peer
        if peer is None or self.adam is None:
            return
        be = self.backend
        n = be.size
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        be.stream.wait_event(ev)
        cs = C.c_void_p(be.stream.cuda_stream)
        h = context().handle
        tab = C.c_void_p * n
        if self.gather_events is None:
            self.gather_events = [torch.cuda.Event() for _ in self.buckets]
            self.start_fence = torch.cuda.Event()
        # one barrier first: every rank has finished the previous step - nobody reads the old parameter values any
        # more (the dX products of a slower rank) and the staging areas are free again
        self._peer_barrier(cs)
        self.start_fence.record(be.stream)
        nb = len(self.buckets)
        order = [nb - 1] + list(range(nb - 2, -1, -1)) if nb > 1 else [0]   # small leaves, then weights first layer first
        for bi in order:
            self._peer_gather(bi)
            self._peer_barrier(cs)      # the peers' blocks of this bucket have landed here
            self.gather_events[bi].record(be.stream)
        self.gather_waited = set()
        self.gathering = True

    def wait_param(self, param):
        """Called by a layer before it reads `param` in a step with deferred gathers."""
        if not getattr(self, "gathering", False) or param is None:
            return
        bi = self.bucket_of.get(id(param))
        if bi is None or bi in self.gather_waited:
            return
        self.gather_waited.add(bi)
        torch.cuda.current_stream().wait_event(self.gather_events[bi])

    def sync_params(self):
        """Brings every rank's parameters up to date (outside a step): runs the deferred gathers now and waits."""
        if self.peer is None or not self.defer_gather:
            return
        self.start_gathers()
        for ev in self.gather_events:
            torch.cuda.current_stream().wait_event(ev)
        self.gathering = False
        torch.cuda.current_stream().synchronize()

    def _peer_barrier(self, cs):
        """A barrier between the ranks on the communication stream (fb_peer_barrier: one warp posting and polling epoch
        words in peer memory): when it completes on this rank, every rank has finished what it enqueued before its own
        call.  A peer that does not arrive within FLUXB200_BARRIER_TIMEOUT_MS (default 10 s) leaves code 9101 in the
        device error word, which the step's error poll raises on the host."""
        peer = self.peer
        n = self.backend.size
        lib.call("fb_peer_barrier", context().handle, cs, (C.c_void_p * n)(*peer["flags"]), n, self.backend.rank,
                 C.c_void_p(peer["epoch"].data_ptr()), peer["timeout_ms"])

    def set_loss(self, loss):
        """The step's loss (device scalar): the captured update kernels skip themselves when it is not finite.  With
        several workers the guard is the SUM of the workers' losses (NaN and Inf survive a sum), so that every rank
        takes the same decision: either all update, or none does (src/train.jl:377 decides per process, which would
        let replicas diverge)."""
        self.loss = loss
        self.guard = loss
        be = self.backend
        if self.gathering and getattr(self, "start_fence", None) is not None:
            # no gradient is written before every rank has left the previous step (a peer may still read this rank's
            # gradient buffer until then); the layers' own waits normally come first
            torch.cuda.current_stream().wait_event(self.start_fence)
        if be.size > 1 and be.comm is not None:
            if self._guard_buf is None:
                self._guard_buf = B200Array(torch.zeros(1, dtype=torch.float32, device=loss.t.device), ())
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            be.stream.wait_event(ev)
            lib.call("fb_allreduce", be.comm, C.c_void_p(be.stream.cuda_stream), loss.ptr, self._guard_buf.ptr, 1, lib.OP["+"])
            self.guard = self._guard_buf
            self.guard_event = torch.cuda.Event()
            self.guard_event.record(be.stream)
        self._mark("forward end")

    def _launch(self, bi):
        self.launched[bi] = True
        be = self.backend
        if be.size == 1:
            return
        start, end = self.buckets[bi][0], self.buckets[bi][1]
        self._mark(f"bucket {bi} ready")
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        be.stream.wait_event(ev)
        self._mark(f"bucket {bi} comm start", be.stream)
        cs = C.c_void_p(be.stream.cuda_stream)
        ptr = C.c_void_p(self.flat.data_ptr() + 4 * start)
        if self.armed and self.adam is not None and self.loss is not None:
            rule, bt = self.adam
            n = be.size
            blk = (end - start) // n
            lo = 4 * (start + be.rank * blk)
            g, pp = self.flat.data_ptr() + lo, self.pflat.data_ptr() + lo
            one = C.c_void_p * 1
            if self.peer is not None:
                self._peer_exchange(bi)
                if self.holds.get(bi, 0) > 0:
                    self.update_pending.add(bi)
                else:
                    self._peer_update(bi, waited=True)
                return
            lib.call("fb_reduce_scatter", be.comm, cs, ptr, C.c_void_p(g), blk, lib.OP["avg"])
            self._mark(f"bucket {bi} reduce-scatter end", be.stream)
            lib.call("fb_adam_step_dev", context().handle, cs, 1, one(pp), one(g), one(self.mflat.data_ptr() + lo),
                     one(self.vflat.data_ptr() + lo), (C.c_int64 * 1)(blk), rule.eta, rule.beta[0], rule.beta[1],
                     rule.epsilon, C.c_void_p(bt.data_ptr()), self.guard.ptr, 1.0)
            self._mark(f"bucket {bi} adam end", be.stream)
            lib.call("fb_allgather", be.comm, cs, C.c_void_p(pp), C.c_void_p(self.pflat.data_ptr() + 4 * start), blk)
        else:
            lib.call("fb_allreduce", be.comm, cs, ptr, ptr, end - start, lib.OP["avg"])
        self._mark(f"bucket {bi} comm end", be.stream)
        self.events[bi].record(be.stream)

    def _peer_block(self, bi):
        start, end = self.buckets[bi][0], self.buckets[bi][1]
        blk = (end - start) // self.backend.size
        return start, blk, 4 * (start + self.backend.rank * blk)

    def _peer_gather(self, bi):
        """My updated block of one bucket -> its place in every peer's parameter buffer."""
        be, peer = self.backend, self.peer
        n = be.size
        _, blk, lo = self._peer_block(bi)
        lib.call("fb_peer_push_blocks", context().handle, C.c_void_p(be.stream.cuda_stream), C.c_void_p(self.pflat.data_ptr() + lo), 0,
                 (C.c_void_p * n)(*[peer["pflat"][r] + lo for r in range(n)]), n, be.rank, blk)

    def _peer_exchange(self, bi):
        """Reduce-scatter of one bucket over peer memory: block p of my gradients goes to slot [me] of peer p's staging
        area; behind a barrier (the peers' blocks have landed here) the N slots of my block are averaged in rank
        order (my own slot is read where it was produced)."""
        be, peer = self.backend, self.peer
        n = be.size
        start, blk, lo = self._peer_block(bi)
        cs = C.c_void_p(be.stream.cuda_stream)
        h = context().handle
        tab = C.c_void_p * n
        g = self.flat.data_ptr() + lo
        lib.call("fb_peer_push_blocks", h, cs, C.c_void_p(self.flat.data_ptr() + 4 * start), blk,
                 tab(*[peer["stage"][r] + 4 * (start + be.rank * blk) for r in range(n)]), n, be.rank, blk)
        self._peer_barrier(cs)
        slots = tab(*[(peer["stage"][be.rank] + 4 * (start + r * blk)) if r != be.rank else g for r in range(n)])
        lib.call("fb_reduce_slots", h, cs, n, slots, C.c_void_p(g), blk, 1.0 / n)
        self._mark(f"bucket {bi} reduce-scatter end", be.stream)

    def _peer_update(self, bi, waited=False):
        """Adam on my block of one bucket and, unless the gathers are deferred to the next step, a barrier (every
        rank has released the bucket's parameters: nobody reads the old values any more) and the copies of my block
        into the peers' parameter buffers.  With waited=False the call comes from a release: the communication stream
        first waits for the kernels enqueued so far, the last readers of the parameter among them."""
        be = self.backend
        _, blk, lo = self._peer_block(bi)
        cs = C.c_void_p(be.stream.cuda_stream)
        if not waited:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            be.stream.wait_event(ev)
        rule, bt = self.adam
        g, pp = self.flat.data_ptr() + lo, self.pflat.data_ptr() + lo
        lib.call("fb_adam_block_dev", context().handle, cs, C.c_void_p(pp), C.c_void_p(g), C.c_void_p(self.mflat.data_ptr() + lo),
                 C.c_void_p(self.vflat.data_ptr() + lo), blk, rule.eta, rule.beta[0], rule.beta[1], rule.epsilon,
                 C.c_void_p(bt.data_ptr()), self.guard.ptr, 1.0)
        self._mark(f"bucket {bi} adam end", be.stream)
        if not self.defer_gather:
            self._peer_barrier(cs)
            self._peer_gather(bi)
        self._mark(f"bucket {bi} comm end", be.stream)
        self.events[bi].record(be.stream)

    def finish(self):
        """Launches whatever is still pending and makes the compute stream wait for every bucket."""
        for bi in range(len(self.buckets)):
            if not self.launched[bi]:
                self._launch(bi)
        self._mark("backward end")
        if self.backend.size > 1:
            for bi in sorted(self.update_pending):      # a pullback that never released: update after everything enqueued
                self._peer_update(bi)
            self.update_pending = set()
            if self.armed and self.peer is not None and not self.defer_gather:
                # the peers' parameter blocks must have landed here before anybody reads the parameters again
                self._peer_barrier(C.c_void_p(self.backend.stream.cuda_stream))
                self.events[-1].record(self.backend.stream)
            for ev in self.events:
                torch.cuda.current_stream().wait_event(ev)
            if self.guard_event is not None:
                torch.cuda.current_stream().wait_event(self.guard_event)
        self._mark("step end")


class DistributedOptimizer(DistributedOptimizerBase):
    """DistributedOptimizer(backend, opt): averages gradients over the workers, then applies `opt`
    (public_api.jl:286-294).  Gradients that a GradBuckets sink already averaged are not reduced twice."""

    def __init__(self, backend, opt, buckets: GradBuckets | None = None):
        self.backend, self.opt, self.buckets = backend, opt, buckets

    def all_finite(self, loss_value: float) -> bool:
        """True when the loss is finite on EVERY worker.  A worker that skipped its update alone would leave the
        others waiting in the gradient collectives and let the replicas diverge, so the decision is taken together
        (one scalar all-reduce)."""
        ok = bool(np.isfinite(loss_value))
        if self.backend.size == 1 or self.backend.comm is None:
            return ok
        flag = B200Array(torch.tensor([0.0 if ok else 1.0], dtype=torch.float32, device="cuda"), (1,))
        allreduce(self.backend, flag, "+")
        return float(flag.t.item()) == 0.0

    def check_async_error(self):
        """Raises when NCCL has reported an asynchronous error on the communicator (polled between steps)."""
        if self.backend.comm is None:
            return
        code = C.c_int32(0)
        lib.call("fb_comm_async_error", self.backend.comm, C.byref(code))
        if code.value != 0:
            raise WorkerLost(f"NCCL reported asynchronous error {code.value} on rank {self.backend.rank}")

    def average_gradients(self, opt_state, gmap: dict):
        if self.buckets is not None:
            self.buckets.finish()
            done = set(self.buckets.views.keys())
        else:
            done = set()
        if self.backend.size == 1:
            return
        for k, g in gmap.items():
            if k in done and g.t.data_ptr() == self.buckets.views[k].t.data_ptr():
                continue
            allreduce(self.backend, g, avg)
