"""CPU checks of the host-side mirror: initialisers (test/utils.jl:53-59, 95-104), constructor dimension logic and
the gradient-bucket bookkeeping for parameters that are used more than once."""
import numpy as np
import pytest

import flux_oracle as O


def test_nfan_table():
    """test/utils.jl:53-59."""
    import fluxb200 as F
    assert F.nfan() == (1, 1)
    assert F.nfan(100) == (1, 100)
    assert F.nfan(100, 200) == (200, 100) == F.nfan((100, 200))
    assert F.nfan(2, 30, 40) == (2 * 30, 2 * 40)
    assert F.nfan(2, 3, 40, 50) == (2 * 3 * 40, 2 * 3 * 50)
    assert F.nfan(2, 3, 4, 50, 60) == (2 * 3 * 4 * 50, 2 * 3 * 4 * 60)


def test_glorot_uniform_variance_and_eltype():
    """test/utils.jl:95-104: variance within 10 % of 2 / (fan_in + fan_out); Float32 output."""
    import fluxb200 as F
    F.seed(0)
    for dims in [(1000,), (100, 100), (100, 400), (2, 3, 32, 64), (2, 3, 4, 32, 64)]:
        v = F.glorot_uniform(*dims)
        fan_in, fan_out = F.nfan(*dims)
        s2 = 2 / (fan_in + fan_out)
        assert v.shape == dims and 0.9 * s2 < v.var() < 1.1 * s2
    assert F.glorot_uniform(3, 4, gain=1.5).dtype == np.float32
    # the same stream and scale as the oracle's restatement of src/utils.jl:81-84
    a = F.glorot_uniform(np.random.default_rng(5), 7, 9, gain=2.0)
    b = O.glorot_uniform(np.random.default_rng(5), 7, 9, gain=2.0)
    assert (a == b).all()
    # glorot_uniform(rng; gain) without dims returns a bound initialiser (src/utils.jl:86)
    init = F.glorot_uniform(np.random.default_rng(5), gain=2.0)
    assert (init(7, 9) == b).all()


def test_create_bias():
    """src/utils.jl:537-543."""
    import fluxb200 as F
    w = np.zeros((3, 4), np.float32)
    assert (F.create_bias(w, True, 3) == np.zeros(3, np.float32)).all()
    assert F.create_bias(w, False, 3) is False
    assert F.create_bias(w, np.arange(3.0), 3).dtype == np.float32
    with pytest.raises(F.DimensionMismatch):
        F.create_bias(w, np.zeros(4), 3)


# ------------------------------------------------------------------ the exchange's order of launches, simulated ---
class _FakeStream:
    cuda_stream = 0

    def wait_event(self, ev):
        pass

    def synchronize(self):
        pass


class _FakeEvent:
    def record(self, stream=None):
        pass


class _FakeArr:
    def __init__(self, t, size):
        self.t, self.size, self.ptr = t, tuple(size), None

    def numel(self):
        return self.t.numel()


def _simulated_rank(monkeypatch, rank, world, defer, log):
    """A GradBuckets of one rank with the library, CUDA events and streams replaced by recorders: what is checked is
    the ORDER in which the exchange's kernels are enqueued, which must be the same on every rank (each rank has to
    enqueue the same sequence of barriers) and must hold an update back until the parameter's last reader is
    enqueued."""
    import types

    import torch

    from fluxb200 import distributed as D
    monkeypatch.setattr(D, "B200Array", _FakeArr)
    monkeypatch.setattr(D, "context", lambda: types.SimpleNamespace(handle=None, stream=None))
    monkeypatch.setattr(D.torch.cuda, "Event", _FakeEvent)
    monkeypatch.setattr(D.torch.cuda, "current_stream", lambda: _FakeStream())
    monkeypatch.setattr(D.lib, "call", lambda name, *a: log.append(name))
    backend = types.SimpleNamespace(size=world, rank=rank, comm=None, stream=_FakeStream())
    # three Dense layers (weight + bias) with a LayerNorm (scale, bias) in front of each, parameter order of the model
    mk = lambda *size: _FakeArr(torch.zeros(int(np.prod(size))), size)
    params = []
    for _ in range(3):
        params += [mk(256), mk(256), mk(256, 256), mk(256)]
    gb = D.GradBuckets(backend, params, bucket_mb=0.25)
    assert len(gb.buckets) == 4 and all((b[1] - b[0]) % world == 0 for b in gb.buckets)   # 3 weights + the small leaves
    n = gb.flat.numel()
    gb.pflat, gb.mflat, gb.vflat = (torch.zeros(n) for _ in range(3))
    gb.adam = (types.SimpleNamespace(eta=1e-3, beta=(0.9, 0.999), epsilon=1e-8), torch.zeros(2))
    gb.peer = {"stage": [0] * world, "pflat": [0] * world, "flags": [0] * world, "epoch": torch.zeros(1, dtype=torch.int32),
               "timeout_ms": 10}
    gb.armed, gb.loss, gb.guard, gb.defer_gather = True, object(), types.SimpleNamespace(ptr=None), defer
    return gb, params


@pytest.mark.parametrize("defer", [False, True])
def test_exchange_enqueues_the_same_barriers_on_every_rank_and_holds_updates_back(monkeypatch, defer):
    world = 2
    logs = []
    for rank in range(world):
        log = []
        gb, params = _simulated_rank(monkeypatch, rank, world, defer, log)
        for step in range(2):
            gb.begin_step()
            if defer:
                gb.start_gathers()
            at_step_start = len(log)
            # reverse sweep: Dense pullback reports its weight early (dW enqueued, dX still reads W), then the sweep
            # reports weight and bias; the LayerNorm in front reports scale and bias
            for layer in reversed(range(3)):
                scale, lbias, W, b = params[4 * layer:4 * layer + 4]
                before = len(log)
                gb.ready(W, early=True)
                during = log[before:]
                assert "fb_reduce_slots" in during and "fb_adam_block_dev" not in during, during   # exchange yes, update no
                gb.ready(W)
                assert log[before + len(during):] [:1] == ["fb_adam_block_dev"]                   # released: the update follows
                gb.ready(b)
                gb.ready(lbias)
                gb.ready(scale)
            gb.finish()
            per_step = log[at_step_start:]
            assert per_step.count("fb_adam_block_dev") == 4 and per_step.count("fb_reduce_slots") == 4
            # reduce-scatter push + barrier per bucket; gathers inside the step add a barrier and a push per bucket
            # plus one closing barrier, deferred gathers add one opening barrier and a push + barrier per bucket
            assert per_step.count("fb_peer_push_blocks") == (4 if defer else 8)
            assert per_step.count("fb_peer_barrier") == (4 if defer else 9)
            if defer:
                start = log[at_step_start - 9:at_step_start]
                assert start == ["fb_peer_barrier"] + ["fb_peer_push_blocks", "fb_peer_barrier"] * 4
        logs.append(log)
    assert logs[0] == logs[1]


def test_nccl_fallback_keeps_its_order_and_ignores_early_reports(monkeypatch):
    """Without mapped peer memory the sharded step uses NCCL per bucket (reduce-scatter, Adam, all-gather) and an early
    report of a weight gradient changes nothing; an unarmed sink averages with one all-reduce per bucket."""
    for armed in (True, False):
        log = []
        gb, params = _simulated_rank(monkeypatch, 0, 2, False, log)
        gb.peer, gb.armed = None, armed
        gb.begin_step()
        for layer in reversed(range(3)):
            scale, lbias, W, b = params[4 * layer:4 * layer + 4]
            before = len(log)
            gb.ready(W, early=True)
            assert len(log) == before            # ignored: nothing may start while the dX product still reads W
            for q in (W, b, lbias, scale):
                gb.ready(q)
        gb.finish()
        if armed:
            assert log == ["fb_reduce_scatter", "fb_adam_step_dev", "fb_allgather"] * 4
        else:
            assert log == ["fb_allreduce"] * 4
