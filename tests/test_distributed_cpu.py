"""CPU checks of the data-parallel host logic with two gloo ranks: shard bookkeeping of DistributedUtils and the
identity 'mean of per-shard gradients == full-batch gradient' the gradient averaging relies on."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import flux_oracle as O


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fluxb200.distributed import shard_indices
        rng = np.random.default_rng(3)
        D, C, N = 12, 5, 16
        blocks = [{"gamma": rng.normal(size=D) + 1, "beta": rng.normal(size=D), "W": rng.normal(size=(D, D)) * .3, "b": rng.normal(size=D) * .1}]
        head = {"W": rng.normal(size=(C, D)) * .3, "b": np.zeros(C)}
        x, labels = rng.normal(size=(D, N)), rng.integers(1, C + 1, size=N)
        idx = shard_indices(N, world, rank)
        assert (idx == O.distributed_shard_indices(N, world, rank)).all()
        loss, gb, gh = O.dp_mlp_fwd_bwd(blocks, head, x[:, idx], O.onehotbatch(labels[idx], C, np.float64))
        t = torch.from_numpy(np.concatenate([gb[0]["W"].ravel(), gb[0]["gamma"], gh["W"].ravel(), [loss]]))
        dist.all_reduce(t)           # gradient mean-allreduce: sum, then divide by the number of workers
        t /= world
        lf, gbf, ghf = O.dp_mlp_fwd_bwd(blocks, head, x, O.onehotbatch(labels, C, np.float64))
        ref = np.concatenate([gbf[0]["W"].ravel(), gbf[0]["gamma"], ghf["W"].ravel(), [lf]])
        np.testing.assert_allclose(t.numpy(), ref, rtol=1e-10, atol=1e-12)
        # broadcast from root (synchronize): everyone ends with rank 0's values
        p = torch.full((7,), float(rank + 1))
        dist.broadcast(p, src=0)
        assert (p == 1).all()
        out.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        out.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_average_to_the_full_batch_gradient():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29400 + os.getpid() % 500
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(0, "ok"), (1, "ok")], res


def _sharded_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # a flat "bucket" whose length divides by the number of workers; every rank holds a different local gradient
        n = 64 * world
        rng = np.random.default_rng(5)
        p0 = rng.normal(size=n)
        g_all = rng.normal(size=(world, n))
        blk = n // world
        lo, hi = rank * blk, (rank + 1) * blk
        # route A (the reference's DistributedOptimizer): all-reduce the gradient, Adam on every rank
        pa, sta = p0.copy(), O.adam_init(p0)
        # route B: reduce-scatter, Adam on this rank's block with block-local moments, all-gather of the parameters
        pb, stb = p0.copy(), O.adam_init(p0[lo:hi])
        for step in range(3):
            g_local = g_all[rank] * (1 + step)
            t = torch.from_numpy(g_local.copy())
            dist.all_reduce(t)
            pa = O.adam_apply(sta, pa, t.numpy() / world)
            # gloo has no reduce_scatter: a reduce per destination block gives the same reduced block
            mine = None
            for dst in range(world):
                piece = torch.from_numpy(g_local[dst * blk:(dst + 1) * blk].copy())
                dist.reduce(piece, dst=dst)
                if dst == rank:
                    mine = piece.numpy() / world
            new_block = O.adam_apply(stb, pb[lo:hi], mine)
            gathered = [torch.empty(blk, dtype=torch.float64) for _ in range(world)]
            dist.all_gather(gathered, torch.from_numpy(np.ascontiguousarray(new_block)))
            pb = np.concatenate([x.numpy() for x in gathered])
            np.testing.assert_allclose(pb, pa, rtol=1e-12, atol=1e-14)
        out.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        out.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_sharded_adam_equals_allreduce_adam():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29900 + os.getpid() % 90
    procs = [ctx.Process(target=_sharded_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(0, "ok"), (1, "ok")], res


def test_shard_sizes_with_ragged_split():
    from fluxb200.distributed import shard_indices
    for n, w in [(10, 3), (10, 4), (8192, 8), (7, 2)]:
        shards = [shard_indices(n, w, r) for r in range(w) if r * int(np.ceil(n / w)) < n]
        assert len(shards[0]) == int(np.ceil(n / w))
        assert sum(len(s) for s in shards) == n
        assert (np.concatenate(shards) == np.arange(n)).all()
    with pytest.raises(IndexError):
        shard_indices(4, 8, 7)


# ------------------------------------------------ failure detection on the host (no GPU involved) ---
def _heartbeat_worker(rank, world, port, out):
    """Rank 1 leaves after two steps (between steps, nothing in flight); rank 0 must learn of it on the host, within
    the heartbeat's limit, before it would launch step 3."""
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fluxb200.distributed import Heartbeat, WorkerLost
        store = dist.distributed_c10d._get_default_store()
        hb = Heartbeat(store, rank, world, timeout_s=1.5)
        t = torch.ones(4)
        for step in range(2):
            hb.beat()
            dist.all_reduce(t)
        if rank == 1:
            out.put((rank, "left"))
            return
        t0 = time.monotonic()
        try:
            hb.beat()
            out.put((rank, "no error"))
        except WorkerLost as e:
            dt = time.monotonic() - t0
            out.put((rank, "lost" if (1.4 < dt < 10 and "1 of 2 workers" in str(e) and e.code == -6) else f"bad: {dt} {e}"))
    except Exception as e:  # noqa: BLE001
        out.put((rank, repr(e)))
    finally:
        if rank == 1:
            time.sleep(3.0)   # keep the store's peer alive while rank 0 polls it
        dist.destroy_process_group()


def test_a_worker_that_never_arrives_is_reported_on_the_host_in_time():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29700 + os.getpid() % 200
    procs = [ctx.Process(target=_heartbeat_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(0, "lost"), (1, "left")], res


def test_mismatched_bucket_layout_is_reported_before_any_collective():
    from fluxb200.distributed import WorkerLost, verify_layout
    store = dist.HashStore()
    layout_a = (((0, 1024), (1024, 4096)), (1024, 3072), 2)
    layout_b = (((0, 2048), (2048, 4096)), (2048, 2048), 2)
    store.set("fluxb200/layout/1", __import__("hashlib").sha256(repr(layout_a).encode()).hexdigest())
    verify_layout(store, 0, 2, layout_a, timeout_s=1.0)                       # same layout: passes
    store2 = dist.HashStore()
    store2.set("fluxb200/layout/1", __import__("hashlib").sha256(repr(layout_b).encode()).hexdigest())
    with pytest.raises(WorkerLost, match="different gradient-bucket layout"):
        verify_layout(store2, 0, 2, layout_a, timeout_s=1.0)
    store3 = dist.HashStore()                                                 # worker 1 never publishes
    with pytest.raises(WorkerLost, match="did not publish"):
        verify_layout(store3, 0, 2, layout_a, timeout_s=0.3)
