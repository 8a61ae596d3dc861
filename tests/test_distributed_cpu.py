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
