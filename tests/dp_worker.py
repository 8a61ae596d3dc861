"""Worker of the multi-GPU DistributedUtils test (one process per GPU, launched by torch.distributed.run).

Checks, like the reference's test/ext_distributed scripts: bcast of ones, reduce / allreduce with + and avg against
closed forms (common.jl:19-87), synchronize of a model and optimiser state (synchronized.jl), shard sizes (data.jl),
and that data-parallel training with bucketed, overlapped gradient averaging reproduces a single-process run on
the full batch (optimizer.jl:8-25 extended to the whole model).
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (os.path.join(ROOT, "flux.jl_b200"), os.path.join(ROOT, "oracle")):
    sys.path.insert(0, p)
import fluxb200 as F  # noqa: E402
import flux_oracle as O  # noqa: E402

DU = F.DistributedUtils


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    backend = DU.initialize(DU.NCCLBackend, device=local)
    assert DU.local_rank(backend) == rank and DU.total_workers(backend) == world

    # collectives: closed forms
    buf = F.gpu(np.ones(512, np.float32) if rank == 0 else np.zeros(512, np.float32))
    DU.bcast(backend, buf, root=0)
    assert (F.cpu(buf) == 1).all()
    tot = sum(range(1, world + 1))
    buf = F.gpu(np.full(512, rank + 1.0, np.float32))
    DU.allreduce(backend, buf, "+")
    assert (F.cpu(buf) == tot).all()
    buf = F.gpu(np.full(512, rank + 1.0, np.float32))
    DU.allreduce(backend, buf, DU.avg)
    np.testing.assert_allclose(F.cpu(buf), tot / world, rtol=1e-6)
    src, dst = F.gpu(np.full(512, rank + 1.0, np.float32)), F.gpu(np.zeros(512, np.float32))
    DU.allreduce(backend, src, dst, "+")
    assert (F.cpu(dst) == tot).all() and (F.cpu(src) == rank + 1).all()
    buf = F.gpu(np.full(512, rank + 1.0, np.float32))
    DU.reduce(backend, buf, "+", root=0)
    assert (F.cpu(buf) == (tot if rank == 0 else rank + 1)).all()

    # native gradient buckets (fb_bucket_*): leaves marked ready out of order, every bucket averaged exactly once
    import ctypes as C
    from fluxb200 import lib
    ctx = F.context()
    flat = torch.full((1000,), float(rank + 1), device="cuda")
    ends = (C.c_int64 * 3)(256, 640, 1000)
    bset = C.c_void_p()
    lib.call("fb_bucket_create", ctx.handle, backend.comm, C.c_void_p(flat.data_ptr()), 1000, 3, ends, None, C.byref(bset))
    ids = []
    for off, cnt in [(0, 100), (100, 156), (256, 384), (640, 200), (840, 160)]:
        lid = C.c_int32(-1)
        lib.call("fb_bucket_register", bset, off, cnt, C.byref(lid))
        ids.append(lid.value)
    try:
        lib.call("fb_bucket_register", bset, 200, 100, C.byref(C.c_int32()))
        raise AssertionError("a leaf that straddles two buckets must be rejected")
    except lib.FluxB200Error:
        pass
    for step in range(2):
        flat.fill_(float(rank + 1) * (step + 1))
        lib.call("fb_bucket_begin_step", bset)
        for lid in (ids[4], ids[2], ids[0], ids[4], ids[1]):     # the last bucket completes first; ids[3] is never marked
            lib.call("fb_bucket_mark_ready", bset, lid, ctx.stream)
        lib.call("fb_bucket_wait", bset, ctx.stream)              # starts the bucket that was still pending
        torch.cuda.synchronize()
        np.testing.assert_allclose(flat.cpu().numpy(), (step + 1) * tot / world, rtol=1e-6)
    lib.call("fb_bucket_destroy", bset)

    # data container: contiguous ceil(n/N) shards whose sizes add up
    nobs = 5 * world - 1                       # a ragged split in which every worker still owns observations
    data = np.arange(nobs * 7, dtype=np.float32).reshape(7, nobs)
    ddc = DU.DistributedDataContainer(backend, data)
    per = int(np.ceil(nobs / world))
    assert len(ddc) == min(per, max(nobs - rank * per, 0)) and len(ddc) >= 1
    cnt = torch.tensor([len(ddc)], dtype=torch.float64)
    if world > 1:
        torch.distributed.all_reduce(cnt)
    assert int(cnt.item()) == nobs

    # data-parallel training == single-process training on the full batch
    rng = np.random.default_rng(7)             # same stream on every rank
    Dm, Cc, NB, GB, steps = 256, 24, 2, 64, 3
    blocks = [{"gamma": (rng.normal(size=Dm) * 0.1 + 1).astype(np.float32), "beta": (rng.normal(size=Dm) * 0.1).astype(np.float32),
               "W": O.glorot_uniform(rng, Dm, Dm), "b": np.zeros(Dm, np.float32)} for _ in range(NB)]
    head = {"W": O.glorot_uniform(rng, Cc, Dm), "b": np.zeros(Cc, np.float32)}
    x = rng.standard_normal((Dm, GB), dtype=np.float32)
    labels = rng.integers(1, Cc + 1, size=GB)
    layers = []
    for blk in blocks:
        ln = F.LayerNorm(Dm)
        # every rank but 0 starts from different values; synchronize must overwrite them
        scale = blk["gamma"] if rank == 0 else blk["gamma"] * 0 + 5
        ln.diag.scale, ln.diag.bias = F.gpu(scale), F.gpu(blk["beta"])
        layers += [ln, F.Dense(blk["W"] if rank == 0 else blk["W"] * 0, blk["b"], "gelu")]
    layers.append(F.Dense(head["W"], head["b"]))
    model = F.Chain(*layers)
    DU.synchronize(backend, DU.FluxDistributedModel(model))
    np.testing.assert_array_equal(F.cpu(model.layers[1].weight), blocks[0]["W"])
    np.testing.assert_array_equal(F.cpu(model.layers[0].diag.scale), blocks[0]["gamma"])
    params = F.trainables(model)
    buckets = DU.GradBuckets(backend, params, bucket_mb=0.2)     # several buckets even for this small model
    assert len(buckets.buckets) >= 3
    opt = F.setup(DU.DistributedOptimizer(backend, F.Adam(1e-3), buckets), model)
    DU.synchronize(backend, opt)
    idx = DU.shard_indices(GB, world, rank)
    xg, yg = F.gpu(np.ascontiguousarray(x[:, idx])), F.onehotbatch(labels[idx], Cc)

    to64 = lambda d: {k: v.astype(np.float64) for k, v in d.items()}
    b64, h64 = [to64(b) for b in blocks], to64(head)
    st_b = [{k: O.adam_init(v) for k, v in b.items()} for b in b64]
    st_h = {k: O.adam_init(v) for k, v in h64.items()}
    y1h = O.onehotbatch(labels, Cc, np.float64)
    for step in range(steps):
        buckets.begin_step()
        l, gs = F.withgradient(lambda m: F.logitcrossentropy(m(xg), yg), model, grad_sink=buckets)
        F.update(opt, model, gs[0])
        lref, gb, gh = O.dp_mlp_fwd_bwd(b64, h64, x.astype(np.float64), y1h)
        # the mean of the per-rank local means equals the full-batch mean for equal shards
        lsum = torch.tensor([l], dtype=torch.float64)
        if world > 1:
            torch.distributed.all_reduce(lsum)
        assert abs(lsum.item() / world - lref) < 1e-4 * abs(lref), (lsum.item() / world, lref)
        if step == 0:
            # averaged gradients (read back from the bucket views) against the full-batch oracle gradients
            g0 = F.cpu(buckets.views[id(model.layers[1].weight)])
            np.testing.assert_allclose(g0, gb[0]["W"], rtol=2e-4, atol=2e-4 * np.abs(gb[0]["W"]).max())
            gl = F.cpu(buckets.views[id(model.layers[0].diag.scale)])
            np.testing.assert_allclose(gl, gb[0]["gamma"], rtol=2e-4, atol=2e-4 * np.abs(gb[0]["gamma"]).max())
        for blk, g, st in zip(b64, gb, st_b):
            for k in blk:
                blk[k] = O.adam_apply(st[k], blk[k], g[k])
        for k in h64:
            h64[k] = O.adam_apply(st_h[k], h64[k], gh[k])
    # replicas stay identical across ranks (bitwise: every rank applies the same averaged gradients)
    w = model.layers[1].weight
    chk = torch.stack([w.t.double().sum(), (w.t.double() ** 2).sum()]).cpu()
    lo, hi = chk.clone(), chk.clone()
    if world > 1:
        torch.distributed.all_reduce(lo, op=torch.distributed.ReduceOp.MIN)
        torch.distributed.all_reduce(hi, op=torch.distributed.ReduceOp.MAX)
    assert torch.equal(lo, hi), "replicas diverged"
    assert np.max(np.abs(F.cpu(w) - b64[0]["W"])) < 3.5e-3        # within the three Adam steps' reach of the oracle
    assert F.context().device_error() == 0

    # N-GPU parameters after k steps == a 1-GPU run on the full batch (same library, no communication), leaf by leaf.
    # Adam's first steps move every element by ~eta * sign(g): an element whose gradient is within rounding of zero
    # can take the other sign in the two runs, so the bulk (99.9 %) is held to 2e-5 and the rest to the steps' reach.
    solo = F.Chain(*([l for blk in blocks for l in (F.LayerNorm(Dm), F.Dense(blk["W"], blk["b"], "gelu"))] + [F.Dense(head["W"], head["b"])]))
    for i, blk in enumerate(blocks):
        solo.layers[2 * i].diag.scale, solo.layers[2 * i].diag.bias = F.gpu(blk["gamma"]), F.gpu(blk["beta"])
    sopt = F.setup(F.Adam(1e-3), solo)
    xf, yf = F.gpu(x), F.onehotbatch(labels, Cc)
    for step in range(steps):
        _, gs = F.withgradient(lambda m: F.logitcrossentropy(m(xf), yf), solo)
        F.update(sopt, solo, gs[0])
    for pd, ps in zip(F.trainables(model), F.trainables(solo)):
        diff = np.abs(F.cpu(pd).astype(np.float64) - F.cpu(ps)).ravel()
        assert np.quantile(diff, 0.999) < 2e-5 and diff.max() < 3.5e-3, (pd.size, np.quantile(diff, 0.999), diff.max())

    # one-launch train step: sharded optimiser (reduce-scatter, Adam on this rank's block, all-gather, all inside the
    # bucket launches) against all-reduce + Adam on every rank
    def build():
        ls = []
        for blk in blocks:
            ln = F.LayerNorm(Dm)
            ln.diag.scale, ln.diag.bias = F.gpu(blk["gamma"]), F.gpu(blk["beta"])
            ls += [ln, F.Dense(blk["W"], blk["b"], "gelu")]
        ls.append(F.Dense(head["W"], head["b"]))
        return F.Chain(*ls)

    runs = []
    for shard, defer in ((False, False), (True, False), (True, True)):
        m = build()
        bk = DU.GradBuckets(backend, F.trainables(m), bucket_mb=0.2)
        o = F.setup(DU.DistributedOptimizer(backend, F.Adam(1e-3), bk), m)
        gs = F.GraphedTrainStep(lambda mm, xx, yy: F.logitcrossentropy(mm(xx), yy), m, o, (xg, yg), grad_sink=bk,
                                shard_optimizer=shard, defer_gather=defer)
        assert gs.sharded == (shard and world > 1)
        losses = [gs(xg, yg) for _ in range(3)]
        gs.sync_params()          # deferred gathers: the peers' blocks of the last update arrive now
        runs.append((m, losses))
    (ma, la), (mb, lb), (mc, lc) = runs
    np.testing.assert_allclose(la, lb, rtol=1e-5)
    np.testing.assert_allclose(la, lc, rtol=1e-5)
    assert la[2] < la[0]
    for pa, pb, pc in zip(F.trainables(ma), F.trainables(mb), F.trainables(mc)):
        np.testing.assert_allclose(F.cpu(pb), F.cpu(pa), rtol=0, atol=3e-6)
        np.testing.assert_allclose(F.cpu(pc), F.cpu(pa), rtol=0, atol=3e-6)
    wb = mb.layers[1].weight
    chk = torch.stack([wb.t.double().sum(), (wb.t.double() ** 2).sum()]).cpu()
    lo, hi = chk.clone(), chk.clone()
    if world > 1:
        torch.distributed.all_reduce(lo, op=torch.distributed.ReduceOp.MIN)
        torch.distributed.all_reduce(hi, op=torch.distributed.ReduceOp.MAX)
    assert torch.equal(lo, hi), "replicas diverged under the sharded optimiser"
    assert F.context().device_error() == 0

    # a non-finite loss on ONE worker: every worker skips the update (the reference decides per process, train.jl:377,
    # which would leave the other workers' collectives without a partner and let the replicas diverge)
    if world > 1:
        bad = rank == world - 1
        xbad = F.gpu(np.full(F.cpu(xg).shape, np.inf, np.float32)) if bad else xg
        for shard in (False, True):
            m = build()
            bk = DU.GradBuckets(backend, F.trainables(m), bucket_mb=0.2)
            o = F.setup(DU.DistributedOptimizer(backend, F.Adam(1e-3), bk), m)
            gs = F.GraphedTrainStep(lambda mm, xx, yy: F.logitcrossentropy(mm(xx), yy), m, o, (xg, yg), grad_sink=bk,
                                    shard_optimizer=shard, defer_gather=shard)
            gs.sync_params()
            before = [F.cpu(q).copy() for q in F.trainables(m)]
            loss = gs(xbad, yg)
            gs.sync_params()
            assert np.isfinite(loss) != bad
            for q, b in zip(F.trainables(m), before):
                assert np.array_equal(F.cpu(q), b), "a worker updated although another worker's loss was not finite"
            gs(xg, yg)             # the next finite step updates again, on every worker
            gs.sync_params()
            assert not np.array_equal(F.cpu(F.trainables(m)[0]), before[0])
        m = build()
        bk = DU.GradBuckets(backend, F.trainables(m), bucket_mb=0.2)
        o = F.setup(DU.DistributedOptimizer(backend, F.Adam(1e-3), bk), m)
        before = [F.cpu(q).copy() for q in F.trainables(m)]
        F.trainstep(lambda mm, xx, yy: F.logitcrossentropy(mm(xx), yy), m, (xbad, yg), o)
        for q, b in zip(F.trainables(m), before):
            assert np.array_equal(F.cpu(q), b)
    assert F.context().device_error() == 0
    if rank == 0:
        print("dp_worker ok", world)


if __name__ == "__main__":
    main()
