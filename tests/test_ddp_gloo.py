"""World-size-2 checks of the data-parallel step on CPU ranks (gloo): the one collective of the step
(mean all-reduce of the flat gradient bucket) and the property it relies on -- dW of the whole batch
is the sum of the shards' dW, computed here through the oracle (reference CPU operators or the
restatement) so that no GPU is needed."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from snntc_2023_b200 import ddp, nets
        from oracle import ref_model
        specs = [("conv", 2, 4, 3, 1), ("pool", 2), ("flatten",), ("dense", 4 * 3 * 3, 5)]
        weights = nets.spec_weights(specs, 77)
        rng = np.random.default_rng(123)
        B = 6
        x = np.exp(rng.random((B, 6, 6, 2))).astype(np.float32)
        labels = rng.integers(0, 5, B)
        layout, total = ddp.bucket_layout([w.shape for w in weights])
        # this rank's shard: mean loss over ITS samples, gradients written into the flat bucket
        a, b = ddp.shard_bounds(B, rank, world)
        loss, grads, kind = ref_model.train_step(specs, weights, x[a:b], labels[a:b], threads=1)
        flat = torch.zeros(total)
        for (off, n, shape), g in zip(layout, grads):
            flat[off:off + n] = torch.from_numpy(np.ascontiguousarray(g)).reshape(-1)
        ddp.allreduce_mean_(flat, world)
        # every rank must now hold the gradient of the mean loss over the GLOBAL batch
        loss_all, grads_all, _ = ref_model.train_step(specs, weights, x, labels, threads=1, kind=kind)
        want = torch.cat([torch.from_numpy(np.ascontiguousarray(g)).reshape(-1) for g in grads_all])
        err = float((flat - want).norm() / want.norm())
        par = torch.tensor([1.0 + rank, 2.0])
        ddp.broadcast_(par, src=0)
        q.put((rank, err, total, float(par[0]), (a, b)))
    finally:
        dist.destroy_process_group()


def test_flat_bucket_allreduce_world2():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    res.sort()
    assert [r[4] for r in res] == [(0, 3), (3, 6)]
    for rank, err, total, par0, _ in res:
        assert total == (2 * 9 + 1) * 4 + (36 + 1) * 5
        assert err < 1e-5, "rank %d: all-reduced bucket differs from the full-batch gradient (rel %.2e)" % (rank, err)
        assert par0 == 1.0   # broadcast from rank 0


def test_shard_bounds_cover_the_batch():
    from snntc_2023_b200 import ddp
    for n in (1, 7, 256, 1000):
        for world in (1, 2, 3, 8):
            spans = [ddp.shard_bounds(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
