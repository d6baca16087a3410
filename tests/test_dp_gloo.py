"""Data-parallel step logic on CPU: two gloo ranks, each with its own shard of the batch, the
gradient bucket summed across ranks and scaled — must equal one process stepping the whole batch."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _shard_grads(rank, world, batch, dims):
    from anneal_b200 import realize as R, workloads as W
    from oracle.binding import OracleExecutor
    R.reset()
    m = W.MLP(batch=batch * world, dims=dims)
    xs = m.x.reshape(batch * world, dims[0])[rank * batch:(rank + 1) * batch]
    ys = m.y.reshape(batch * world, dims[2])[rank * batch:(rank + 1) * batch]
    local = W.MLP(batch=batch, dims=dims)
    local.x, local.y = xs.reshape(-1).copy(), ys.reshape(-1).copy()
    for p, q in zip(local.params, m.params):
        p.value[:] = q.value
    g = local.graph()
    items, out_ids = R.build_schedule(g.targets())
    out = OracleExecutor(1).run(items, R.leaf_inputs(g.targets()))
    return [out[i] for i in out_ids]


def _worker(rank, world, port, batch, dims, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    outs = _shard_grads(rank, world, batch, dims)
    # one contiguous bucket, one all-reduce, scale by 1/world: what ResidentTrainer does on the GPU
    bucket = torch.from_numpy(np.concatenate([o.reshape(-1) for o in outs]))
    dist.all_reduce(bucket, op=dist.ReduceOp.SUM)
    bucket /= world
    if rank == 0:
        q.put(bucket.numpy().copy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_equal_one_big_batch():
    world, batch, dims = 2, 8, (12, 16, 5)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, batch, dims, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    sys.path.insert(0, ROOT)
    from anneal_b200 import realize as R, workloads as W
    from oracle.binding import OracleExecutor
    R.reset()
    m = W.MLP(batch=batch * world, dims=dims)
    g = m.graph()
    items, out_ids = R.build_schedule(g.targets())
    out = OracleExecutor(1).run(items, R.leaf_inputs(g.targets()))
    want = np.concatenate([out[i].reshape(-1) for i in out_ids])
    # mean loss over equal shards averages to the global mean; so do its gradients
    assert np.allclose(got, want, rtol=1e-4, atol=1e-6), float(np.abs(got - want).max())


def test_trainer_bucket_layout_is_aligned():
    from anneal_b200.train import _round_up
    sizes = [4096 * 4096, 4096, 1000 * 4096, 1000, 7]
    offs, total = [], 0
    for s in sizes:
        offs.append(total)
        total += _round_up(s)
    assert all(o % 128 == 0 for o in offs) and total >= sum(sizes)
