"""Run by `torch.distributed.run` on 2+ GPUs (see test_gpu_multi.py): the three ways of applying
the gradients across ranks — sharded update, all-reduce with full update, and one bucket all-reduce
after the backward pass — must leave identical parameters, every rank must hold the same ones, and
N ranks with batch B each must train like ONE rank with the N batches concatenated (same seeds):
the data-parallel step is the big-batch step, up to the f16 rounding of each rank's gradients."""
import os
import sys

import numpy as np
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from anneal_b200 import realize as R, workloads as W          # noqa: E402
from anneal_b200.device import Device                         # noqa: E402
from anneal_b200.train import ResidentTrainer                 # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    dev = Device(local)
    uid = [dev.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    dev.comm_init(rank, world, uid[0])
    dev.comm_set_timeout(60000)
    results = []
    for overlap, shard in ((True, True), (True, False), (False, False)):
        R.reset()
        m = W.WideMLP(batch=512, width=2048, classes=72, depth=2, rank=rank)
        x, y = m.make_inputs()
        tr = ResidentTrainer(dev, m, 0.05, world=world, use_graph=overlap, resident_inputs=True, overlap=overlap, shard_update=shard)
        tr.load_batch(x, y)
        for _ in range(3):
            tr.step()
        results.append(np.concatenate(tr.parameters()))
        dist.barrier()
    ok = True
    # two ranks: a + b is the same in any order, so the three modes agree bit for bit;
    # more ranks: the collectives may sum in different orders, f16 gradients differ in the last place
    tol = 0.0 if world == 2 else 1e-3
    for k, r in enumerate(results[1:]):
        d = float(np.abs(r - results[0]).max())
        if d > tol * max(1.0, float(np.abs(results[0]).max())):
            ok = False
            print(f"rank {rank}: mode {k + 1} differs from the sharded update by {d:.3e}", flush=True)
    gathered = [None] * world
    dist.all_gather_object(gathered, results[0].tobytes())
    if not all(g == gathered[0] for g in gathered):
        ok = False
        if rank == 0:
            print("ranks hold different parameters after the sharded update", flush=True)
    # one rank, batch N*B: the same samples in rank order, through the same trainer without a collective
    if rank == 0:
        R.reset()
        B = 512
        big = W.WideMLP(batch=world * B, width=2048, classes=72, depth=2)
        parts = [W.WideMLP(batch=B, width=2048, classes=72, depth=2, rank=r).make_inputs() for r in range(world)]
        xb = np.concatenate([p[0] for p in parts])
        yb = np.concatenate([p[1] for p in parts])
        one = ResidentTrainer(dev, big, 0.05, world=1, use_graph=True, resident_inputs=True)
        one.load_batch(xb, yb)
        for _ in range(3):
            one.step()
        ref = np.concatenate(one.parameters())
        start = np.concatenate([p.value for p in big.params])
        moved = float(np.abs(ref - start).max())
        d = float(np.abs(results[1] - ref).max())
        # each rank rounds its own gradient to f16 before the sum; the big batch rounds once
        if not (moved > 0 and d <= 4e-3 * moved):
            ok = False
            print(f"{world} ranks x batch {B} differ from one rank x batch {world * B} by {d:.3e} (the parameters moved by {moved:.3e})", flush=True)
        else:
            print(f"DP_BIG_BATCH ok: difference {d:.3e}, parameters moved by {moved:.3e}", flush=True)
    dist.barrier()
    flags = [None] * world
    dist.all_gather_object(flags, bool(ok))
    dev.synchronize()
    dev.close()
    dist.destroy_process_group()
    if rank == 0:
        print("DP_CHECK", "OK" if all(flags) else "MISMATCH", flush=True)
    sys.exit(0 if all(flags) else 1)


if __name__ == "__main__":
    main()
