"""Run by `torch.distributed.run` on two GPUs (see test_gpu_multi.py).  Rank 1 leaves cleanly BETWEEN
steps — nothing of its own in flight, nothing on any GPU faults or spins.  Rank 0's next step then
contains an all-reduce that can never finish; the watchdog must end it within the timeout with
ANL_ERR_COMM, later collectives must refuse, and after a new communicator (of one rank) training
must go on.  NVLS is off (NCCL_NVLS_ENABLE=0, set by the launcher) and no kernel of this library uses
multicast memory."""
import os
import signal
import sys
import time

import numpy as np
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from anneal_b200 import realize as R, workloads as W          # noqa: E402
from anneal_b200.device import Device, DeviceError            # noqa: E402
from anneal_b200.train import ResidentTrainer                 # noqa: E402
from anneal_b200.uop import dtypes                            # noqa: E402


def main():
    # whatever happens, no rank outlives this: a stuck process would keep its GPU busy for the next user
    signal.signal(signal.SIGALRM, lambda *_: os._exit(3))
    signal.alarm(120)
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    assert world == 2
    dist.init_process_group("gloo", rank=rank, world_size=world)
    dev = Device(local)
    uid = [dev.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    dev.comm_init(rank, world, uid[0])
    dev.comm_set_timeout(3000)
    m = W.WideMLP(batch=256, width=512, classes=72, depth=2, rank=rank)
    x, y = m.make_inputs()
    # one bucket all-reduce after the backward pass, launched eagerly: exactly ONE collective is in
    # flight when the peer is missing, so the abort has nothing queued behind it to clean up
    tr = ResidentTrainer(dev, m, 0.05, world=world, use_graph=False, resident_inputs=True, overlap=False)
    tr.load_batch(x, y)
    for _ in range(2):
        tr.step()
    first = tr.loss()                 # waits for the device: both ranks have finished two steps
    dist.barrier()
    if rank == 1:
        dev.synchronize()
        dev.close()
        dist.destroy_process_group()
        sys.exit(0)
    # rank 0 does not take part in destroy_process_group's exchange; give the peer time to be gone
    time.sleep(2.0)
    problems = []
    t0 = time.time()
    try:
        tr.step()                      # queues the step; its one all-reduce waits for a peer that is gone
        dev.synchronize()
        problems.append("the step after the peer left did not fail")
    except DeviceError as e:
        waited = time.time() - t0
        if "communicator aborted" not in str(e):
            problems.append(f"unexpected error text: {e}")
        if not (2.0 <= waited <= 15.0):
            problems.append(f"the watchdog took {waited:.1f} s for a 3 s timeout")
    probe = dev.buffer(dtypes.float32, 256)
    try:
        dev.allreduce_sum(probe)
        problems.append("a collective was accepted on the aborted communicator")
    except DeviceError as e:
        if "aborted" not in str(e):
            problems.append(f"unexpected refusal text: {e}")
    # the device itself is fine: a new communicator (this rank alone) and training continues
    dev.synchronize()
    dev.comm_init(0, 1, dev.comm_unique_id())
    R.reset()
    m1 = W.WideMLP(batch=256, width=512, classes=72, depth=2, rank=0)
    solo = ResidentTrainer(dev, m1, 0.05, world=1, use_graph=True, resident_inputs=True)
    solo.load_batch(x, y)
    losses = []
    for _ in range(3):
        solo.step()
        losses.append(solo.loss())
    if not (np.isfinite(losses).all() and losses[-1] < losses[0]):
        problems.append(f"training after recovery did not progress: {losses}")
    dev.synchronize()
    dev.close()
    for p in problems:
        print("RANK_FAILURE problem:", p, flush=True)
    print("RANK_FAILURE", "OK" if not problems else "MISMATCH", f"(first loss {first:.4f})", flush=True)
    os._exit(0 if not problems else 1)       # the gloo group cannot be torn down collectively any more


if __name__ == "__main__":
    main()
