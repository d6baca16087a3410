"""Training loop with device-resident parameters.

The reference's loop (examples/mlp.go:111-142, tensor/nn/nn.go:56-106) rebuilds
the graph every step, re-uploads every weight through ``Parameter.Load`` and
applies SGD on the host. ``ResidentTrainer`` keeps that loop's meaning — f32
master weights, storage-dtype copies re-quantised after each update, plain SGD —
but builds the schedule once (the JIT's job, tensor/jit.go:86-118), keeps
parameters, masters and gradients in three contiguous device buckets, replays
the step as one CUDA graph, all-reduces the gradient bucket across ranks and
updates on the device. Per step only the batch goes up and the loss comes down.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np

from . import realize as R
from .device import Device, GradientTarget, ResidentBuffer, pinned_array
from .uop import dtypes


def _round_up(n: int, m: int = 128) -> int:
    return (n + m - 1) // m * m


class ResidentTrainer:
    def __init__(self, dev: Device, model, lr: float, world: int = 1, use_graph: bool = True,
                 materialize="auto", resident_inputs: bool = False, overlap: bool = True,
                 force_allreduce: bool = False, shard_update: bool = False):
        self.dev, self.model, self.lr, self.world, self.use_graph = dev, model, float(lr), world, use_graph
        # materialize: which contraction operands are written to buffers first — "auto" decides per
        # operand by cost (schedule.materialize_contraction_operands), True all of them, False none
        self.overlap = overlap
        self.shard_update = shard_update
        prev = R.MATERIALIZE_CONTRACTION_OPERANDS
        R.MATERIALIZE_CONTRACTION_OPERANDS = materialize
        try:
            g = model.graph()
            self.items, out_ids = R.build_schedule(g.targets())
        finally:
            R.MATERIALIZE_CONTRACTION_OPERANDS = prev
        self.loss_id, self.grad_ids = out_ids[0], out_ids[1:]
        self.grad_scale = float(g.grad_scale)
        self.x_id, self.y_id = g.inputs["x"].node.idx, g.inputs["y"].node.idx
        self.x_elems = int(np.prod(g.inputs["x"].shape))
        self.y_elems = int(np.prod(g.inputs["y"].shape))
        self.in_dtype = g.inputs["x"].dtype
        params = g.params
        self.params = params
        sdt = params[0].dtype
        offs, total = [], 0
        for p in params:
            offs.append(total)
            total += _round_up(p.value.size)
        self.total = total
        self.master = dev.buffer(dtypes.float32, total)
        self.store = self.master if sdt is dtypes.float32 else dev.buffer(sdt, total)
        self.grad = dev.buffer(sdt, total)
        flat = np.zeros(total, dtype=np.float32)
        for p, o in zip(params, offs):
            flat[o:o + p.value.size] = p.value
        self.master.upload(flat)
        if self.store is not self.master:
            self.store.upload(flat)
        self.offsets = offs
        self.inputs: Dict[int, object] = {}
        self.placed: Dict[int, object] = {}
        self._views = []
        self.fused: Dict[int, object] = {}
        for p, o, gid in zip(params, offs, self.grad_ids):
            pv = self.store.view(o, p.value.size)
            gv = self.grad.view(o, p.value.size)
            mv = self.master.view(o, p.value.size)
            self._views += [pv, gv, mv]
            self.inputs[p.t.node.idx] = pv
            self.placed[gid] = gv
            # overlapped mode: each gradient is all-reduced and applied right behind its kernel
            # across ranks: reduce-scatter the gradient, update this rank's shard of the parameter,
            # all-gather the new values (shard_update), or all-reduce and update everything everywhere
            mode = (2 if shard_update else 1) if (world > 1 or force_allreduce) else 0
            self.fused[gid] = GradientTarget(gv, mv, pv, self.lr, self.grad_scale / world, allreduce=mode)
        self.loss_host = pinned_array(1)
        self.placed[self.loss_id] = self.loss_host
        self.resident_inputs = resident_inputs
        if resident_inputs:
            self.x_res = dev.buffer(self.in_dtype, self.x_elems)
            self.y_res = dev.buffer(self.in_dtype, self.y_elems)
            self.loss_res = dev.buffer(g.loss.dtype, 1)
            self.placed[self.loss_id] = self.loss_res

    def load_batch(self, x: np.ndarray, y: np.ndarray) -> None:
        """Resident-input mode: stage one batch on the device ahead of the timed region."""
        self.x_res.upload(x)
        self.y_res.upload(y)

    def prefetch(self, x: np.ndarray, y: np.ndarray) -> None:
        """Resident-input mode: start moving the NEXT batch to the device on the copy stream while
        the steps already queued run; the following ``step`` picks it up. ``x`` and ``y`` are
        contiguous host arrays (pinned for a truly asynchronous copy) that stay untouched until
        that step has been issued: float32, or float16 when the inputs are stored as f16 (half the
        bytes over PCIe and no conversion pass; rounding to f16 on the host is what the reference
        does when a leaf is set, tensor/tensor.go:58-68)."""
        self.x_res.upload_begin(x)
        self.y_res.upload_begin(y)
        self._staged = True

    def step(self, x: Optional[np.ndarray] = None, y: Optional[np.ndarray] = None) -> Optional[float]:
        inputs = dict(self.inputs)
        if self.resident_inputs and getattr(self, "_staged", False):
            self.x_res.upload_commit()
            self.y_res.upload_commit()
            self._staged = False
        if self.resident_inputs:
            inputs[self.x_id], inputs[self.y_id] = self.x_res, self.y_res
        else:
            inputs[self.x_id], inputs[self.y_id] = x, y
        run = self.dev.replay if self.use_graph else self.dev.run
        if self.overlap:
            placed = dict(self.placed)
            placed.update(self.fused)
            run(self.items, inputs, None, placed)
        else:
            run(self.items, inputs, None, self.placed)
            if self.world > 1:
                self.dev.allreduce_sum(self.grad)
            self.dev.sgd_step(self.master, self.store, self.grad, self.lr, self.grad_scale / self.world)
        return None if self.resident_inputs else float(self.loss_host[0])

    def loss_begin(self, slot: np.ndarray) -> None:
        """Resident-input mode: queue the read-back of the loss of the step just issued into ``slot``
        (one pinned float32) and return at once; the value is there after ``loss_wait``."""
        self.loss_res.download_begin(slot)

    def loss_wait(self) -> float:
        return float(self.loss_res.download_wait()[0])

    def loss(self) -> float:
        if self.resident_inputs:
            return float(self.loss_res.download()[0])
        return float(self.loss_host[0])

    def _named(self, names=None) -> Dict[str, object]:
        names = list(names) if names is not None else [f"param.{i}" for i in range(len(self.params))]
        if len(names) != len(self.params):
            raise ValueError(f"checkpoint: {len(names)} names for {len(self.params)} parameters")
        return dict(zip(names, self.params))

    def save_checkpoint(self, path: str, names=None) -> None:
        """Master weights → host ``Parameter.value`` → safetensors file (tensor/safetensors/safetensors.go:75).
        SGD keeps no optimiser state, so this is all a resume needs."""
        from . import safetensors
        for p, v in zip(self.params, self.parameters()):
            p.value[:] = v
        safetensors.save(path, self._named(names))

    def load_checkpoint(self, path: str, names=None) -> None:
        """safetensors file → host values → master and storage-dtype buckets on the device."""
        from . import safetensors
        safetensors.load(path, self._named(names))
        flat = np.zeros(self.total, dtype=np.float32)
        for p, o in zip(self.params, self.offsets):
            flat[o:o + p.value.size] = p.value
        self.master.upload(flat)
        if self.store is not self.master:
            self.store.upload(flat)

    def parameters(self) -> List[np.ndarray]:
        """Master weights back on the host, one array per parameter (for checkpoints and tests).
        With the update sharded across ranks each rank's f32 masters are current only in its own
        shard of every parameter (the storage-dtype copies are complete): the shards are gathered
        first. Every rank must make this call."""
        if self.world > 1 and self.overlap and self.shard_update and self.store is not self.master:
            for p, o in zip(self.params, self.offsets):
                if p.value.size % self.world == 0:
                    mv = self.master.view(o, p.value.size)
                    self.dev.allgather(mv)
                    self.dev.synchronize()
                    mv.release()
        flat = self.master.download()
        return [flat[o:o + p.value.size].copy() for p, o in zip(self.params, self.offsets)]

    def gradients(self) -> List[np.ndarray]:
        flat = self.grad.download()
        return [flat[o:o + p.value.size].copy() for p, o in zip(self.params, self.offsets)]
