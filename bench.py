"""Train-step throughput of the data-parallel wide MLP (f16 storage, f32 accumulation) on N B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints one JSON line. `value` is samples/s with the batch already resident in HBM; `e2e` repeats
the measurement through the public API with the batch in pinned host memory, the host→device copy
and the loss read-back inside the timed region. On one GPU the line also carries `sustained` (the
same step looped for seconds, with the clocks it ran at) and `configs` (the other four benchmark
configurations and the update pass, a few hundred milliseconds each). `--impl reference` times the
CPU restatement of the reference's kernels (the reference itself needs a Go toolchain and a graphics
stack, neither exists here) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "train_step_samples_per_s"
UNIT = "samples/s"
CFG = dict(batch=8192, width=4096, classes=1000, depth=4)


#: DRAM bytes (read + write) of one launch of the dominant kernel from a separate ncu capture; a
#: constant of that capture, not a measurement of this run
PAIR_GEMM_TRAFFIC = {"bytes": 376.5e6, "of": "one 4096x4096x8192 weight-gradient launch under ncu (346.3 MB read + 30.2 MB written), 160 MB algorithmic (operands 128 MB, output 32 MB); a forward launch with its fused bias + GELU: 148.3 + 106.5 MB against 96 MB operands + 128 MB of outputs"}
ROW_CHAIN_TRAFFIC = {"bytes": 775.7e6, "of": "one row_chain launch over 8192x8192 under ncu, 805.3 MB algorithmic"}


def flops_per_step(batch, width, classes, depth):
    fwd = depth * 2 * batch * width * width + 2 * batch * width * classes
    dx = (depth - 1) * 2 * batch * width * width + 2 * batch * width * classes
    return fwd + fwd + dx          # forward, weight gradients, input gradients


class ClockSampler(threading.Thread):
    """Samples SM clock, power and clock-event reasons while the timed region runs: NVML polled every
    few milliseconds (read-only queries), nvidia-smi at its 200 ms minimum when NVML cannot be loaded."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    BITS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.rows, self.proc = index, [], None
        self.sm, self.mx, self.power, self.reasons = [], [], [], set()
        self._stop_flag = threading.Event()
        self.source = None

    def _nvml(self):
        import pynvml as nv
        nv.nvmlInit()
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        idx = self.index
        if vis:
            ids = [v for v in vis.split(",") if v.strip()]
            if idx < len(ids) and ids[idx].strip().isdigit():
                idx = int(ids[idx])
        h = nv.nvmlDeviceGetHandleByIndex(idx)
        mx = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
        self.source = "nvml"
        while not self._stop_flag.is_set():
            self.sm.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
            self.mx.append(float(mx))
            try:
                self.power.append(nv.nvmlDeviceGetPowerUsage(h) / 1000.0)
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for n, bit in self.BITS.items():
                    if r & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(0.004)
        nv.nvmlShutdown()

    def run(self):
        try:
            self._nvml()
            return
        except Exception:
            pass
        try:
            self.source = "nvidia-smi"
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            for line in self.proc.stdout:
                r = [c.strip() for c in line.split(",")]
                if len(r) > 8 and r[1].replace(".", "").isdigit():
                    self.sm.append(float(r[1]))
                    self.mx.append(float(r[2]))
                    for n, v in zip(names, r[5:9]):
                        if v.lower().startswith("active"):
                            self.reasons.add(n)
        except Exception:
            pass

    def reset(self):
        if self.source == "nvml":
            self.sm, self.mx, self.power, self.reasons = [], [], [], set()

    def stop(self):
        self._stop_flag.set()
        if self.proc:
            self.proc.terminate()
        self.join(timeout=2)
        return {"sm_mhz": float(np.median(self.sm)) if self.sm else None, "sm_min_mhz": min(self.sm) if self.sm else None,
                "sm_max_mhz": max(self.mx) if self.mx else None,
                "power_w": float(np.median(self.power)) if self.power else None,
                "reasons": sorted(self.reasons), "samples": len(self.sm), "source": self.source}


NUMA_NOTE = None      # why the binding below did or did not happen; carried in the e2e record


def bind_to_gpu_numa_node(index: int):
    """Restrict this process to the CPUs NVML lists as local to GPU `index`, before any pinned memory is
    allocated, so that the staged batches sit on the GPU's own NUMA node (with one process per GPU all
    ranks otherwise tend to allocate on one socket and share its memory controllers and PCIe root).
    Changes only this process's scheduling mask; returns the CPU list or None (NUMA_NOTE says why)."""
    global NUMA_NOTE
    try:
        import pynvml as nv
        nv.nvmlInit()
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if index < len(ids) and ids[index].isdigit():
                h = nv.nvmlDeviceGetHandleByIndex(int(ids[index]))
            elif index < len(ids):
                h = nv.nvmlDeviceGetHandleByUUID(ids[index].encode() if isinstance(ids[index], str) else ids[index])
            else:
                h = nv.nvmlDeviceGetHandleByIndex(index)
        else:
            h = nv.nvmlDeviceGetHandleByIndex(index)
        words = (os.cpu_count() + 63) // 64
        mask = nv.nvmlDeviceGetCpuAffinity(h, words)
        local = [w * 64 + b for w, m in enumerate(mask) for b in range(64) if (m >> b) & 1]
        allowed = os.sched_getaffinity(0)
        cpus = [c for c in local if c in allowed]
        nv.nvmlShutdown()
        if cpus and len(cpus) < len(allowed):
            os.sched_setaffinity(0, cpus)
            NUMA_NOTE = f"bound to {len(cpus)} of the {len(allowed)} CPUs this process may use ({len(local)} are local to the GPU)"
            return cpus
        NUMA_NOTE = (f"not bound: {len(local)} CPUs are local to the GPU, this process may use {len(allowed)}, "
                     f"{len(cpus)} of them local" + (" (already all local)" if cpus and len(cpus) == len(allowed) else ""))
    except Exception as e:
        NUMA_NOTE = f"not bound: {type(e).__name__}: {e}"
    return None


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return p, "measured"
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


#: rows of the wide MLP's batch that one CPU step computes, in `cpu_baseline` and in `--impl reference` alike
CPU_SAMPLE_BATCH = 2


class CpuStep:
    """One train step of the wide MLP on `sample_batch` rows through the oracle on all host threads.
    The schedule is built once; each call times one run of it."""

    def __init__(self, sample_batch: int, threads: int):
        from anneal_b200 import realize as R, workloads as W
        from anneal_b200.realize import leaf_inputs
        from oracle.binding import OracleExecutor
        R.reset()
        R.MATERIALIZE_CONTRACTION_OPERANDS = True
        try:
            m = W.WideMLP(batch=sample_batch, width=CFG["width"], classes=CFG["classes"], depth=CFG["depth"])
            x, y = m.make_inputs()
            g = m.graph(x, y)
            self.items, _ = R.build_schedule(g.targets())
        finally:
            R.MATERIALIZE_CONTRACTION_OPERANDS = False
        self.inputs = leaf_inputs(g.targets())
        self.ex = OracleExecutor(threads)
        self.batch = sample_batch
        R.reset()

    def __call__(self) -> float:
        t0 = time.perf_counter()
        self.ex.run(self.items, self.inputs)
        return time.perf_counter() - t0


def run_reference(args):
    """The reference arm: the CPU port of the reference's kernels, all host threads, `--warmup` untimed
    and `--steps` timed steps of CPU_SAMPLE_BATCH rows each, cut short when a time budget runs out
    (the line says how many steps were timed)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    budget_s = 150.0
    step = CpuStep(CPU_SAMPLE_BATCH, threads)
    t_start = time.perf_counter()
    warm = 0
    for _ in range(max(args.warmup, 0)):
        step()
        warm += 1
        if time.perf_counter() - t_start > budget_s / 4:
            break
    times = []
    for _ in range(max(args.steps, 1)):
        times.append(step())
        if time.perf_counter() - t_start > budget_s:
            break
    ms = 1e3 * sum(times) / len(times)
    v = CPU_SAMPLE_BATCH / (ms / 1e3)
    desc = f"{CPU_SAMPLE_BATCH} rows of the {CFG['batch']}-row batch per step, full widths, {len(times)} timed steps after {warm} warm-up"
    emit(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": len(times),
        "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": "wide_mlp_train_step", **CFG, "per_gpu_batch": CFG["batch"], "sample_batch": CPU_SAMPLE_BATCH,
                   "steps_requested": args.steps, "warmup_requested": args.warmup, "time_budget_s": budget_s},
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_ours(args):
    import torch
    import torch.distributed as dist
    from anneal_b200 import realize as R, workloads as W
    from anneal_b200.device import Device
    from anneal_b200.train import ResidentTrainer

    # NCCL writes its log to stdout, where rank 0 prints its one JSON line: when a log was asked for and
    # no file was named, send it to stderr instead (the setting itself is left alone)
    if os.environ.get("NCCL_DEBUG") and not os.environ.get("NCCL_DEBUG_FILE"):
        os.environ["NCCL_DEBUG_FILE"] = "/dev/stderr"
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    numa_cpus = bind_to_gpu_numa_node(local) if world > 1 else None
    if world > 1:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    dev = Device(local)
    if world > 1:
        uid = [dev.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        dev.comm_init(rank, world, uid[0])

    def barrier():
        if world > 1:
            dist.barrier()

    if args.gemm_tuning:
        names = ("tile_n", "stages", "group_m", "stream_stores", "single_cta", "whole_tail")
        dev.gemm_defaults(**{n: int(v) for n, v in zip(names, args.gemm_tuning.split(","))})
    model = W.WideMLP(rank=rank, **CFG)
    x, y = model.make_inputs()
    R.reset()
    tr = ResidentTrainer(dev, model, model.lr, world=world, use_graph=not args.no_graph, resident_inputs=True,
                         overlap=not args.no_overlap, shard_update=args.shard_update)
    tr.load_batch(x, y)
    for _ in range(args.warmup):
        tr.step()
    dev.synchronize()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.25)
    sampler.reset()                      # keep only samples taken while the timed steps run
    launches0 = dev.stats()["kernels_launched"]
    dev.timer_start()
    for _ in range(args.steps):
        tr.step()
    ms = dev.timer_stop()
    dev.synchronize()
    barrier()
    launches = dev.stats()["kernels_launched"] - launches0
    graph_replays = dev.stats()["graph_replays"]
    clocks = sampler.stop()
    loss_value = tr.loss()
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    value = CFG["batch"] * world * args.steps / (ms / 1e3)

    # instrumented re-run of the same steps, eager launches with an event pair around each kernel
    tr_prof = tr
    tr_prof.use_graph = False
    dev.profile(True)
    for _ in range(min(args.steps, 5)):
        tr_prof.step()
    prof = dev.profile_read()
    dev.profile(False)
    tr_prof.use_graph = not args.no_graph
    pk, pk_kind = peaks()
    roof = None
    if "gemm" in prof and prof["gemm"]["total_ms"] > 0:
        gp = prof["gemm"]
        ach = gp["flops"] / (gp["total_ms"] / 1e3) / 1e12
        peak = pk["bf16_tflops"]
        roof = {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak, "traffic": PAIR_GEMM_TRAFFIC["bytes"],
                "traffic_of": PAIR_GEMM_TRAFFIC["of"],
                "peak_kind": f"{pk_kind} burst dense 16-bit", "kernel": "gemm_f16_tcgen05_pair", "launches": gp["launches"],
                "frac_of_sustained_peak": ach / pk.get("bf16_tflops_sustained", peak),
                "avg_launch_ms": gp["total_ms"] / gp["launches"],
                "share_of_kernel_time": gp["total_ms"] / sum(v["total_ms"] for v in prof.values()),
                "how": "instrumented eager re-run of the same steps, CUDA event pair around every launch"}

    # end to end: every step's batch starts in pinned host memory and its loss is read back on the
    # host.  The copy of batch i+1 is issued on the copy stream right after step i is queued (what a
    # data loader does), so it overlaps step i's kernels; the loss read-back then blocks the host.
    R.reset()
    from anneal_b200.device import pinned_array
    tr2 = ResidentTrainer(dev, model, model.lr, world=world, use_graph=not args.no_graph, resident_inputs=True,
                          overlap=not args.no_overlap, shard_update=args.shard_update)
    host = []
    # batches wait in the loader in the stored format: f16 rows (rounded on the host once, as the
    # reference rounds a leaf when it is set) unless --e2e-f32-host asks for float32 rows, which the
    # device then converts
    hdt = np.float32 if args.e2e_f32_host else np.float16
    for _ in range(2):
        xh, yh = pinned_array(x.size, hdt), pinned_array(y.size, hdt)
        xh[:] = x
        yh[:] = y
        host.append((xh, yh))
    e2e_loss = None
    loss_slots = [pinned_array(1), pinned_array(1)]

    def e2e_steps(n):
        # every step: its batch comes up from pinned host memory (copy stream, under the previous
        # step), its loss goes down to the host; the host reads step i-1's loss while step i runs
        # and only the last read waits
        nonlocal e2e_loss
        for i in range(n):
            tr2.step()                       # commits the staged batch, then the captured step
            if i > 0:
                e2e_loss = tr2.loss_wait()   # step i-1's loss: on the host by now
            tr2.loss_begin(loss_slots[i % 2])
            tr2.prefetch(*host[(i + 1) % 2])  # next batch: host -> device behind this step
        e2e_loss = tr2.loss_wait()

    tr2.prefetch(*host[0])
    e2e_steps(max(args.warmup, 1))
    dev.synchronize()
    barrier()
    t0 = time.perf_counter()
    dev.timer_start()
    e2e_steps(args.steps)
    ms2 = dev.timer_stop()
    dev.synchronize()
    wall2 = (time.perf_counter() - t0) * 1e3
    barrier()
    ms2 = max(ms2, wall2)          # the loss read-back blocks the host: take the slower clock
    if world > 1:
        t = torch.tensor([ms2], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms2 = float(t[0])
    e2e = {"value": CFG["batch"] * world * args.steps / (ms2 / 1e3), "unit": UNIT,
           "h2d_bytes_per_step": int((x.size + y.size) * np.dtype(hdt).itemsize), "host_batch_dtype": np.dtype(hdt).name, "d2h_bytes_per_step": 4, "ms_per_step": ms2 / args.steps,
           "how": "batch i+1 copied from pinned host memory on a copy stream while step i runs; every step's loss is copied to the host behind the step and read there while the next step runs",
           "host_cpus_bound": len(numa_cpus) if numa_cpus else None, "host_cpus_note": NUMA_NOTE,
           "loss": e2e_loss}

    # the same step looped for seconds: what the clocks settle at under the power limit, and the
    # step rate there (the burst above lasts tens of milliseconds)
    sustained = None
    if world == 1 and args.sustained_s > 0:
        n_sus = max(50, int(args.sustained_s * 1e3 / (ms / args.steps)))
        s2 = ClockSampler(local)
        s2.start()
        time.sleep(0.25)
        for _ in range(20):
            tr.step()
        dev.synchronize()
        s2.reset()
        dev.timer_start()
        for _ in range(n_sus):
            tr.step()
        ms_sus = dev.timer_stop()
        ck = s2.stop()
        per = ms_sus / n_sus
        tf = flops_per_step(**CFG) / (per / 1e3) / 1e12
        sustained = {"steps": n_sus, "seconds": ms_sus / 1e3, "ms_per_step": per, "value": CFG["batch"] / (per / 1e3), "unit": UNIT,
                     "step_tflops": tf, "frac_of_sustained_peak": tf / pk.get("bf16_tflops_sustained", pk["bf16_tflops"]),
                     "peak_sustained_tflops": pk.get("bf16_tflops_sustained"), "clocks": ck,
                     "ms_times_sm_mhz": per * ck["sm_mhz"] if ck.get("sm_mhz") else None,
                     "burst_ms_times_sm_mhz": (ms / args.steps) * clocks["sm_mhz"] if clocks.get("sm_mhz") else None,
                     "note": "whole-step FLOP rate (contractions and everything else) against the sustained dense 16-bit GEMM peak; clocks sampled, never set"}

    # the other configurations and the update pass, a few hundred milliseconds each
    configs = None
    if world == 1 and not args.no_configs:
        configs = {}
        for name, (st, wu) in {"mlp": (300, 20), "cnn": (100, 10), "softmax": (30, 5), "sgd": (30, 5), "dynmlp": (20, 3)}.items():
            try:
                r = measure_other(dev, name, st, wu)
                configs[name] = {k: r[k] for k in ("metric", "unit", "value", "ms_per_step", "dtype", "config", "steps", "gpu_launches") if k in r}
                if "roofline" in r:
                    configs[name]["roofline"] = r["roofline"]
            except Exception as e:                      # a failing side measurement must not lose the headline line
                configs[name] = {"error": str(e)[:300]}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        step = CpuStep(CPU_SAMPLE_BATCH, threads)
        step()                                # one untimed step
        dts = [step() for _ in range(2)]
        dt = sum(dts) / len(dts)
        cpu = {"value": CPU_SAMPLE_BATCH / dt, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": f"{CPU_SAMPLE_BATCH} rows of the {CFG['batch']}-row batch per step, full widths, 2 timed steps after 1 warm-up ({dt:.1f} s per step); the same sample as --impl reference"}

    if rank == 0:
        fl = flops_per_step(**CFG)
        out = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": "wide_mlp_train_step", **CFG, "per_gpu_batch": CFG["batch"], "global_batch": CFG["batch"] * world,
                       "parallelism": f"dp{world}", "update": ("sharded" if world > 1 and args.shard_update and not args.no_overlap else "replicated"), "l2": "working set 1.6 GB per step exceeds the 126 MB L2",
                       "optimizer": "sgd lr=1e-3 on f32 masters, in the timed region", "loss": loss_value},
            "e2e": e2e, "gpu_launches": int(launches), "graph_replays": int(graph_replays), "clocks": clocks,
            "step_tflops": fl * world / (ms / args.steps / 1e3) / 1e12,
            "roofline": roof, "cpu_baseline": cpu, "sustained": sustained, "configs": configs,
            "fused": {k: int(dev.stats()[k]) for k in ("epilogues_fused", "colsums_fused")},
            "kernel_classes": {k: {"launches": v["launches"], "ms": round(v["total_ms"], 3)} for k, v in prof.items()},
        }
        emit(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    dev.close()


def measure_other(dev, workload, steps, warmup, materialize=-1, dyn_batches="1,17,256,4096,65536"):
    """One of the other four configurations (or the update pass) on one GPU: samples/s, or GB/s for
    the bandwidth-bound ones, with inputs resident, timed with CUDA events over graph replays."""
    from anneal_b200 import realize as R, workloads as W
    from anneal_b200.train import ResidentTrainer
    from anneal_b200.uop import dtypes

    class A:
        pass
    args = A()
    args.workload, args.steps, args.warmup, args.materialize, args.dyn_batches = workload, steps, warmup, materialize, dyn_batches
    launches0 = dev.stats()["kernels_launched"]
    out = {"data": "synthetic", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True}
    if args.workload in ("mlp", "cnn"):
        m = W.MLP() if args.workload == "mlp" else W.SmallCNN()
        # the im2col of a convolution is a 9- or 72-term padded sum: as an operand expression it is
        # re-evaluated inside every step of the contraction's reduce loop, as a buffer it is written once
        mat = "auto" if args.materialize < 0 or args.materialize == 2 else bool(args.materialize)
        tr = ResidentTrainer(dev, m, m.lr, use_graph=True, materialize=mat, resident_inputs=True)
        tr.load_batch(m.x, m.y)
        for _ in range(args.warmup):
            tr.step()
        dev.synchronize()
        dev.timer_start()
        for _ in range(args.steps):
            tr.step()
        ms = dev.timer_stop()
        out.update(metric=METRIC, unit=UNIT, value=m.batch * args.steps / (ms / 1e3), ms_per_step=ms / args.steps, dtype="f32",
                   config={"workload": args.workload + "_train_step", "batch": m.batch, "kernels_per_step": len(tr.items), "loss": tr.loss(),
                           "contraction_operands_materialized": mat})
    elif args.workload == "softmax":
        s = W.SoftmaxFwdBwd(8192, 8192)
        ts, ins = s.graph()
        items, out_ids = R.build_schedule(ts)
        xb = dev.buffer(dtypes.float32, s.x.size).upload(s.x)
        gb = dev.buffer(dtypes.float32, s.g.size).upload(s.g)
        ob = dev.buffer(dtypes.float32, s.x.size)
        inputs = {ins["x"].node.idx: xb, ins["g"].node.idx: gb}
        placed = {out_ids[0]: ob}
        for _ in range(args.warmup):
            dev.replay(items, inputs, None, placed)
        dev.synchronize()
        dev.timer_start()
        for _ in range(args.steps):
            dev.replay(items, inputs, None, placed)
        ms = dev.timer_stop()
        for bb in (xb, gb, ob):
            bb.release()
        algo = 3 * s.x.size * 4
        pk, kind = peaks()
        gbs = algo * args.steps / (ms / 1e3) / 1e9
        out.update(metric="softmax_fwd_bwd_hbm_gbs", unit="GB/s", value=gbs, ms_per_step=ms / args.steps, dtype="f32",
                   config={"workload": "softmax_fwd_bwd_8192x8192", "kernels_per_step": len(items), "algorithmic_bytes": algo},
                   roofline={"bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"],
                             "traffic": ROW_CHAIN_TRAFFIC["bytes"], "traffic_of": ROW_CHAIN_TRAFFIC["of"],
                             "peak_kind": kind + " copy", "kernel": "row_chain",
                             "note": "the whole schedule is this one launch; timed over graph replays"})
    elif args.workload == "sgd":
        # the fused SGD + re-quantise pass alone, over the wide MLP's parameter count: f32 masters and
        # f16 gradients read, f32 masters and f16 parameters written (12 bytes per parameter)
        n = 71_200_000 // 128 * 128
        mb, pb, gb = dev.buffer(dtypes.float32, n), dev.buffer(dtypes.float16, n), dev.buffer(dtypes.float16, n)
        zeros = np.zeros(n, np.float32)
        for b in (mb, pb, gb):
            b.upload(zeros)
        for _ in range(args.warmup):
            dev.sgd_step(mb, pb, gb, 1e-3, 1.0)
        dev.synchronize()
        dev.timer_start()
        for _ in range(args.steps):
            dev.sgd_step(mb, pb, gb, 1e-3, 1.0)
        ms = dev.timer_stop()
        for bb in (mb, pb, gb):
            bb.release()
        algo = n * 12
        pk, kind = peaks()
        gbs = algo * args.steps / (ms / 1e3) / 1e9
        out.update(metric="sgd_update_hbm_gbs", unit="GB/s", value=gbs, ms_per_step=ms / args.steps, dtype="f32",
                   config={"workload": "sgd_update_71.2M_params", "algorithmic_bytes": algo, "l2": "854 MB per pass exceeds the 126 MB L2"},
                   roofline={"bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"],
                             "traffic": None, "peak_kind": kind + " copy", "kernel": "sgd_kernel"})
    elif args.workload == "dynmlp":
        m = W.DynMLP()
        res = {}
        R.DEFAULT_EXECUTOR = dev
        R.MATERIALIZE_CONTRACTION_OPERANDS = True
        batches = [int(v) for v in args.dyn_batches.split(",")]
        for b in batches:
            R.reset()
            x, y = m.inputs(b)
            outt, loss, grads, ins = m.graph(b)
            items, out_ids = R.build_schedule([outt] + grads)
            bufs = {}
            for t, d in ((ins["x"], x), (ins["y"], y)):
                bufs[t.node.idx] = dev.buffer(dtypes.float32, d.size).upload(d)
            for p in m.params:
                bufs[p.t.node.idx] = dev.buffer(dtypes.float32, p.value.size).upload(p.value)
            placed = {}
            for oid, it in ((o, next(i for i in items if i.bufs[0].uop_idx == o)) for o in out_ids):
                n = int(np.prod([d if d else b for d in it.bufs[0].shape])) if it.bufs[0].shape else 1
                placed[oid] = dev.buffer(dtypes.float32, n)
            steps = max(2, args.steps if b <= 4096 else 2)
            for _ in range(2):
                dev.replay(items, bufs, {"n": b}, placed)
            dev.synchronize()
            dev.timer_start()
            for _ in range(steps):
                dev.replay(items, bufs, {"n": b}, placed)
            ms = dev.timer_stop() / steps
            res[str(b)] = {"us_per_replay": ms * 1e3, "samples_per_s": b / (ms / 1e3), "tflops": 42e6 * b / (ms / 1e3) / 1e12}
            for v in list(bufs.values()) + list(placed.values()):
                v.release()
        R.DEFAULT_EXECUTOR = None
        R.MATERIALIZE_CONTRACTION_OPERANDS = False
        out.update(metric=METRIC, unit=UNIT, value=res[str(batches[-1])]["samples_per_s"], ms_per_step=res[str(batches[-1])]["us_per_replay"] / 1e3, dtype="f32",
                   config={"workload": "dynmlp_symbolic_batch", "per_batch": res, "nvrtc_compiles": dev.stats()["nvrtc_compiles"]})
    out["gpu_launches"] = int(dev.stats()["kernels_launched"] - launches0)
    R.reset()
    return out


def run_other(args):
    from anneal_b200.device import Device
    dev = Device(int(os.environ.get("LOCAL_RANK", "0")))
    emit(json.dumps(measure_other(dev, args.workload, args.steps, args.warmup, args.materialize, args.dyn_batches)))
    dev.close()


_REAL_STDOUT = None


def keep_stdout_for_the_json_line():
    """Libraries below (NCCL prints its version and, when asked, its log on stdout) must not share
    the stream on which the one JSON line goes out: file descriptor 1 is pointed at stderr for the
    life of the process and the line is written through a saved copy."""
    global _REAL_STDOUT
    if _REAL_STDOUT is None:
        sys.stdout.flush()
        _REAL_STDOUT = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)


def emit(line: str):
    out = _REAL_STDOUT or sys.stdout
    out.write(line + "\n")
    out.flush()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="wide_mlp", choices=["wide_mlp", "mlp", "cnn", "softmax", "dynmlp", "sgd"],
                    help="wide_mlp is the headline configuration; the others print a one-GPU line for the remaining configurations")
    ap.add_argument("--shard-update", action="store_true", help="N>1: reduce-scatter, update this rank's shard, all-gather, instead of all-reducing and updating everything on every rank (measured slower on 8 GPUs: 3.82 against 3.64 ms per step)")
    ap.add_argument("--dyn-batches", default="1,17,256,4096,65536", help="dynmlp: batch sizes bound in turn; the last one is reported")
    ap.add_argument("--materialize", type=int, default=-1, help="mlp/cnn: 1/0 forces contraction operands to be buffers or expressions; default: decided per operand by cost")
    ap.add_argument("--e2e-f32-host", action="store_true", help="e2e: host batches as float32 rows (converted on the device) instead of rows already rounded to the f16 storage format")
    ap.add_argument("--gemm-tuning", default="", help="tile_n,stages,group_m,stream_stores,single_cta,whole_tail for the contraction kernel (0 = heuristic); for A/B runs")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="one GPU: skip the other configurations' side measurements")
    ap.add_argument("--sustained-s", type=float, default=3.0, help="one GPU: seconds the step is looped for the sustained record (0 skips it)")
    ap.add_argument("--no-graph", action="store_true", help="launch kernels one by one instead of replaying a CUDA graph")
    ap.add_argument("--no-overlap", action="store_true", help="all-reduce the whole gradient bucket after the backward pass")
    args = ap.parse_args()
    keep_stdout_for_the_json_line()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload != "wide_mlp":
        run_other(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
