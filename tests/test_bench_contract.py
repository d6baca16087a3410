"""bench.py's host side, on CPU: the reference arm's JSON line has the keys the driver reads, ranks
other than 0 print nothing, and the NUMA helper reports instead of failing when NVML has no GPU."""
import argparse
import importlib.util
import json
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reference_arm_line_carries_the_contract_keys(monkeypatch):
    b = _bench()
    lines = []

    class QuickStep:                      # stands in for the timed CPU step: the line, not the speed, is under test
        def __init__(self, sample_batch, threads):
            self.batch = sample_batch

        def __call__(self):
            return 0.25

    monkeypatch.setattr(b, "CpuStep", QuickStep)
    monkeypatch.setattr(b, "emit", lines.append)
    monkeypatch.setenv("RANK", "0")
    b.run_reference(argparse.Namespace(steps=3, warmup=1, gpus=1))
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == b.METRIC and d["unit"] == b.UNIT
    assert d["steps"] == 3 and d["warmup"] == 1 and d["higher_is_better"] is True and d["vs_baseline"] is None
    assert abs(d["value"] - b.CPU_SAMPLE_BATCH / 0.25) < 1e-9 and abs(d["ms_per_step"] - 250.0) < 1e-9
    assert d["config"]["workload"] == "wide_mlp_train_step" and d["config"]["sample_batch"] == b.CPU_SAMPLE_BATCH
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] == (os.cpu_count() or 1) and cb["value"] == d["value"] and "rows" in cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": b.UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_is_silent_on_other_ranks(monkeypatch):
    b = _bench()
    lines = []
    monkeypatch.setattr(b, "CpuStep", lambda *a: (_ for _ in ()).throw(AssertionError("rank 1 must not build the CPU step")))
    monkeypatch.setattr(b, "emit", lines.append)
    monkeypatch.setenv("RANK", "1")
    b.run_reference(argparse.Namespace(steps=3, warmup=1, gpus=2))
    assert lines == []


def test_numa_helper_reports_why_it_did_not_bind():
    b = _bench()
    before = os.sched_getaffinity(0)
    assert b.bind_to_gpu_numa_node(0) is None          # no GPU here: NVML cannot be initialised
    assert os.sched_getaffinity(0) == before
    assert isinstance(b.NUMA_NOTE, str) and b.NUMA_NOTE.startswith("not bound")


def test_flops_per_step_of_the_wide_mlp():
    b = _bench()
    # forward 4 x (2 B W W) + 2 B W C, weight gradients the same, input gradients one wide layer fewer
    B, Wd, C, D = 8192, 4096, 1000, 4
    fwd = D * 2 * B * Wd * Wd + 2 * B * Wd * C
    assert b.flops_per_step(B, Wd, C, D) == fwd + fwd + ((D - 1) * 2 * B * Wd * Wd + 2 * B * Wd * C)
