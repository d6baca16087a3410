"""BEAM autotuning of generated kernels (codegen/beam.go): guard, cache determinism, collision guard."""
import os

import numpy as np
import pytest

from anneal_b200 import realize as R
from anneal_b200.device import Device
from anneal_b200.tensor import Tensor
from util import schedule

pytestmark = pytest.mark.gpu


def test_search_improves_or_keeps_and_caches(cuda, tmp_path):
    cache = str(tmp_path / "beam.json")
    x = Tensor.new_leaf((2048, 1024))
    items, _ = R.build_schedule([x.exp2().sum([0])])          # column sums: the layout heuristic is not always best
    r1 = cuda.beam_search(items[0], cache_path=cache)
    assert not r1["from_cache"] and r1["tried"] > 5 and r1["best_us"] <= r1["base_us"] * 1.0001
    r2 = cuda.beam_search(items[0], cache_path=cache)
    assert r2["from_cache"] and r2["opts"] == r1["opts"]       # TestB5 cache determinism
    assert os.path.exists(cache) and '"opts"' in open(cache).read()


def test_elementwise_guard_is_bit_identity(cuda, tmp_path):
    x = Tensor.new_leaf((512, 768))
    items, _ = R.build_schedule([x.mul(x).add(x.sin())])
    r = cuda.beam_search(items[0], cache_path=str(tmp_path / "b.json"))
    assert r["rejected"] == 0          # every block size / vector width gives the same bits


def test_collision_guard_ignores_entries_with_a_different_source(cuda, tmp_path):
    # codegen/beam.go:184-190: an entry whose source hash does not match is not applied
    cache = str(tmp_path / "beam.json")
    x = Tensor.new_leaf((300, 700))
    items, _ = R.build_schedule([x.sum([1])])
    r1 = cuda.beam_search(items[0], cache_path=cache)
    line = open(cache).read().splitlines()[0]
    key = line.split('"key":"')[1][:16]
    with open(cache, "w") as f:
        f.write('{"key":"%s","src":"%016x","opts":[64,1,0,0],"us":0.001}\n' % (key, 0xDEADBEEF))
    other = str(tmp_path / "other.json")          # force a reload from the doctored file
    cuda.beam_search(items[0], cache_path=other)
    r2 = cuda.beam_search(items[0], cache_path=cache)
    assert not r2["from_cache"]


def test_tuned_device_gives_the_same_results(oracle, tmp_path, monkeypatch):
    monkeypatch.setenv("ANNEAL_BEAM_CACHE", str(tmp_path / "beam.json"))
    dev = Device(0, flags=Device.BEAM)
    try:
        rng = np.random.default_rng(0)
        x = Tensor.new_leaf((257, 129)).set_data(rng.standard_normal(257 * 129))
        y = x.exp2().sum([1]).reshape((257, 1)).expand((257, 129)).mul(x)
        items, out_ids, inputs = schedule([y])
        got = dev.run(items, inputs)[out_ids[0]]
        want = oracle.run(items, inputs)[out_ids[0]]
        assert np.abs(got - want).max() <= 1e-4 * np.abs(want).max()
    finally:
        dev.close()


def test_contraction_search_covers_the_tensor_core_kernel(cuda, tmp_path):
    """A dense f16 contraction is searched over the tcgen05 kernel's own tunables (tile width, ring
    depth, raster group, flags); every candidate must reproduce the default configuration's output
    bit for bit, the winner is cached, and a device opened with the search applied gives the same
    values as one without."""
    from anneal_b200.uop import dtypes
    rng = np.random.default_rng(3)
    a = Tensor.new_leaf((1024, 512), dtypes.float16).set_data(rng.standard_normal(1024 * 512) * 0.1)
    w = Tensor.new_leaf((768, 512), dtypes.float16).set_data(rng.standard_normal(768 * 512) * 0.1)
    y = a.matmul(w.permute((1, 0)))
    items, out_ids, inputs = schedule([y])
    cache = str(tmp_path / "gemm_beam.json")
    r1 = cuda.beam_search(items[0], cache_path=cache)
    assert not r1["from_cache"] and r1["tried"] >= 10, r1
    assert r1["rejected"] == 0, r1                       # no tunable reorders a sum
    assert r1["best_us"] <= r1["base_us"] * 1.0001
    r2 = cuda.beam_search(items[0], cache_path=cache)
    assert r2["from_cache"] and r2["opts"] == r1["opts"]
    want = cuda.run(items, inputs)[out_ids[0]]
    os.environ["ANNEAL_BEAM_CACHE"] = cache
    try:
        tuned = Device(0, Device.BEAM)
        try:
            g0 = tuned.stats()["gemm_launched"]
            got = tuned.run(items, inputs)[out_ids[0]]
            assert tuned.stats()["gemm_launched"] - g0 == 1
        finally:
            tuned.close()
    finally:
        os.environ.pop("ANNEAL_BEAM_CACHE", None)
    assert np.array_equal(got, want)
