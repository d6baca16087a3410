"""Feeds damaged kernel-IR blobs to the code generator's C entry points. Run as a child process by
test_abi.py: the contract is that every entry point returns a status, so a crash of this process is
the failure being looked for.

    python tests/kir_fuzz.py <seed> <mutations>
"""
import ctypes
import os
import random
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from anneal_b200 import device, kir, realize as R, workloads as W  # noqa: E402


def main(seed: int, mutations: int) -> None:
    R.MATERIALIZE_CONTRACTION_OPERANDS = True
    graphs = [W.MLP().graph().targets(), W.SoftmaxFwdBwd(16, 128).graph(True)[0],
              W.WideMLP(batch=32, width=64, classes=10, depth=1).graph().targets()]
    L = device.load_library()
    src = ctypes.create_string_buffer(1 << 16)
    n = ctypes.c_size_t()
    k, b, o = ctypes.c_int(), ctypes.c_int(), ctypes.c_int64()
    note = ctypes.create_string_buffer(256)
    rng = random.Random(seed)
    calls = rejected = 0
    for targets in graphs:
        items, _ = R.build_schedule(targets)
        blob = kir.serialize(items)

        def lower(bl, idx):
            nonlocal calls, rejected
            calls += 1
            rc = L.anl_lower(None, bl, len(bl), idx, None, src, 1 << 16, ctypes.byref(n), ctypes.byref(k),
                             ctypes.byref(b), ctypes.byref(o), note, 256)
            rejected += rc != 0
            L.anl_lower_chain(bl, len(bl), 0, min(len(items), 5), src, 1 << 16, ctypes.byref(n), note, 256)

        assert L.anl_lower(None, blob, len(blob), 0, None, src, 1 << 16, ctypes.byref(n), ctypes.byref(k),
                           ctypes.byref(b), ctypes.byref(o), note, 256) == 0
        for cut in range(0, len(blob), 97):                      # truncations
            lower(blob[:cut], 0)
        for _ in range(mutations):                               # a few damaged bytes each
            bl = bytearray(blob)
            for _ in range(rng.randint(1, 4)):
                bl[rng.randrange(len(bl))] = rng.randrange(256)
            lower(bytes(bl), rng.randrange(len(items)))
    print(f"calls={calls} rejected={rejected}")


if __name__ == "__main__":
    main(int(sys.argv[1]) if len(sys.argv) > 1 else 0, int(sys.argv[2]) if len(sys.argv) > 2 else 300)
