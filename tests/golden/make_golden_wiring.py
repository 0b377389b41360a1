"""Regenerates tests/golden/wiring_golden.npz: the connection tables a fresh layer of the UNMODIFIED reference draws under each of
its wiring rules (include/bb/ConnectionTable.h:150-284), for fixed node shapes and seeds.

    make -C oracle && python tests/golden/make_golden_wiring.py
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from oracle import ref  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "wiring_golden.npz")
# (rule, input node shape, output node shape, layer seed)
CASES = [("pointwise", [12, 5, 4], [9, 5, 4], 7), ("pointwise", [32, 16, 16], [64, 16, 16], 1), ("depthwise", [7, 6, 5], [7, 3, 4], 7),
         ("depthwise", [32, 16, 16], [32, 16, 16], 1), ("gauss", [3, 16, 16], [2, 8, 8], 7), ("gauss", [64], [32], 3), ("serial", [10], [7], 1),
         ("random", [3, 8, 8], [4, 4, 4], 7), ("", [784], [1024], 1)]


def key(rule, ins, outs, seed):
    return f"wiring_{rule or 'default'}_{'x'.join(map(str, ins))}_{'x'.join(map(str, outs))}_s{seed}"


def main():
    assert ref.available(), "build oracle/_ref first (make -C oracle)"
    g = {key(*c): ref.init_connection(c[1], c[2], seed=c[3], connection=c[0]) for c in CASES}
    np.savez_compressed(OUT, **g)
    print("wrote", OUT, os.path.getsize(OUT))


if __name__ == "__main__":
    main()
