"""Regenerates tests/golden/lut_cnn_golden.npz: the LUT-CNN (two 3x3 conv blocks of per-pixel DifferentiableLut6 trees with 2x2
max pooling and a dense head, 14 LUT layers) run forward + backward by the UNMODIFIED reference classes (bb::Sequential,
bb::Convolution2d, bb::MaxPooling, bb::DifferentiableLutN<6> behind oracle/ref_driver.cpp).

    make -C oracle && python tests/golden/make_golden_cnn.py          # several minutes: the reference's LUT backward is a serial loop

Batch 32, 3x32x32 images.  Inputs, wiring and tables are rebuilt from integer hashing (oracle.det_uniform / det_wiring) by the tests,
so only the reference's outputs are stored: y, dx and the table gradients of every layer, for two table initialisations --
"fresh" N(0.5, 0.01)-like tables (the variance of every node at its floor, gamma * rstd = 95) and "spread" tables (uniform, std 0.25).
A second, small case (batch 8, 3x16x16 images; keys cnns_*) serves the CPU test of the oracle's C restatement: y, dx, and per layer
the projection of the table gradients on a fixed hashed vector (dW @ r, r = det_uniform(64, 399) - 0.5).

    python tests/golden/make_golden_cnn.py --small-only      # regenerates the small case only, keeping the stored full-size arrays
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from oracle import ref, det_uniform, det_wiring  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lut_cnn_golden.npz")
B, HW = 32, 32


def cnn_inputs(spread, hw=HW, batch=B):
    """x [3*hw*hw, batch], dy [10, batch], wiring and tables of the 14 layers; `spread`: table std 0.25 instead of 0.01."""
    x = det_uniform((3 * hw * hw, batch), 301)
    dy = det_uniform((10, batch), 302) - 0.5
    idx, W = [], []
    for l, (n_in, n_out) in enumerate(zip(ref.cnn_input_widths(hw), ref.CNN_WIDTHS)):
        idx.append(det_wiring(n_in, n_out, 310 + l))
        u = det_uniform((n_out, 64), 330 + l) - 0.5                      # uniform, std 1/sqrt(12)
        W.append(np.clip(0.5 + (0.25 if spread else 0.01) * 3.4641 * u, 0, 1).astype(np.float32))
    return x, dy, idx, W


SMALL_B, SMALL_HW = 8, 16


def projection_vector():
    return (det_uniform((64,), 399) - 0.5).astype(np.float32)


def main():
    assert ref.available(), "build oracle/_ref first (make -C oracle)"
    ref.use_all_cores()
    g = {}
    small_only = "--small-only" in sys.argv
    if small_only:
        g.update({k: v for k, v in np.load(OUT).items() if not k.startswith("cnns_")})
    r64 = projection_vector()
    for name, spread in (("fresh", False), ("spread", True)):
        x, dy, idx, W = cnn_inputs(spread, hw=SMALL_HW, batch=SMALL_B)
        r = ref.lut_cnn_step(x, dy, idx, W, hw=SMALL_HW)
        g[f"cnns_{name}_y"] = r["y"]
        g[f"cnns_{name}_dx"] = r["dx"]
        for l, dW in enumerate(r["dW"]):
            g[f"cnns_{name}_dWp{l}"] = dW @ r64
    for name, spread in (() if small_only else (("fresh", False), ("spread", True))):
        x, dy, idx, W = cnn_inputs(spread)
        r = ref.lut_cnn_step(x, dy, idx, W, hw=HW)
        g[f"cnn_{name}_y"] = r["y"]
        g[f"cnn_{name}_dx"] = r["dx"]
        for l, dW in enumerate(r["dW"]):
            g[f"cnn_{name}_dW{l}"] = dW
        print(name, "y", r["y"][:, :2].ravel(), "|dx|", np.abs(r["dx"]).mean(), "|dW|", [float(np.abs(d).mean()) for d in r["dW"]][:4])
    np.savez_compressed(OUT, **g)
    print("wrote", OUT, os.path.getsize(OUT))


if __name__ == "__main__":
    main()
