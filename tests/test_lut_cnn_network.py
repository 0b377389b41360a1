"""The LUT-CNN as a network, forward + backward, against the reference's own run of it.

Two 3x3 'same' conv blocks of per-pixel DifferentiableLut6 trees (27 -> 216 -> 36 -> 32, 288 -> 216 -> 36 -> 32, 2x2 max pooling,
288 -> 384 -> 64, 576 -> 384 -> 64, 2x2 max pooling) and a dense head 4096 -> 1024 -> 420 -> 70 -> 10; 3x32x32 images, batch 32, fp32,
batch norm on, non-binary.  The golden y / dx / dW of all 14 layers were produced by bb::Sequential / Convolution2d / MaxPooling /
DifferentiableLutN<6> of the unmodified reference (tests/golden/make_golden_cnn.py); inputs, wiring and tables are rebuilt from
integer hashing.  The device side is the C++ host classes of binarybrain_b200.core over the bbcu_* operators.

Tolerances.  Fourteen batch-normalised layers are chained.  Each multiplies last-ulp differences of its LUT values by gamma * rstd
(about 3-9 for the "spread" tables, 95 for the "fresh" N(0.5, 0.01)-like ones, whose node variances all sit at the 1e-5 floor), and a
frame whose hard-tanh decision flips moves every gradient of its node by a relative 1 / frames.  At network level this is what
separates ANY two implementations: the oracle's C restatement, which agrees with the reference operator by operator to 1e-6,
ends 3e-4 (y), 2e-3 (dx) and up to 8e-3 (dW) away from the reference's own classes on the small "spread" network, and 5-12 % away
in the gradients of the "fresh" one (measured here, CPU against CPU).  Gradients are therefore compared in the relative L2 norm
(a handful of flipped frames does not dominate it), with bars a few times those figures -- far below what a wrong index map,
mask or batch-norm term produces (errors of the size of the values themselves).  The tight, operator-level bars live in
test_gpu_parity.py and test_conv_lowering.py; this test is about the composition.
"""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))

CNN_GOLDEN = os.path.join(ROOT, "tests", "golden", "lut_cnn_golden.npz")
B, HW = 32, 32
# name: (y max abs, dx relative L2, dW relative L2 per layer)
TOLERANCE = {"spread": (2e-3, 1e-2, 3e-2), "fresh": (5e-4, 0.2, 0.3)}


def rel_l2(a, b):
    return float(np.linalg.norm((a - b).astype(np.float64)) / max(1e-30, np.linalg.norm(b.astype(np.float64))))


def build_network(core, idx, W):
    luts = []

    def lut(n):
        layer = core.DifferentiableLut6_fp32_fp32.create([n])
        layer.send_command("binary false")
        luts.append(layer)
        return layer

    def conv(widths):
        seq = core.Sequential.create()
        for n in widths:
            seq.add(lut(n))
        return core.Convolution2d_fp32_fp32.create(seq, 3, 3, padding="same")

    net = core.Sequential.create()
    net.add(conv([216, 36, 32]))
    net.add(conv([216, 36, 32]))
    net.add(core.MaxPooling_fp32_fp32.create(2, 2))
    net.add(conv([384, 64]))
    net.add(conv([384, 64]))
    net.add(core.MaxPooling_fp32_fp32.create(2, 2))
    for n in (1024, 420, 70, 10):
        net.add(lut(n))
    net.set_input_shape([3, HW, HW])
    for layer, i, w in zip(luts, idx, W):
        layer.set_connection(i)
        layer.W().set_numpy(w)
    return net, luts


def test_cnn_golden_inputs_are_reproducible():
    """The hashed inputs the golden file was made from: shapes and a few fixed values (no GPU, no reference needed)."""
    from make_golden_cnn import cnn_inputs
    x, dy, idx, W = cnn_inputs(False)
    assert x.shape == (3 * HW * HW, B) and dy.shape == (10, B) and len(idx) == 14 and len(W) == 14
    assert [i.shape[0] for i in idx] == [216, 36, 32, 216, 36, 32, 384, 64, 384, 64, 1024, 420, 70, 10]
    assert all(len(set(r)) == 6 for i in idx for r in i.tolist())
    assert abs(float(W[0].std()) - 0.01) < 1e-3 and abs(float(cnn_inputs(True)[3][0].std()) - 0.25) < 2e-2
    z = np.load(CNN_GOLDEN)
    assert z["cnn_fresh_y"].shape == (10, B) and z["cnn_spread_dx"].shape == (3 * HW * HW, B) and z["cnn_spread_dW10"].shape == (1024, 64)
    assert z["cnns_fresh_y"].shape == (10, 8) and z["cnns_spread_dWp10"].shape == (1024,)


def oracle_network(x, dy, idx, W, B=B, HW=HW):
    """The same network composed from the CPU oracle's operators; returns y, dx and the 14 table gradients."""
    from oracle import port
    tape, k = [], [0]

    def lut(h):
        l = k[0]
        k[0] += 1
        p = port.dl6_forward_train(h, idx[l], W[l], np.zeros(idx[l].shape[0]), np.ones(idx[l].shape[0]), binary=False)
        tape.append(("lut", l, h, p["mean"], p["rstd"]))
        return p["y"]

    def conv(h, c, hw, n_layers):
        cols = port.im2col_forward(h, c, hw, hw, 3, 3, padding="same")
        tape.append(("im2col", c, hw))
        for _ in range(n_layers):
            cols = lut(cols)
        tape.append(("col2im", cols.shape[0], hw))
        return port.col2im_forward(cols, cols.shape[0], hw, hw, B)

    def pool(h, c, hw):
        y, am = port.maxpool_forward(h, c, hw, hw, 2, 2)
        tape.append(("pool", c, hw, am))
        return y

    h = conv(x, 3, HW, 3)
    h = conv(h, 32, HW, 3)
    h = pool(h, 32, HW)
    h = conv(h, 32, HW // 2, 2)
    h = conv(h, 64, HW // 2, 2)
    h = pool(h, 64, HW // 2)
    for _ in range(4):
        h = lut(h)
    y, g, dW = h, dy, [None] * 14
    for op in reversed(tape):
        if op[0] == "lut":
            _, l, xin, mean, rstd = op
            g, dW[l] = port.dl6_backward(xin, g, idx[l], W[l], mean, rstd, xin.shape[0], binary=False)
        elif op[0] == "im2col":
            g = port.im2col_backward(g, op[1], op[2], op[2], 3, 3, padding="same")
        elif op[0] == "col2im":
            g = port.col2im_backward(g, op[1], op[2], op[2])
        else:
            g = port.maxpool_backward(op[3], g, op[1], op[2], op[2], 2, 2)
    return y, g, dW


@pytest.mark.parametrize("tables", ["spread", "fresh"])
def test_oracle_port_network_against_the_reference(tables):
    """Pins the C restatement at network level on the small case (3x16x16 images, batch 8): its operators, chained, against the
    reference's own classes, with the bars of the GPU test."""
    from make_golden_cnn import cnn_inputs, projection_vector, SMALL_B, SMALL_HW
    z = np.load(CNN_GOLDEN)
    x, dy, idx, W = cnn_inputs(tables == "spread", hw=SMALL_HW, batch=SMALL_B)
    y, dx, dW = oracle_network(x, dy, idx, W, B=SMALL_B, HW=SMALL_HW)
    tol_y, tol_dx, tol_dW = TOLERANCE[tables]
    r64 = projection_vector()
    e_dW = [rel_l2(dW[k] @ r64, z[f"cnns_{tables}_dWp{k}"]) for k in range(14)]
    print(f"oracle port lut-cnn {tables}: y {np.abs(y - z[f'cnns_{tables}_y']).max():.2e} dx {rel_l2(dx, z[f'cnns_{tables}_dx']):.2e} dW {max(e_dW):.2e}")
    assert np.abs(y - z[f"cnns_{tables}_y"]).max() <= tol_y
    assert rel_l2(dx, z[f"cnns_{tables}_dx"]) <= tol_dx
    assert max(e_dW) <= tol_dW, e_dW


@pytest.mark.gpu
@pytest.mark.parametrize("tables", ["spread", "fresh"])
def test_lut_cnn_forward_backward_against_the_reference(tables):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from binarybrain_b200 import build
    build.build_all()
    import binarybrain_b200.core as core
    from make_golden_cnn import cnn_inputs
    z = np.load(CNN_GOLDEN)
    x, dy, idx, W = cnn_inputs(tables == "spread")
    net, luts = build_network(core, idx, W)
    y = net.forward(core.FrameBuffer.from_numpy_fp32(np.ascontiguousarray(x.T).reshape(B, 3, HW, HW)), True).numpy_fp32().reshape(B, -1).T
    dx = net.backward(core.FrameBuffer.from_numpy_fp32(np.ascontiguousarray(dy.T))).numpy_fp32().reshape(B, -1).T
    tol_y, tol_dx, tol_dW = TOLERANCE[tables]
    want_y, want_dx = z[f"cnn_{tables}_y"], z[f"cnn_{tables}_dx"]
    e_y = float(np.abs(y - want_y).max())
    e_dx = rel_l2(dx, want_dx)
    e_dW = [rel_l2(l.dW().numpy(), z[f"cnn_{tables}_dW{k}"]) for k, l in enumerate(luts)]
    print(f"lut-cnn {tables}: y {e_y:.2e}  dx {e_dx:.2e}  dW {max(e_dW):.2e} (layer {int(np.argmax(e_dW))})")
    assert y.shape == want_y.shape and e_y <= tol_y
    assert e_dx <= tol_dx
    assert max(e_dW) <= tol_dW, e_dW
