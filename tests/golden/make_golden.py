"""Regenerates tests/golden/lut6_golden.npz from the UNMODIFIED reference CPU path.

Run where a reference checkout exists (oracle/Makefile builds oracle/_ref/libbbref.so from the
reference headers with the reference's own flags: g++ -O2 -mavx2 -mfma -fopenmp -std=c++14):

    make -C oracle && python tests/golden/make_golden.py

Shapes follow the reference's own unit tests: StochasticLutNTest.cpp:235-246 and :437-449,
SparseLutNTest.cpp:308-370, BinaryLutTest.cpp:187-190.  Inputs come from numpy's PCG64 with the
seeds below; wiring and tables are drawn here and handed to the reference object, the way the
reference's tests copy them between their CPU and GPU objects (StochasticLutNTest.cpp:36-53).
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from oracle import ref, port, pack_bits, det_uniform, det_wiring  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lut6_golden.npz")


def wiring(rng, n_in, n_out):
    return np.stack([rng.permutation(n_in)[:6] for _ in range(n_out)]).astype(np.int32)


def main():
    assert ref.available(), "build oracle/_ref first (make -C oracle)"
    g = {}
    rng = np.random.default_rng(20240601)

    # StochasticLutN<6,float> CPU (generic branch, host_simd=false) and the AVX2 branch where F % 8 == 0
    for (I, O, F) in [(6, 1, 1), (14, 16, 8), (14, 64, 3), (13, 17, 193)]:
        for binary in (0, 1):
            for lb in (0, 1):
                k = f"sl6_{I}_{O}_{F}_b{binary}_l{lb}"
                idx = wiring(rng, I, O)
                W = np.clip(rng.normal(0.5, 0.25, (O, 64)), 0, 1).astype(np.float32)
                x = rng.random((I, F), dtype=np.float32)
                dy = rng.random((O, F), dtype=np.float32)
                dW0 = rng.random((O, 64), dtype=np.float32)
                r = ref.stochastic_lut6(x, idx, W, binary=binary, lut_binarize=lb, host_simd=False, dy=dy, dW=dW0)
                g.update({k + "_idx": idx, k + "_W": W, k + "_x": x, k + "_dy": dy, k + "_dW0": dW0,
                          k + "_y": r["y"], k + "_dx": r["dx"], k + "_dW": r["dW"]})
                if F % 8 == 0:
                    r = ref.stochastic_lut6(x, idx, W, binary=binary, lut_binarize=lb, host_simd=True, dy=dy, dW=dW0)
                    g.update({k + "_y_simd": r["y"], k + "_dx_simd": r["dx"], k + "_dW_simd": r["dW"]})

    # StochasticLutN<6,Bit>
    for (I, O, F) in [(14, 16, 8), (13, 17, 161)]:
        for lb in (0, 1):
            k = f"sl6bit_{I}_{O}_{F}_l{lb}"
            idx = wiring(rng, I, O)
            W = np.clip(rng.normal(0.5, 0.25, (O, 64)), 0, 1).astype(np.float32)
            xb = pack_bits(rng.random((I, F)) > 0.5)
            dy = rng.random((O, F), dtype=np.float32)
            r = ref.stochastic_lut6(xb, idx, W, frames=F, lut_binarize=lb, dy=dy)
            g.update({k + "_idx": idx, k + "_W": W, k + "_x": xb, k + "_dy": dy, k + "_y": r["y"], k + "_dx": r["dx"], k + "_dW": r["dW"]})

    # DifferentiableLutN<6,float> with batch norm (generic CPU branch), train + inference
    for (I, O, F) in [(6, 1, 1), (12, 2, 39), (24, 16, 64), (16, 16, 131)]:
        for binary in (0, 1):
            for lb in (0, 1):
                k = f"dl6_{I}_{O}_{F}_b{binary}_l{lb}"
                idx = wiring(rng, I, O)
                W = np.clip(rng.normal(0.5, 0.25, (O, 64)), 0, 1).astype(np.float32)
                x = rng.random((I, F), dtype=np.float32)
                dy = rng.random((O, F), dtype=np.float32)
                rm0 = rng.random(O, dtype=np.float32)
                rv0 = rng.random(O, dtype=np.float32) + 0.5
                r = ref.differentiable_lut6(x, idx, W, binary=binary, lut_binarize=lb, running_mean=rm0, running_var=rv0, dy=dy)
                ri = ref.differentiable_lut6(x, idx, W, binary=binary, lut_binarize=lb, running_mean=rm0, running_var=rv0, train=False)
                g.update({k + "_idx": idx, k + "_W": W, k + "_x": x, k + "_dy": dy, k + "_rm0": rm0, k + "_rv0": rv0,
                          k + "_y": r["y"], k + "_mean": r["mean"], k + "_rstd": r["rstd"], k + "_rm": r["running_mean"],
                          k + "_rv": r["running_var"], k + "_dx": r["dx"], k + "_dW": r["dW"], k + "_y_infer": ri["y"]})

    # DifferentiableLutN<6,Bit>
    for (I, O, F) in [(12, 2, 39), (24, 16, 64), (16, 16, 131)]:
        for lb in (0, 1):
            k = f"dl6bit_{I}_{O}_{F}_l{lb}"
            idx = wiring(rng, I, O)
            W = np.clip(rng.normal(0.5, 0.25, (O, 64)), 0, 1).astype(np.float32)
            xb = pack_bits(rng.random((I, F)) > 0.5)
            dy = rng.random((O, F), dtype=np.float32)
            r = ref.differentiable_lut6(xb, idx, W, frames=F, lut_binarize=lb, dy=dy)
            ri = ref.differentiable_lut6(xb, idx, W, frames=F, lut_binarize=lb, running_mean=r["running_mean"],
                                         running_var=r["running_var"], train=False)
            g.update({k + "_idx": idx, k + "_W": W, k + "_x": xb, k + "_dy": dy, k + "_y": r["y"], k + "_mean": r["mean"],
                      k + "_rstd": r["rstd"], k + "_rm": r["running_mean"], k + "_rv": r["running_var"], k + "_dx": r["dx"],
                      k + "_dW": r["dW"], k + "_y_infer": ri["y"]})

    # DifferentiableLutN without batch norm, fp32 and Bit
    for binary in (0, 1):
        k = f"dl6nobn_14_16_40_b{binary}"
        idx = wiring(rng, 14, 16)
        W = np.clip(rng.normal(0.5, 0.25, (16, 64)), 0, 1).astype(np.float32)
        x = rng.random((14, 40), dtype=np.float32)
        dy = rng.random((16, 40), dtype=np.float32)
        r = ref.differentiable_lut6(x, idx, W, batch_norm=False, binary=binary, dy=dy)
        g.update({k + "_idx": idx, k + "_W": W, k + "_x": x, k + "_dy": dy, k + "_y": r["y"], k + "_dx": r["dx"], k + "_dW": r["dW"]})
    k = "dl6nobnbit_14_16_70"
    idx = wiring(rng, 14, 16)
    W = np.clip(rng.normal(0.5, 0.25, (16, 64)), 0, 1).astype(np.float32)
    xb = pack_bits(rng.random((14, 70)) > 0.5)
    dy = rng.random((16, 70), dtype=np.float32)
    r = ref.differentiable_lut6(xb, idx, W, frames=70, batch_norm=False, dy=dy)
    g.update({k + "_idx": idx, k + "_W": W, k + "_x": xb, k + "_dy": dy, k + "_y": r["y"], k + "_dx": r["dx"], k + "_dW": r["dW"]})

    # BinaryLutN<6,Bit>: AVX2 and generic branches
    for (I, O, F) in [(16, 16, 32), (40, 33, 300)]:
        k = f"bl6_{I}_{O}_{F}"
        idx = wiring(rng, I, O)
        table = rng.integers(-2**31, 2**31, (O, 2)).astype(np.int32)
        xb = pack_bits(rng.random((I, F)) > 0.5)
        r0 = ref.binary_lut6(xb, idx, table, F, host_simd=False)
        r1 = ref.binary_lut6(xb, idx, table, F, host_simd=True)
        assert (r0["y"] == r1["y"]).all()
        g.update({k + "_idx": idx, k + "_table": table, k + "_x": xb, k + "_y": r0["y"]})

    # StochasticBatchNormalization<float>
    for (O, F) in [(3, 1), (16, 39), (8, 200)]:
        k = f"sbn_{O}_{F}"
        x = rng.random((O, F), dtype=np.float32)
        dy = rng.random((O, F), dtype=np.float32)
        rm0 = rng.random(O, dtype=np.float32)
        rv0 = rng.random(O, dtype=np.float32) + 0.5
        r = ref.stochastic_bn(x, mode=0, running_mean=rm0, running_var=rv0, dy=dy)
        r2 = ref.stochastic_bn(x, mode=2, running_mean=rm0, running_var=rv0)
        g.update({k + "_x": x, k + "_dy": dy, k + "_rm0": rm0, k + "_rv0": rv0, k + "_y": r["y"], k + "_mean": r["mean"],
                  k + "_rstd": r["rstd"], k + "_rm": r["running_mean"], k + "_rv": r["running_var"], k + "_dx": r["dx"],
                  k + "_y_re": r2["y"]})

    # A fresh layer's seeded wiring and table, as the reference draws them (layer seed 1)
    idx, W = ref.init_layer(32, 16, 1)
    g.update({"init_32_16_s1_idx": idx, "init_32_16_s1_W": W})
    idx, W = ref.init_layer(784, 1024, 1)
    g.update({"init_784_1024_s1_idx_head": idx[:8], "init_784_1024_s1_idx_sum": np.array([idx.astype(np.int64).sum()]),
              "init_784_1024_s1_W_head": W[:2]})

    # 100 Adam steps on a small DifferentiableLut6 layer (fixed x, dy).
    # "adam": batch norm on, tables N(0.5, 0.25): well conditioned.  "adamnobn": batch norm off, tables
    # N(0.5, 0.01) as a fresh layer has them.  (Batch norm on WITH N(0.5, 0.01) tables is not a usable
    # fixture: the per-node variance sits at the 1e-5 clamp, and two builds of the reference that differ
    # only in FMA contraction already end 1.5e-3 apart after 100 steps.)
    I, O, F = 24, 16, 64
    idx = wiring(rng, I, O)
    x = rng.random((I, F), dtype=np.float32)
    dy = (rng.random((O, F), dtype=np.float32) - 0.5) * 0.1
    W = np.clip(rng.normal(0.5, 0.25, (O, 64)), 0, 1).astype(np.float32)
    r = ref.differentiable_lut6_adam(x, idx, W, dy, 100, binary=False)
    g.update({"adam_idx": idx, "adam_W0": W, "adam_x": x, "adam_dy": dy, "adam_W100": r["W"], "adam_y100": r["y"],
              "adam_rm100": r["running_mean"], "adam_rv100": r["running_var"]})
    W = np.clip(rng.normal(0.5, 0.01, (O, 64)), 0, 1).astype(np.float32)
    r = ref.differentiable_lut6_adam(x, idx, W, dy, 100, batch_norm=False, binary=False)
    g.update({"adamnobn_W0": W, "adamnobn_W100": r["W"], "adamnobn_y100": r["y"]})

    # One whole training step of the small MLP: 784 -> 1024 -> 420 -> 70 DifferentiableLut6 (fp32, batch norm, non-binary),
    # Reduce to 10 classes, softmax cross-entropy, Adam, 512 frames.  Inputs come from integer hashing (oracle.det_uniform), so only
    # the results are stored: logits, loss, dx and W checksums plus a few rows.
    widths, classes, F = [784, 1024, 420, 70], 10, 512
    x = det_uniform((widths[0], F), 101)
    labels = (det_uniform((F,), 102) * classes).astype(np.int64)
    t = np.zeros((classes, F), np.float32)
    t[labels, np.arange(F)] = 1.0
    idx_l = [det_wiring(widths[l], widths[l + 1], 110 + l) for l in range(3)]
    W_l = [np.clip(0.5 + 0.25 * (det_uniform((widths[l + 1], 64), 120 + l) - 0.5) * 3.46, 0, 1).astype(np.float32) for l in range(3)]
    r = ref.lut_mlp_step(x, t, widths, classes, idx_l, W_l)
    g.update({"cfg0_y": r["y"], "cfg0_loss": np.array([r["loss"]]), "cfg0_dx_rows": r["dx"][:4], "cfg0_dx_abs_sum": np.array([np.abs(r["dx"]).sum(dtype=np.float64)])})
    for l in range(3):
        g.update({f"cfg0_W{l}_rows": r["W"][l][:4], f"cfg0_W{l}_sum": np.array([r["W"][l].sum(dtype=np.float64)]),
                  f"cfg0_dWstep{l}_abs_sum": np.array([np.abs(r["W"][l] - W_l[l]).sum(dtype=np.float64)])})
    # the losses and Reduce on their own
    yl = det_uniform((10, 40), 130) * 4 - 2
    tl = np.zeros((10, 40), np.float32)
    tl[(det_uniform((40,), 131) * 10).astype(np.int64), np.arange(40)] = 1.0
    import ctypes as C  # noqa: E402
    g.update({"loss_y": yl, "loss_t": tl})

    # Binary modulation (config 2 neighbours): RealToBinary with frame modulation 7 (deterministic and with seeded thresholds from
    # the reference's UniformDistributionGenerator), BinaryToReal integration back to 10 outputs with its backward.
    xm = det_uniform((12, 9), 140)
    for ps in (1, 4):
        yb, _ = ref.real_to_binary(xm, frame_mod=7, depth_mod=2, seed=0, point_size=ps)
        ys, th = ref.real_to_binary(xm, frame_mod=7, depth_mod=2, seed=7, point_size=ps)
        g.update({f"r2b_p{ps}_det": yb, f"r2b_p{ps}_seeded": ys, f"r2b_p{ps}_th": th})
    g["r2b_x"] = xm
    xb, _ = ref.real_to_binary(det_uniform((60, 8), 141), frame_mod=7, seed=3)
    dyb = det_uniform((10, 8), 142)
    yb2r, dxb2r = ref.binary_to_real(xb, 10, 8, 7, dy=dyb)
    g.update({"b2r_x": xb, "b2r_dy": dyb, "b2r_y": yb2r, "b2r_dx": dxb2r})

    # Convolution lowering (config 3 neighbours): ConvolutionIm2Col / ConvolutionCol2Im / MaxPooling of the reference, fp32 and bit
    # frames, forward and backward.  Inputs are det_uniform(seed) and are regenerated by the tests; the case tables are stored.
    PADS, BORDERS = ["valid", "same"], ["constant", "reflect", "reflect_101", "replicate", "wrap"]
    im2col_cases = [  # c, h, w, fh, fw, y_stride, x_stride, padding, border, frames
        (3, 8, 8, 3, 3, 1, 1, 1, 2, 5), (2, 7, 9, 3, 3, 1, 1, 0, 0, 4), (2, 8, 8, 3, 3, 2, 2, 1, 3, 3), (1, 6, 5, 5, 3, 1, 2, 1, 4, 2),
        (2, 6, 6, 3, 3, 1, 1, 1, 1, 3), (2, 9, 7, 2, 2, 2, 1, 0, 2, 3), (2, 8, 8, 3, 3, 1, 1, 1, 0, 40), (3, 8, 4, 3, 3, 1, 1, 1, 2, 37)]
    for k, (c, h, w, fh, fw, ys, xs, pad, bm, F) in enumerate(im2col_cases):
        x = det_uniform((c * h * w, F), 300 + k)
        oh, ow, _, _ = port.im2col_geometry(h, w, fh, fw, ys, xs, PADS[pad])
        dy = det_uniform((c * fh * fw, F * oh * ow), 320 + k)
        y, dx = ref.im2col(x, c, h, w, fh, fw, ys, xs, PADS[pad], BORDERS[bm], dy=dy)
        yb, _ = ref.im2col(pack_bits(x > 0.5), c, h, w, fh, fw, ys, xs, PADS[pad], BORDERS[bm], frames=F)
        g.update({f"im2col{k}_y": y, f"im2col{k}_dx": dx, f"im2col{k}_ybits": yb})
    g["im2col_cases"] = np.array(im2col_cases, np.int32)
    col2im_cases = [(3, 4, 5, 7), (2, 8, 8, 33), (5, 1, 1, 9), (2, 4, 8, 70)]      # c, h, w, output frames
    for k, (c, h, w, Fo) in enumerate(col2im_cases):
        x = det_uniform((c, Fo * h * w), 340 + k)
        dy = det_uniform((c * h * w, Fo), 350 + k)
        y, dx = ref.col2im(x, c, h, w, Fo, dy=dy)
        yb, _ = ref.col2im(pack_bits(x > 0.5), c, h, w, Fo)
        g.update({f"col2im{k}_y": y, f"col2im{k}_dx": dx, f"col2im{k}_ybits": yb})
    g["col2im_cases"] = np.array(col2im_cases, np.int32)
    pool_cases = [(3, 8, 8, 2, 2, 9), (2, 7, 5, 2, 2, 33), (2, 9, 9, 3, 3, 5), (1, 4, 6, 2, 3, 70)]   # c, h, w, fh, fw, frames
    for k, (c, h, w, fh, fw, F) in enumerate(pool_cases):
        x = np.floor(det_uniform((c * h * w, F), 360 + k) * 4).astype(np.float32) / 4          # few distinct values: ties on purpose
        oh, ow = (h + fh - 1) // fh, (w + fw - 1) // fw
        dy = det_uniform((c * oh * ow, F), 370 + k)
        y, dx = ref.maxpool(x, c, h, w, fh, fw, dy=dy)
        xb = pack_bits(det_uniform((c * h * w, F), 380 + k) > 0.7)
        yb, dxb = ref.maxpool(xb, c, h, w, fh, fw, dy=dy, frames=F)
        g.update({f"pool{k}_y": y, f"pool{k}_dx": dx, f"pool{k}_ybits": yb, f"pool{k}_dxbits": dxb})
    g["pool_cases"] = np.array(pool_cases, np.int32)

    # Serialised layers: DumpObject bytes written by the reference's own classes (wiring det_wiring(10, 3, 500), tables det_uniform 501).
    ser_idx, ser_W = det_wiring(10, 3, 500), det_uniform((3, 64), 501)
    g["ser_dl6_fp32"] = ref.layer_dump("dl6_fp32", 10, ser_idx, ser_W, running_mean=[0.1, 0.2, 0.3], running_var=[1.5, 2.5, 3.5], lut_binarize=True,
                                       binary=False, gamma=0.25, beta=0.4, momentum=0.8)
    g["ser_dl6_bit"] = ref.layer_dump("dl6_bit", 10, ser_idx, ser_W)
    g["ser_sl6_fp32"] = ref.layer_dump("sl6_fp32", 10, ser_idx, ser_W, binary=False, lut_binarize=True)
    g["ser_binary_lut6"] = ref.layer_dump("binary_lut6", 10, ser_idx, np.array([[1, 2], [3, 4], [5, -6]], np.int32))

    np.savez_compressed(OUT, **g)
    print("wrote", OUT, os.path.getsize(OUT), "bytes,", len(g), "arrays")


if __name__ == "__main__":
    main()
