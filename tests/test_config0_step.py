"""One whole training step of the small MLP (784 -> 1024 -> 420 -> 70 nodes, 512 frames) against the reference's own run of it.

784 -> 1024 -> 420 -> 70 DifferentiableLut6 (fp32, batch norm on, non-binary), bb::Reduce to 10 classes, softmax cross-entropy,
Adam; 512 frames.  The golden values come from bb::Sequential + LossSoftmaxCrossEntropy + OptimizerAdam of the unmodified
reference (tests/golden/make_golden.py); inputs are rebuilt from integer hashing.  Checked on the CPU with the oracle port
(pins the oracle's Reduce / loss / layer chaining) and on the GPU through the bbcu_* operators.
Tolerances: logits 1e-4 (three batch-normalised layers chained, each amplifying last-ulp differences by gamma*rstd);
loss 1e-5 relative; W after the Adam step 1e-4 absolute in sum-normalised form (|sum W - golden| / count).
"""
import numpy as np
import pytest

from oracle import port, det_uniform, det_wiring

WIDTHS, CLASSES, F = [784, 1024, 420, 70], 10, 512


def inputs():
    x = det_uniform((WIDTHS[0], F), 101)
    labels = (det_uniform((F,), 102) * CLASSES).astype(np.int64)
    t = np.zeros((CLASSES, F), np.float32)
    t[labels, np.arange(F)] = 1.0
    idx = [det_wiring(WIDTHS[l], WIDTHS[l + 1], 110 + l) for l in range(3)]
    W = [np.clip(0.5 + 0.25 * (det_uniform((WIDTHS[l + 1], 64), 120 + l) - 0.5) * 3.46, 0, 1).astype(np.float32) for l in range(3)]
    return x, t, idx, W


def check(golden, y, loss, dx, W_new, W_old):
    assert np.abs(y - golden["cfg0_y"]).max() <= 1e-4
    assert abs(loss - float(golden["cfg0_loss"][0])) <= 1e-5 * abs(float(golden["cfg0_loss"][0]))
    scale = float(golden["cfg0_dx_abs_sum"][0]) / dx.size
    assert np.abs(dx[:4] - golden["cfg0_dx_rows"]).max() <= 0.05 * scale + 1e-9       # rows of d(loss)/dx: mean magnitude `scale`
    assert abs(np.abs(dx).sum(dtype=np.float64) - float(golden["cfg0_dx_abs_sum"][0])) <= 1e-3 * float(golden["cfg0_dx_abs_sum"][0])
    for l in range(3):
        assert np.abs(W_new[l][:4] - golden[f"cfg0_W{l}_rows"]).max() <= 1e-4
        assert abs(W_new[l].sum(dtype=np.float64) - float(golden[f"cfg0_W{l}_sum"][0])) / W_new[l].size <= 1e-5
        step = np.abs(W_new[l] - W_old[l]).sum(dtype=np.float64)
        assert abs(step - float(golden[f"cfg0_dWstep{l}_abs_sum"][0])) <= 2e-3 * float(golden[f"cfg0_dWstep{l}_abs_sum"][0])


def test_config0_step_oracle_port(golden):
    x, t, idx, W = inputs()
    acts, stats = [x], []
    for l in range(3):
        p = port.dl6_forward_train(acts[-1], idx[l], W[l], np.zeros(WIDTHS[l + 1]), np.ones(WIDTHS[l + 1]), binary=False)
        acts.append(p["y"])
        stats.append(p)
    y = port.reduce_forward(acts[-1], CLASSES)
    dy, loss = port.softmax_cross_entropy(y, t)
    g = port.reduce_backward(dy, WIDTHS[-1])
    W_new = []
    for l in (2, 1, 0):
        g, dW = port.dl6_backward(acts[l], g, idx[l], W[l], stats[l]["mean"], stats[l]["rstd"], WIDTHS[l], binary=False)
        Wl = W[l].copy()
        port.adam_update(Wl, dW, np.zeros_like(Wl), np.zeros_like(Wl), np.ones(2, np.float32))
        W_new.insert(0, Wl)
    check(golden, y, loss, g, W_new, W)


def test_losses_and_reduce_oracle_properties(golden):
    y, t = golden["loss_y"], golden["loss_t"]
    dy, loss = port.softmax_cross_entropy(y, t)
    sm = np.exp(y - y.max(0)) / np.exp(y - y.max(0)).sum(0)
    assert np.abs(dy - (sm - t) / t.sum()).max() <= 1e-6 and abs(loss + np.log(sm[t > 0] + 1e-7).mean()) <= 1e-5
    dy, loss = port.mean_squared_error(y, t)
    assert np.abs(dy - 2 * (y - t) / y.size).max() <= 1e-7 and abs(loss - ((y - t) ** 2).mean(0).sum() / y.shape[1] * 1.0) <= 1e-5
    r = port.reduce_forward(np.arange(70 * 3, dtype=np.float32).reshape(70, 3), 10)
    assert np.allclose(r[2], np.arange(70 * 3).reshape(7, 10, 3)[:, 2].mean(0))
    assert np.allclose(port.reduce_backward(r, 70)[12], r[2] / 7)


@pytest.mark.gpu
def test_config0_step_gpu(golden):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from binarybrain_b200 import ops
    from gpu_util import dev
    x, t, idx, W = inputs()
    xd, td = dev(x), dev(t)
    idx_d = [dev(i) for i in idx]
    W_d = [dev(w.copy()) for w in W]
    dW_d = [torch.zeros_like(w) for w in W_d]
    opt = ops.Adam(W_d, dW_d)
    acts, stats = [xd], []
    for l in range(3):
        n = WIDTHS[l + 1]
        y, mean, rstd = ops.differentiable_lut6_forward_training(acts[-1], idx_d[l], W_d[l], torch.zeros(n, device="cuda"),
                                                                 torch.ones(n, device="cuda"), F, binary=False)
        acts.append(y)
        stats.append((mean, rstd))
    logits = ops.reduce_forward(acts[-1], CLASSES, F)
    dy, loss = ops.softmax_cross_entropy(logits, td, F)
    g = ops.reduce_backward(dy, WIDTHS[-1], F)
    for l in (2, 1, 0):
        g = ops.differentiable_lut6_backward(acts[l], g, idx_d[l], W_d[l], dW_d[l], stats[l][0], stats[l][1], WIDTHS[l], F, binary=False)
    opt.update()
    check(golden, logits.cpu().numpy(), float(loss.item()), g.cpu().numpy(), [w.cpu().numpy() for w in W_d], W)
    # MSE and Reduce operators against the oracle
    yl, tl = golden["loss_y"], golden["loss_t"]
    dy_m, buf = ops.mean_squared_error(dev(yl), dev(tl), yl.shape[1])
    want_dy, want_loss = port.mean_squared_error(yl, tl)
    assert np.abs(dy_m.cpu().numpy() - want_dy).max() <= 1e-7 and abs(float(buf.sum().item()) / yl.shape[1] - want_loss) <= 1e-6
    dy_c, loss_c = ops.softmax_cross_entropy(dev(yl), dev(tl), yl.shape[1])
    want_dy, want_loss = port.softmax_cross_entropy(yl, tl)
    assert np.abs(dy_c.cpu().numpy() - want_dy).max() <= 1e-6 and abs(float(loss_c.item()) - want_loss) <= 1e-5
