"""GPU parity: every bbcu_* operator, called through the C ABI, against the CPU oracle.

Tolerances (north-star): BinaryLut6 and gather indexing bit-exact; fp32 y / dx / dW within 1e-5 of the
value range.  Two documented refinements where a decision threshold or the batch-norm condition number
makes a literal 1e-5 meaningless:
  * outputs that pass through a threshold (binarised y, the hard-tanh mask in dx) may differ from the
    oracle only where the oracle's pre-threshold value is within 1e-4 of the threshold;
  * batch-normalised fp32 outputs are compared with 1e-5 * max(1, gamma*rstd): the normalisation
    multiplies the last-ulp difference between a lerp tree and the CPU's product form by gamma*rstd
    (up to 95 when the variance sits at its 1e-5 floor).

Hard-tanh mask in the DifferentiableLut6 backward: a frame whose pre-activation lies within 1e-4 * gamma*rstd of 0 or 1 may
take the other side of the mask on the GPU, and through the batch sums (dmean, dvar) one flipped frame moves every gradient of
its node by a relative 1/frames.  The tests therefore never skip an assert; they make such frames harmless instead: where the
inputs are the test's own, dy is set to zero on those frames (a masked and an unmasked zero are the same), and where dy is fixed
by a golden file, the nodes that own such a frame (and the input rows they feed) are left out of that one comparison, the
same case being checked in full against the oracle with dy zeroed on those frames.
"""
import numpy as np
import pytest
import torch

from conftest import golden_cases
from oracle import port, pack_bits, unpack_bits

pytestmark = pytest.mark.gpu

TOL = 1e-5
# Batch-normalised values: the factor in front of gamma*rstd.  Both sides evaluate the LUT to about 2 ulp of a value near 0.5
# (6e-8 each, different operation order) and the mean to 1 ulp; (raw - mean) * rstd * gamma turns their sum, up to 3e-7, into
# 3e-7 * gamma*rstd.  The gradients pass through the same rstd once more (dxc = gamma * dy * rstd) and add the rounding of the
# fp32 atomics that accumulate dx and dW, hence 2 there.
BN_Y_FACTOR = 3.0
BN_GRAD_FACTOR = 2.0


def _edges(pre, amp):
    """Frames whose hard-tanh decision the last bits of the pre-activation could flip."""
    return (np.abs(pre) < 1e-4 * amp) | (np.abs(pre - 1) < 1e-4 * amp)


def _untouched(edge, idx, n_in):
    """(nodes without an edge frame, input rows fed by such nodes only)."""
    node_ok = ~edge.any(axis=1)
    row_ok = np.ones(n_in, bool)
    row_ok[np.unique(idx[~node_ok])] = False
    return node_ok, row_ok


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from binarybrain_b200 import ops as o
    return o


def _flags(case):
    d = {}
    for p in case.split("_"):
        if p[0] == "b" and p[1:].isdigit():
            d["binary"] = int(p[1:])
        if p[0] == "l" and p[1:].isdigit():
            d["lut_binarize"] = int(p[1:])
    return d


# --------------------------------------------------------------------------------------------- StochasticLut6
def _sl6_check(ops, x, idx, W, dy, dW0, fl, want, stride=None):
    from gpu_util import dev_fp32, dev, host_fp32, err
    I, F = x.shape
    O = idx.shape[0]
    xd = dev_fp32(x, stride)
    y = ops.stochastic_lut6_forward(xd, dev(idx), dev(W), F, **fl)
    assert err(host_fp32(y, F), want["y"]) <= TOL
    dWd = dev(dW0.copy())
    dx = ops.stochastic_lut6_backward(xd, dev_fp32(dy, stride), dev(idx), dev(W), dWd, I, F, **fl)
    assert err(host_fp32(dx, F), want["dx"]) <= TOL
    assert err(dWd.cpu().numpy(), want["dW"]) <= TOL


@pytest.mark.parametrize("case", golden_cases("sl6"))
def test_sl6_fp32_golden(ops, golden, case):
    g = lambda n: golden[case + "_" + n]
    _sl6_check(ops, g("x"), g("idx"), g("W"), g("dy"), g("dW0"), _flags(case), dict(y=g("y"), dx=g("dx"), dW=g("dW")))


@pytest.mark.parametrize("I,O,F,stride", [(13, 17, 1529, None), (14, 1024, 8, None), (14, 1024, 3, 16), (300, 700, 2100, 2112),
                                          (6, 1, 1, None), (2048, 4096, 640, None)])
@pytest.mark.parametrize("binary,lut_binarize", [(0, 0), (1, 1)])
def test_sl6_fp32_oracle(ops, I, O, F, stride, binary, lut_binarize):
    from gpu_util import wiring
    rng = np.random.default_rng(I * 7 + O + F)
    idx = wiring(rng, I, O)
    W = np.clip(rng.normal(0.5, 0.25, (O, 64)), 0, 1).astype(np.float32)
    x = (rng.random((I, F), dtype=np.float32) * 1.2 - 0.1).astype(np.float32)     # also exercises the [0,1] clip
    dy = rng.random((O, F), dtype=np.float32)
    dW0 = rng.random((O, 64), dtype=np.float32)
    fl = dict(binary=binary, lut_binarize=lut_binarize)
    y = port.sl6_forward(x, idx, W, **fl)
    dx, dW = port.sl6_backward(x, dy, idx, W, I, dW=dW0, **fl)
    _sl6_check(ops, x, idx, W, dy, dW0, fl, dict(y=y, dx=dx, dW=dW), stride)


@pytest.mark.parametrize("case", golden_cases("sl6bit"))
def test_sl6_bit_golden(ops, golden, case):
    from gpu_util import dev_bits, dev_fp32, dev, host_fp32, host_bits, err
    g = lambda n: golden[case + "_" + n]
    fl = _flags(case)
    F = g("dy").shape[1]
    I = g("x").shape[0]
    xd = dev_bits(g("x"), F)
    y = ops.stochastic_lut6_forward(xd, dev(g("idx")), dev(g("W")), F, **fl)
    assert err(host_fp32(y, F), g("y")) <= TOL
    dWd = torch.zeros((g("idx").shape[0], 64), device="cuda")
    dx = ops.stochastic_lut6_backward(xd, dev_fp32(g("dy")), dev(g("idx")), dev(g("W")), dWd, I, F, **fl)
    assert err(host_fp32(dx, F), g("dx")) <= TOL and err(dWd.cpu().numpy(), g("dW")) <= TOL
    # bit -> bit: y = lut > 0.5, compared where the oracle is not on the threshold
    yb = ops.stochastic_lut6_forward(xd, dev(g("idx")), dev(g("W")), F, bit_output=True, **fl)
    raw, want = port.sl6_forward(g("x"), g("idx"), g("W"), frames=F, want_bits=True, **fl)
    bad = unpack_bits(host_bits(yb, F), F) != unpack_bits(want, F)
    assert (np.abs(raw[bad] - 0.5) < 1e-4).all() and bad.mean() < 1e-3


# --------------------------------------------------------------------------------------------- DifferentiableLut6
def _dl6_fp32_check(ops, x, idx, W, dy, rm0, rv0, fl, stride=None):
    from gpu_util import dev_fp32, dev, host_fp32, err
    I, F = x.shape
    O = idx.shape[0]
    p = port.dl6_forward_train(x, idx, W, rm0, rv0, **fl)
    xd = dev_fp32(x, stride)
    rm, rv = dev(rm0.copy()), dev(rv0.copy())
    y, mean, rstd = ops.differentiable_lut6_forward_training(xd, dev(idx), dev(W), rm, rv, F, **fl)
    yh = host_fp32(y, F)
    assert err(mean.cpu().numpy(), p["mean"]) <= TOL
    amp = max(1.0, 0.3 * float(p["rstd"].max()))
    # rstd = 1/sqrt(var) with var = E[y^2] - mean^2 taken in fp32 by both sides: what can be held is the variance to a few
    # ulps of E[y^2] ~ 0.25 (3e-8 each), whatever that is relative to a variance that may sit near its 1e-5 floor
    assert np.abs(1.0 / rstd.cpu().numpy().astype(np.float64) ** 2 - 1.0 / p["rstd"].astype(np.float64) ** 2).max() <= 2e-7
    assert err(rm.cpu().numpy(), p["running_mean"]) <= TOL and err(rv.cpu().numpy(), p["running_var"]) <= TOL
    if fl["binary"]:
        bad = yh != p["y"]
        assert (np.abs(p["y_pre"][bad] - 0.5) < 1e-4 * amp).all() and bad.mean() < 1e-2
    else:
        assert np.abs(yh - p["y"]).max() <= BN_Y_FACTOR * TOL * amp
    # backward with the oracle's own mean / rstd so that only this operator is under test; dy = 0 on the frames whose mask
    # decision is within rounding (see the module docstring), so that every other frame is compared without exception
    edge = _edges(p["y_pre"], amp)
    dy = np.where(edge, np.float32(0), dy).astype(np.float32)
    dx_w, dW_w = port.dl6_backward(x, dy, idx, W, p["mean"], p["rstd"], I, **fl)
    dWd = torch.zeros((O, 64), device="cuda")
    dx = ops.differentiable_lut6_backward(xd, dev_fp32(dy, stride), dev(idx), dev(W), dWd, dev(p["mean"]), dev(p["rstd"]), I, F, **fl)
    dxh = host_fp32(dx, F)
    scale = max(1.0, float(np.abs(dx_w).max()))
    assert np.abs(dxh - dx_w).max() <= BN_GRAD_FACTOR * TOL * scale * amp
    assert err(dWd.cpu().numpy(), dW_w) <= BN_GRAD_FACTOR * TOL * amp
    # inference
    pi = port.dl6_forward_infer(x, idx, W, rm0, rv0, **fl)
    yi = host_fp32(ops.differentiable_lut6_forward_inference(xd, dev(idx), dev(W), dev(rm0), dev(rv0), F, **fl), F)
    if fl["binary"]:
        bad = yi != pi["y"]
        assert (np.abs(pi["y_pre"][bad] - 0.5) < 1e-4).all()
    else:
        assert np.abs(yi - pi["y"]).max() <= BN_Y_FACTOR * TOL
    return int(edge.sum())


@pytest.mark.parametrize("case", golden_cases("dl6"))
def test_dl6_fp32_golden(ops, golden, case):
    from gpu_util import dev_fp32, dev, host_fp32, err
    g = lambda n: golden[case + "_" + n]
    fl = _flags(case)
    _dl6_fp32_check(ops, g("x"), g("idx"), g("W"), g("dy"), g("rm0"), g("rv0"), fl)
    # and against the reference's own numbers
    F = g("x").shape[1]
    rm, rv = dev(g("rm0").copy()), dev(g("rv0").copy())
    y, mean, rstd = ops.differentiable_lut6_forward_training(dev_fp32(g("x")), dev(g("idx")), dev(g("W")), rm, rv, F, **fl)
    assert err(mean.cpu().numpy(), g("mean")) <= TOL and err(rm.cpu().numpy(), g("rm")) <= TOL
    if not fl["binary"]:
        assert np.abs(host_fp32(y, F) - g("y")).max() <= BN_Y_FACTOR * TOL * max(1.0, 0.3 * float(g("rstd").max()))
    # the reference's own dx / dW for the golden dy, outside the nodes that own a frame with an undecidable mask
    p = port.dl6_forward_train(g("x"), g("idx"), g("W"), g("rm0"), g("rv0"), **fl)
    amp = max(1.0, 0.3 * float(p["rstd"].max()))
    I, O = g("x").shape[0], g("idx").shape[0]
    node_ok, row_ok = _untouched(_edges(p["y_pre"], amp), g("idx"), I)
    dWd = torch.zeros((O, 64), device="cuda")
    dx = ops.differentiable_lut6_backward(dev_fp32(g("x")), dev_fp32(g("dy")), dev(g("idx")), dev(g("W")), dWd, dev(g("mean")), dev(g("rstd")),
                                          I, F, **fl)
    scale = max(1.0, float(np.abs(g("dx")).max()))
    assert np.abs(host_fp32(dx, F) - g("dx"))[row_ok].max(initial=0.0) <= BN_GRAD_FACTOR * TOL * scale * amp
    assert np.abs(dWd.cpu().numpy() - g("dW"))[node_ok].max(initial=0.0) <= BN_GRAD_FACTOR * TOL * amp * max(1.0, float(np.abs(g("dW")).max()))


@pytest.mark.parametrize("I,O,F,stride", [(16, 16, 131, None), (24, 1024, 64, None), (200, 300, 1100, 1104), (6, 2, 39, 64),
                                          (1024, 2048, 512, None), (6, 1, 1, None), (16, 16, 1024, None)])
@pytest.mark.parametrize("binary,lut_binarize", [(0, 0), (1, 0), (1, 1), (0, 1)])
def test_dl6_fp32_oracle(ops, I, O, F, stride, binary, lut_binarize):
    from gpu_util import wiring
    rng = np.random.default_rng(I + 31 * O + F)
    idx = wiring(rng, I, O)
    W = np.clip(rng.normal(0.5, 0.25, (O, 64)), 0, 1).astype(np.float32)
    x = rng.random((I, F), dtype=np.float32)
    dy = rng.random((O, F), dtype=np.float32)
    rm0 = rng.random(O, dtype=np.float32)
    rv0 = rng.random(O, dtype=np.float32) + 0.5
    _dl6_fp32_check(ops, x, idx, W, dy, rm0, rv0, dict(binary=binary, lut_binarize=lut_binarize), stride)


def test_dl6_fp32_fresh_layer_tables(ops):
    """Tables N(0.5, 0.01) as a new layer has them: variance at the 1e-5 floor, gamma*rstd = 95."""
    from gpu_util import wiring
    rng = np.random.default_rng(99)
    I, O, F = 784, 1024, 512
    idx = wiring(rng, I, O)
    W = np.clip(rng.normal(0.5, 0.01, (O, 64)), 0, 1).astype(np.float32)
    x = rng.random((I, F), dtype=np.float32)
    dy = rng.random((O, F), dtype=np.float32)
    n_edge = _dl6_fp32_check(ops, x, idx, W, dy, np.zeros(O, np.float32), np.ones(O, np.float32), dict(binary=0, lut_binarize=0))
    assert n_edge < 0.02 * O * F          # the zeroed-dy frames are a small minority: the comparison above covered the rest


@pytest.mark.parametrize("case", golden_cases("dl6bit"))
def test_dl6_bit_golden(ops, golden, case):
    from gpu_util import dev_bits, dev_fp32, dev, host_fp32, host_bits, err
    g = lambda n: golden[case + "_" + n]
    fl = _flags(case)
    F = g("dy").shape[1]
    I = g("x").shape[0]
    O = g("idx").shape[0]
    p = port.dl6_forward_train(g("x"), g("idx"), g("W"), np.zeros(O), np.ones(O), frames=F, **fl)
    xd = dev_bits(g("x"), F)
    rm, rv = torch.zeros(O, device="cuda"), torch.ones(O, device="cuda")
    y, mean, rstd = ops.differentiable_lut6_forward_training(xd, dev(g("idx")), dev(g("W")), rm, rv, F, **fl)
    assert err(mean.cpu().numpy(), g("mean")) <= TOL and np.abs(rstd.cpu().numpy() / g("rstd") - 1).max() <= 1e-4
    assert err(rm.cpu().numpy(), g("rm")) <= TOL and err(rv.cpu().numpy(), g("rv")) <= TOL
    amp = max(1.0, 0.3 * float(g("rstd").max()))
    bad = unpack_bits(host_bits(y, F), F) != unpack_bits(g("y"), F)
    assert (np.abs(p["y_pre"][bad] - 0.5) < 1e-4 * amp).all()
    # the reference's dx / dW for the golden dy, outside the nodes that own a frame with an undecidable mask ...
    edge = _edges(p["y_pre"], amp)
    node_ok, row_ok = _untouched(edge, g("idx"), I)
    dWd = torch.zeros((O, 64), device="cuda")
    dx = ops.differentiable_lut6_backward(xd, dev_fp32(g("dy")), dev(g("idx")), dev(g("W")), dWd, dev(g("mean")), dev(g("rstd")), I, F, **fl)
    scale = max(1.0, float(np.abs(g("dx")).max()))
    assert np.abs(host_fp32(dx, F) - g("dx"))[row_ok].max(initial=0.0) <= BN_GRAD_FACTOR * TOL * scale * amp
    assert np.abs(dWd.cpu().numpy() - g("dW"))[node_ok].max(initial=0.0) <= BN_GRAD_FACTOR * TOL * amp * max(1.0, float(np.abs(g("dW")).max()))
    # ... and every node against the oracle with dy zeroed on those frames
    dy0 = np.where(edge, np.float32(0), g("dy")).astype(np.float32)
    dx_w, dW_w = port.dl6_backward(g("x"), dy0, g("idx"), g("W"), g("mean"), g("rstd"), I, frames=F, **fl)
    dWd = torch.zeros((O, 64), device="cuda")
    dx = ops.differentiable_lut6_backward(xd, dev_fp32(dy0), dev(g("idx")), dev(g("W")), dWd, dev(g("mean")), dev(g("rstd")), I, F, **fl)
    assert err(host_fp32(dx, F), dx_w) <= BN_GRAD_FACTOR * TOL * amp and err(dWd.cpu().numpy(), dW_w) <= BN_GRAD_FACTOR * TOL * amp
    yi = ops.differentiable_lut6_forward_inference(xd, dev(g("idx")), dev(g("W")), dev(g("rm")), dev(g("rv")), F, **fl)
    pi = port.dl6_forward_infer(g("x"), g("idx"), g("W"), g("rm"), g("rv"), frames=F, **fl)
    bad = unpack_bits(host_bits(yi, F), F) != unpack_bits(g("y_infer"), F)
    assert (np.abs(pi["y_pre"][bad] - 0.5) < 1e-4).all()


def test_dl6_bit_oracle_odd_sizes(ops):
    from gpu_util import dev_bits, dev_fp32, dev, host_fp32, host_bits, err, wiring
    rng = np.random.default_rng(5)
    for (I, O, F) in [(40, 33, 1529), (512, 1024, 1024), (7, 3, 31), (6, 1, 1), (16, 2, 39)]:
        idx = wiring(rng, I, O)
        W = np.clip(rng.normal(0.5, 0.25, (O, 64)), 0, 1).astype(np.float32)
        xb = pack_bits(rng.random((I, F)) > 0.5)
        dy = rng.random((O, F), dtype=np.float32)
        p = port.dl6_forward_train(xb, idx, W, np.zeros(O), np.ones(O), frames=F)
        xd = dev_bits(xb, F)
        rm, rv = torch.zeros(O, device="cuda"), torch.ones(O, device="cuda")
        y, mean, rstd = ops.differentiable_lut6_forward_training(xd, dev(idx), dev(W), rm, rv, F)
        amp = max(1.0, 0.3 * float(p["rstd"].max()))
        assert err(mean.cpu().numpy(), p["mean"]) <= TOL
        bad = unpack_bits(host_bits(y, F), F) != unpack_bits(p["y_bits"], F)
        assert (np.abs(p["y_pre"][bad] - 0.5) < 1e-4 * amp).all() and bad.mean() < 1e-3
        dy = np.where(_edges(p["y_pre"], amp), np.float32(0), dy).astype(np.float32)      # frames with an undecidable mask carry no gradient
        dx_w, dW_w = port.dl6_backward(xb, dy, idx, W, p["mean"], p["rstd"], I)
        dWd = torch.zeros((O, 64), device="cuda")
        dx = ops.differentiable_lut6_backward(xd, dev_fp32(dy), dev(idx), dev(W), dWd, dev(p["mean"]), dev(p["rstd"]), I, F)
        assert err(host_fp32(dx, F), dx_w) <= BN_GRAD_FACTOR * TOL * amp and err(dWd.cpu().numpy(), dW_w) <= BN_GRAD_FACTOR * TOL * amp


# --------------------------------------------------------------------------------------------- StochasticBatchNormalization
@pytest.mark.parametrize("O,F,stride", [(16, 39, None), (8, 200, None), (33, 10000, 10008), (5, 7, 16)])
def test_sbn_oracle(ops, O, F, stride):
    from gpu_util import dev_fp32, dev, host_fp32, err
    rng = np.random.default_rng(O + F)
    x = rng.random((O, F), dtype=np.float32)
    dy = rng.random((O, F), dtype=np.float32)
    rm0 = rng.random(O, dtype=np.float32)
    rv0 = rng.random(O, dtype=np.float32) + 0.5
    p = port.sbn_forward_train(x, rm0, rv0)
    xd = dev_fp32(x, stride)
    rm, rv = dev(rm0.copy()), dev(rv0.copy())
    y, mean, rstd = ops.stochastic_bn_forward_training(xd, rm, rv, F)
    assert err(host_fp32(y, F), p["y"]) <= 2e-5
    assert err(mean.cpu().numpy(), p["mean"]) <= TOL and np.abs(rstd.cpu().numpy() / p["rstd"] - 1).max() <= 2e-5
    assert err(rm.cpu().numpy(), p["running_mean"]) <= TOL and err(rv.cpu().numpy(), p["running_var"]) <= TOL
    assert err(host_fp32(ops.stochastic_bn_reforward(xd, dev(p["mean"]), dev(p["rstd"]), F), F), port.sbn_reforward(x, p["mean"], p["rstd"])) <= TOL
    assert err(host_fp32(ops.stochastic_bn_forward_inference(xd, dev(rm0), dev(rv0), F), F), port.sbn_forward_infer(x, rm0, rv0)) <= TOL
    dx = ops.stochastic_bn_backward(xd, dev_fp32(dy, stride), dev(p["mean"]), dev(p["rstd"]), F)
    assert err(host_fp32(dx, F), port.sbn_backward(x, dy, p["mean"], p["rstd"])) <= 2e-5


# --------------------------------------------------------------------------------------------- BinaryLut6
@pytest.mark.parametrize("case", golden_cases("bl6"))
def test_binary_lut6_golden_bit_exact(ops, golden, case):
    from gpu_util import dev_bits, dev, host_bits
    g = lambda n: golden[case + "_" + n]
    F = int(case.split("_")[-1])
    y = ops.binary_lut6_forward(dev_bits(g("x"), F), dev(g("idx")), dev(g("table")), F)
    assert (unpack_bits(host_bits(y, F), F) == unpack_bits(g("y"), F)).all()


def test_binary_lut6_truth_tables(ops):
    from gpu_util import dev_bits, dev, host_bits
    frames = np.arange(64)
    x = pack_bits(((frames[None, :] >> np.arange(6)[:, None]) & 1).astype(np.uint8))
    idx = np.arange(6, dtype=np.int32)[None, :]
    for t in (0x8000000000000000, 0xFFFFFFFFFFFFFFFE, 0x6996966996696996, 0x0123456789ABCDEF, 0, 2**64 - 1):
        table = np.array([[t & 0xFFFFFFFF, t >> 32]], dtype=np.uint64).astype(np.uint32).view(np.int32)
        y = unpack_bits(host_bits(ops.binary_lut6_forward(dev_bits(x, 64), dev(idx), dev(table), 64), 64), 64)[0]
        assert (y == [(t >> i) & 1 for i in range(64)]).all()


@pytest.mark.parametrize("I,O,F,stride", [(16, 16, 32, None), (40, 33, 300, None), (1000, 3000, 5000, None), (64, 70000, 64, None),
                                          (50, 20, 100, 5), (1, 1, 1, None)])
def test_binary_lut6_oracle_bit_exact(ops, I, O, F, stride):
    from gpu_util import dev_bits, dev, host_bits, wiring
    rng = np.random.default_rng(I + O + F)
    idx = wiring(rng, I, O) if I >= 6 else np.zeros((O, 6), np.int32)
    table = rng.integers(-2**31, 2**31, (O, 2)).astype(np.int32)
    xb = pack_bits(rng.random((I, F)) > 0.5)
    want = port.binary_lut6_forward(xb, idx, table, F)
    y = ops.binary_lut6_forward(dev_bits(xb, F, stride), dev(idx), dev(table), F)
    assert (unpack_bits(host_bits(y, F), F) == unpack_bits(want, F)).all()


@pytest.mark.parametrize("I,O,F", [(16, 16, 32), (40, 33, 300), (1000, 3000, 5000), (64, 9000, 16384 + 96), (6, 1, 1)])
def test_binary_lut6_lop3_immediate_kernel_bit_exact(ops, I, O, F):
    """The truth-table-immediate evaluation (one indexed branch per table byte) against the oracle: ragged last item, ragged last
    word, node counts that do not fill the last group, every table byte value."""
    from gpu_util import dev_bits, dev, host_bits, wiring
    rng = np.random.default_rng(I + O + F + 1)
    idx = wiring(rng, I, O)
    table = rng.integers(-2**31, 2**31, (O, 2)).astype(np.int32)
    if O >= 256:        # every byte value 0..255 in every byte position
        t64 = np.zeros(256, np.uint64)
        for pos in range(8):
            t64 ^= (np.arange(256, dtype=np.uint64) ^ np.uint64(37 * pos)) % np.uint64(256) << np.uint64(8 * pos)
        table[:256] = np.stack([(t64 & np.uint64(0xFFFFFFFF)), (t64 >> np.uint64(32))], axis=1).astype(np.uint32).view(np.int32)
    xb = pack_bits(rng.random((I, F)) > 0.5)
    want = port.binary_lut6_forward(xb, idx, table, F)
    y = ops.binary_lut6_forward(dev_bits(xb, F), dev(idx), dev(table), F, lop3_immediate=True)
    assert (unpack_bits(host_bits(y, F), F) == unpack_bits(want, F)).all()


def test_binary_lut6_host_buffers_bit_exact(ops):
    """The host-buffer entry point (chunked upload / kernel / download) against the oracle; ragged last chunk and last word."""
    from gpu_util import wiring
    rng = np.random.default_rng(77)
    for (I, O, F, pinned) in [(300, 200, 32 * 4096 * 2 + 1000, True), (64, 48, 999, False)]:
        idx = wiring(rng, I, O)
        table = rng.integers(-2**31, 2**31, (O, 2)).astype(np.int32)
        xb = pack_bits(rng.random((I, F)) > 0.5)
        hx = torch.from_numpy(xb.view(np.int32))
        hy = torch.zeros((O, xb.shape[1]), dtype=torch.int32)
        if pinned:
            hx, hy = hx.pin_memory(), hy.pin_memory()
        ops.binary_lut6_forward_host(hx, torch.from_numpy(idx), torch.from_numpy(table), F, y=hy)
        want = port.binary_lut6_forward(xb, idx, table, F)
        got = np.ascontiguousarray(hy.numpy()).view(np.uint32)
        assert (unpack_bits(got, F) == unpack_bits(want, F)).all()


def test_binary_lut6_full_size_properties(ops):
    """The full-size shape (16384 -> 16384 nodes, 2^20 frames): properties that need no CPU pass.

    (a) a table that projects input k reproduces that input row bit for bit (gather indexing);
    (b) complementing the table complements the output; (c) a 4096-node x 8192-frame window agrees with the oracle."""
    I = O = 16384
    F = 1 << 20
    S = F // 32
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randint(-2**31, 2**31 - 1, (I, S), dtype=torch.int32, device="cuda", generator=g)
    idx = torch.stack([torch.randperm(I, device="cuda", generator=g)[:O] for _ in range(6)], dim=1).to(torch.int32).contiguous()
    # (a) projection tables: node n projects input (n % 6)
    proj = [0xAAAAAAAAAAAAAAAA, 0xCCCCCCCCCCCCCCCC, 0xF0F0F0F0F0F0F0F0, 0xFF00FF00FF00FF00, 0xFFFF0000FFFF0000, 0xFFFFFFFF00000000]
    tab = np.array([[p & 0xFFFFFFFF, p >> 32] for p in proj], dtype=np.uint64).astype(np.uint32).view(np.int32)
    k = torch.arange(O, device="cuda") % 6
    table = torch.from_numpy(tab).cuda()[k].contiguous()
    y = ops.binary_lut6_forward(x, idx, table, F)
    src = idx.gather(1, k[:, None].to(torch.int64)).squeeze(1).to(torch.int64)
    for lo in range(0, O, 2048):
        assert torch.equal(y[lo:lo + 2048], x[src[lo:lo + 2048]])
    # (b) complement
    table = torch.randint(-2**31, 2**31 - 1, (O, 2), dtype=torch.int32, device="cuda", generator=g)
    y1 = ops.binary_lut6_forward(x, idx, table, F)
    y2 = ops.binary_lut6_forward(x, idx, ~table, F)
    assert torch.equal(y1, ~y2)
    # (c) window against the oracle
    xs = np.ascontiguousarray(x[:, :256].cpu().numpy()).view(np.uint32)
    want = port.binary_lut6_forward(xs, idx[:4096].cpu().numpy(), table[:4096].cpu().numpy(), 8192)
    got = np.ascontiguousarray(y1[:4096, :256].cpu().numpy()).view(np.uint32)
    assert (got == want).all()


# --------------------------------------------------------------------------------------------- behaviour of the ABI
def test_backward_uses_the_callers_scratch_and_falls_back_for_unaligned_rows(ops):
    """dev_dx_tmp, as the reference's callers hand it in, serves as the backward's scratch (the device heap does not grow); a buffer
    that is too small is ignored; rows that are not 16-byte aligned (odd stride) take the plain-load kernels.  All against the oracle."""
    from gpu_util import dev_fp32, dev, host_fp32, err, wiring
    rng = np.random.default_rng(17)
    I, O, F = 120, 200, 700
    idx = wiring(rng, I, O)
    W = np.clip(rng.normal(0.5, 0.25, (O, 64)), 0, 1).astype(np.float32)
    x, dy = rng.random((I, F), dtype=np.float32), rng.random((O, F), dtype=np.float32)
    dx_w, dW_w = port.sl6_backward(x, dy, idx, W, I)
    L = ops.abi.lib()
    for stride, tmp_cols in ((704, 256), (704, 8), (701, 256), (703, None)):
        xd, dyd = dev_fp32(x, stride), dev_fp32(dy, stride)
        tmp = None if tmp_cols is None else torch.empty((6 * O, tmp_cols), device="cuda")
        dW = torch.zeros((O, 64), device="cuda")
        torch.cuda.synchronize()
        before = L.bbcu_LocalHeap_GetAllocatedSize()
        dx = ops.stochastic_lut6_backward(xd, dyd, dev(idx), dev(W), dW, I, F, dx_tmp=tmp)
        torch.cuda.synchronize()
        if stride % 4 == 0 and tmp_cols == 256:
            assert L.bbcu_LocalHeap_GetAllocatedSize() == before           # the caller's buffer was enough
        assert err(host_fp32(dx, F), dx_w) <= TOL and err(dW.cpu().numpy(), dW_w) <= TOL, (stride, tmp_cols)
    # DifferentiableLut6 through the same two routes, and the forward on unaligned rows
    p = port.dl6_forward_train(x, idx, W, np.zeros(O), np.ones(O), binary=False)
    amp = max(1.0, 0.3 * float(p["rstd"].max()))
    dyz = np.where(_edges(p["y_pre"], amp), np.float32(0), dy).astype(np.float32)
    dx_w, dW_w = port.dl6_backward(x, dyz, idx, W, p["mean"], p["rstd"], I, binary=False)
    for stride, tmp_cols in ((704, 256), (701, None)):
        xd = dev_fp32(x, stride)
        y, mean, rstd = ops.differentiable_lut6_forward_training(xd, dev(idx), dev(W), torch.zeros(O, device="cuda"), torch.ones(O, device="cuda"), F,
                                                                 binary=False)
        assert np.abs(host_fp32(y, F) - p["y"]).max() <= BN_Y_FACTOR * TOL * amp and err(mean.cpu().numpy(), p["mean"]) <= TOL
        tmp = None if tmp_cols is None else torch.empty((6 * O, tmp_cols), device="cuda")
        dW = torch.zeros((O, 64), device="cuda")
        dx = ops.differentiable_lut6_backward(xd, dev_fp32(dyz, stride), dev(idx), dev(W), dW, dev(p["mean"]), dev(p["rstd"]), I, F, binary=False,
                                              dx_tmp=tmp)
        scale = max(1.0, float(np.abs(dx_w).max()))
        assert np.abs(host_fp32(dx, F) - dx_w).max() <= BN_GRAD_FACTOR * TOL * scale * amp
        assert err(dW.cpu().numpy(), dW_w) <= BN_GRAD_FACTOR * TOL * amp
        ys = ops.stochastic_lut6_forward(xd, dev(idx), dev(W), F)
        assert err(host_fp32(ys, F), port.sl6_forward(x, idx, W)) <= TOL



def test_binary_mode_takes_the_tree_kernels_when_the_pattern_scratch_is_refused(ops):
    """Binary mode on fp32 frames normally goes through per-pattern tables that need one byte of scratch per node-frame; when the
    device heap refuses that block the operators must decline to the per-frame tree kernels and give the same results.  The heap's
    byte limit is set to what is already allocated (the small per-stream scratch of a plain-mode call), so nothing on the GPU runs
    out of memory."""
    from gpu_util import dev_fp32, dev, wiring
    rng = np.random.default_rng(23)
    I, O, F = 48, 64, 2048
    idx = wiring(rng, I, O)
    W = np.clip(rng.normal(0.5, 0.25, (O, 64)), 0, 1).astype(np.float32)
    x, dy = rng.random((I, F), dtype=np.float32), rng.random((O, F), dtype=np.float32)
    rm0, rv0 = np.zeros(O, np.float32), np.ones(O, np.float32)
    L = ops.abi.lib()
    torch.cuda.synchronize()
    L.bbcu_LocalHeap_GarbageCollect()                                # earlier tests' scratch (possibly large enough already) goes back
    ops.differentiable_lut6_forward_training(dev_fp32(x), dev(idx), dev(W), dev(rm0.copy()), dev(rv0.copy()), F, binary=False)
    torch.cuda.synchronize()
    allocated = L.bbcu_LocalHeap_GetAllocatedSize()
    assert allocated > 0
    L.bbcu_LocalHeap_SetByteLimit(allocated)
    try:
        for lut_binarize in (0, 1):
            _dl6_fp32_check(ops, x, idx, W, dy, rm0, rv0, dict(binary=1, lut_binarize=lut_binarize))
        assert L.bbcu_LocalHeap_GetAllocatedSize() == allocated      # nothing grew
    finally:
        L.bbcu_LocalHeap_SetByteLimit(0)


def test_determinism_and_dw_accumulation(ops):
    from gpu_util import dev_fp32, dev, wiring
    rng = np.random.default_rng(3)
    I, O, F = 256, 512, 777
    idx, W = dev(wiring(rng, I, O)), dev(rng.random((O, 64), dtype=np.float32))
    x, dy = dev_fp32(rng.random((I, F), dtype=np.float32)), dev_fp32(rng.random((O, F), dtype=np.float32))
    y1 = ops.stochastic_lut6_forward(x, idx, W, F)
    y2 = ops.stochastic_lut6_forward(x, idx, W, F)
    assert torch.equal(y1[:, :F], y2[:, :F])
    dW = torch.zeros((O, 64), device="cuda")
    ops.stochastic_lut6_backward(x, dy, idx, W, dW, I, F)
    once = dW.clone()
    ops.stochastic_lut6_backward(x, dy, idx, W, dW, I, F)          # dW is accumulated into, dx overwritten
    assert torch.allclose(dW, 2 * once, rtol=1e-5, atol=1e-5)


def test_argument_errors_do_not_reach_the_gpu(ops):
    from binarybrain_b200 import abi
    L = abi.lib()
    x = torch.zeros((8, 8), device="cuda")
    idx = torch.zeros((4, 6), dtype=torch.int32, device="cuda")
    W = torch.zeros((4, 64), device="cuda")
    p = lambda t: t.data_ptr()
    assert L.bbcu_fp32_StochasticLut6_Forward(0, p(x), p(idx), p(W), 4, 8, 8, 0, 0, 0.25, None) == -1
    assert L.bbcu_fp32_StochasticLut6_Forward(p(x), p(x), p(idx), p(W), -1, 8, 8, 0, 0, 0.25, None) == -2
    assert L.bbcu_fp32_StochasticLut6_Forward(p(x), p(x), p(idx), p(W), 4, 9, 8, 0, 0, 0.25, None) == -3
    assert L.bbcu_bit_BinaryLut6_Forward(p(x), p(x), p(idx), 0, 4, 8, 8, None) == -1
    assert b"stride" in L.bbcu_b200_error_string(-3)
    with pytest.raises(abi.BbcuError):
        abi.call("bbcu_fp32_StochasticLut6_Forward", 0, 0, 0, 0, 1, 1, 1, 0, 0, 0.25, None)
    # empty inputs are a no-op, not an error
    assert L.bbcu_fp32_StochasticLut6_Forward(p(x), p(x), p(idx), p(W), 0, 8, 8, 0, 0, 0.25, None) == 0
    assert L.bbcu_bit_BinaryLut6_Forward(p(x), p(x), p(idx), p(idx), 4, 0, 8, None) == 0
    torch.cuda.synchronize()


def test_no_kernel_recorded_a_fault(ops):
    """Kernels with bounded waits record a fault code instead of hanging; after a normal run it is still 0."""
    from binarybrain_b200 import abi
    from gpu_util import dev_bits, dev, wiring
    rng = np.random.default_rng(2)
    I, O, F = 512, 1000, 40000              # several pipeline rounds per warp, ragged last tile and last node group
    xb = pack_bits(rng.random((I, F)) > 0.5)
    y = ops.binary_lut6_forward(dev_bits(xb, F), dev(wiring(rng, I, O)), dev(rng.integers(-2**31, 2**31, (O, 2)).astype(np.int32)), F)
    assert y.shape[0] == O
    assert abi.lib().bbcu_b200_device_fault() == 0


def test_a_wait_that_nothing_completes_gives_up_and_is_reported(ops):
    """The bounded-wait path itself: the library's self-test arms a barrier that no copy completes; the warp gives up after its
    attempt limit, records fault code 1 and returns.  The context stays usable and the next query is clean."""
    from binarybrain_b200 import abi
    from gpu_util import dev_bits, dev, host_bits, wiring
    L = abi.lib()
    assert L.bbcu_b200_device_fault() == 0
    abi.call("bbcu_b200_selftest_wait_expiry", torch.cuda.current_stream().cuda_stream)
    assert L.bbcu_b200_device_fault() == 1          # reported once ...
    assert L.bbcu_b200_device_fault() == 0          # ... and cleared
    rng = np.random.default_rng(6)
    I, O, F = 64, 40, 3000
    idx, table = wiring(rng, I, O), rng.integers(-2**31, 2**31, (O, 2)).astype(np.int32)
    xb = pack_bits(rng.random((I, F)) > 0.5)
    y = ops.binary_lut6_forward(dev_bits(xb, F), dev(idx), dev(table), F)
    assert (unpack_bits(host_bits(y, F), F) == unpack_bits(port.binary_lut6_forward(xb, idx, table, F), F)).all()
    assert L.bbcu_b200_device_fault() == 0


def test_heap_cache_and_out_of_memory(ops):
    from binarybrain_b200 import abi
    L = abi.lib()
    a = L.bbcu_LocalHeap_Malloc(1 << 20)
    assert a and L.bbcu_LocalHeap_GetAllocatedSize() >= (1 << 20)
    L.bbcu_LocalHeap_Free(a)
    b = L.bbcu_LocalHeap_Malloc((1 << 20) - 4096)            # within 1.5x of the cached block: reused
    assert b == a
    L.bbcu_LocalHeap_Free(b)
    L.bbcu_LocalHeap_GarbageCollect()
    L.bbcu_LocalHeap_SetByteLimit(1 << 20)
    try:
        assert L.bbcu_LocalHeap_Malloc(1 << 22) is None       # refused on the host: no GPU memory is exhausted
    finally:
        L.bbcu_LocalHeap_SetByteLimit(0)
    assert L.bbcu_IsDeviceAvailable() == 1 and L.bbcu_GetDeviceCount() >= 1


def test_adam_100_steps(ops, golden):
    """100 x (forward, backward, Adam update) of one DifferentiableLut6 layer on the GPU vs the reference run: |dW| <= 1e-4."""
    from gpu_util import dev_fp32, dev, host_fp32
    idx, x, dy = golden["adam_idx"], golden["adam_x"], golden["adam_dy"]
    I, F = x.shape
    O = idx.shape[0]
    for key, bn in (("adam", True), ("adamnobn", False)):
        W = dev(golden[key + "_W0"].copy())
        dW = torch.zeros_like(W)
        opt = ops.Adam([W], [dW])
        xd, dyd, idxd = dev_fp32(x), dev_fp32(dy), dev(idx)
        rm, rv = torch.zeros(O, device="cuda"), torch.ones(O, device="cuda")
        for _ in range(100):
            ops.clamp_(W)
            if bn:
                y, mean, rstd = ops.differentiable_lut6_forward_training(xd, idxd, W, rm, rv, F, binary=False)
                ops.differentiable_lut6_backward(xd, dyd, idxd, W, dW, mean, rstd, I, F, binary=False)
            else:
                y = ops.stochastic_lut6_forward(xd, idxd, W, F)
                ops.stochastic_lut6_backward(xd, dyd, idxd, W, dW, I, F)
            opt.update()
        assert np.abs(W.cpu().numpy() - golden[key + "_W100"]).max() <= 1e-4
        if bn:
            assert np.abs(rm.cpu().numpy() - golden["adam_rm100"]).max() <= 1e-4


def test_frame_sharded_halves_equal_the_whole(ops):
    """ForwardStats|ForwardNormalize and BackwardStats|BackwardApply on two frame shards, with the [O,2] fp64 sums added by
    hand (what the all-reduce does), against the unsharded operators on the same GPU."""
    from gpu_util import dev, wiring
    rng = np.random.default_rng(21)
    I, O, F = 300, 500, 1024
    idx, W = dev(wiring(rng, I, O)), dev(np.clip(rng.normal(0.5, 0.25, (O, 64)), 0, 1).astype(np.float32))
    x, dy = dev(rng.random((I, F), dtype=np.float32)), dev(rng.random((O, F), dtype=np.float32))
    rm, rv = torch.zeros(O, device="cuda"), torch.ones(O, device="cuda")
    y_w, mean_w, rstd_w = ops.differentiable_lut6_forward_training(x, idx, W, rm, rv, F, binary=False)
    dW_w = torch.zeros((O, 64), device="cuda")
    dx_w = ops.differentiable_lut6_backward(x, dy, idx, W, dW_w, mean_w, rstd_w, I, F, binary=False)
    cuts = [(0, 384), (384, 1024)]
    xs = [x[:, b:e].contiguous() for b, e in cuts]
    dys = [dy[:, b:e].contiguous() for b, e in cuts]
    ys = [torch.empty((O, e - b), device="cuda") for b, e in cuts]
    sums = [torch.zeros((O, 2), dtype=torch.float64, device="cuda") for _ in cuts]
    for k, (b, e) in enumerate(cuts):
        ops.dl6_forward_stats(xs[k], idx, W, e - b, ys[k], sums[k], binary=False)
    total = sums[0] + sums[1]
    mean, rstd = torch.empty(O, device="cuda"), torch.empty(O, device="cuda")
    for k, (b, e) in enumerate(cuts):
        rm2, rv2 = torch.zeros(O, device="cuda"), torch.ones(O, device="cuda")
        ops.dl6_forward_normalize(ys[k], total, mean, rstd, rm2, rv2, e - b, F, binary=False)
    assert torch.allclose(mean, mean_w, atol=1e-6) and torch.allclose(rstd, rstd_w, rtol=1e-4)
    assert torch.allclose(rm2, rm, atol=1e-6) and torch.allclose(rv2, rv, atol=1e-6)
    assert torch.allclose(torch.cat(ys, 1), y_w, atol=2e-4)
    for k, (b, e) in enumerate(cuts):
        ops.dl6_backward_stats(xs[k], dys[k], idx, W, mean_w, rstd_w, e - b, sums[k], binary=False)
    total = sums[0] + sums[1]
    # the same sums from the layer's output instead of a second LUT evaluation
    from_y = torch.zeros((O, 2), dtype=torch.float64, device="cuda")
    ops.dl6_backward_stats_from_output(y_w, dy, rstd_w, F, from_y)
    scale = float(total.abs().max())
    assert torch.allclose(from_y, total, rtol=1e-4, atol=1e-5 * scale)
    dW = torch.zeros((O, 64), device="cuda")
    dxs = [ops.dl6_backward_apply(xs[k], dys[k], torch.empty((I, e - b), device="cuda"), idx, W, dW, mean_w, rstd_w, total, I, e - b, F, binary=False)
           for k, (b, e) in enumerate(cuts)]
    assert torch.allclose(torch.cat(dxs, 1), dx_w, rtol=1e-4, atol=1e-4 * float(dx_w.abs().max()))
    assert torch.allclose(dW, dW_w, rtol=1e-4, atol=1e-4 * float(dW_w.abs().max()))


@pytest.mark.parametrize("I,O,F", [(14, 16, 8), (14, 1024, 1024), (13, 17, 1529)])
def test_fp32_binary_layer_equals_bit_layer(ops, I, O, F):
    """The reference's cross-check (tests/gtest/StochasticLutNTest.cpp:253-449): a StochasticLut6 layer in binary mode on fp32 frames
    holding 0/1 and the bit-packed layer on the same Bernoulli inputs give the same forward values and the same gradients, although
    they run through different kernels here (the pipelined fp32 tree and the per-pattern tables)."""
    from gpu_util import dev, dev_fp32, dev_bits, host_fp32, wiring
    from oracle import pack_bits
    rng = np.random.default_rng(31)
    idx = wiring(rng, I, O)
    W = np.clip(rng.normal(0.5, 0.25, (O, 64)), 0, 1).astype(np.float32)
    bits = rng.random((I, F)) > 0.5
    dy = rng.random((O, F), dtype=np.float32)
    for lut_binarize in (True, False):
        y_f = ops.stochastic_lut6_forward(dev_fp32(bits.astype(np.float32)), dev(idx), dev(W), F, binary=True, lut_binarize=lut_binarize)
        y_b = ops.stochastic_lut6_forward(dev_bits(pack_bits(bits), F), dev(idx), dev(W), F, lut_binarize=lut_binarize)
        assert np.array_equal(host_fp32(y_f, F), host_fp32(y_b, F))
        dW_f, dW_b = torch.zeros((O, 64), device="cuda"), torch.zeros((O, 64), device="cuda")
        dx_f = ops.stochastic_lut6_backward(dev_fp32(bits.astype(np.float32)), dev_fp32(dy), dev(idx), dev(W), dW_f, I, F, binary=True,
                                            lut_binarize=lut_binarize)
        dx_b = ops.stochastic_lut6_backward(dev_bits(pack_bits(bits), F), dev_fp32(dy), dev(idx), dev(W), dW_b, I, F, lut_binarize=lut_binarize)
        scale = max(1.0, float(dx_f[:, :F].abs().max()))
        assert float((dx_f[:, :F] - dx_b[:, :F]).abs().max()) <= 1e-5 * scale
        assert float((dW_f - dW_b).abs().max()) <= 1e-5 * max(1.0, float(dW_f.abs().max()))


def test_single_rank_binary_layer_uses_the_unsplit_operators(ops):
    """On one rank a binary-mode layer of binarybrain_b200.dist runs the unsplit operators (per-pattern table route); its results equal
    the split halves that the sharded path uses (the same route, cut at the two exchange points): outputs except next to the
    threshold, gradients to 1e-4."""
    from binarybrain_b200.dist import ShardedDifferentiableLut6
    from gpu_util import dev, wiring
    rng = np.random.default_rng(41)
    I, O, F = 200, 300, 1024
    idx, W = dev(wiring(rng, I, O)), dev(np.clip(rng.normal(0.5, 0.25, (O, 64)), 0, 1).astype(np.float32))
    x, dy = dev(rng.random((I, F), dtype=np.float32)), dev(rng.random((O, F), dtype=np.float32))
    layer = ShardedDifferentiableLut6(idx, W.clone(), I, binary=True)
    y = layer.forward(x, F, F)
    assert layer._fused
    dx = layer.backward(dy)
    dW = layer.wait_grad()
    # the halves, by hand
    y_h = torch.empty((O, F), device="cuda")
    sums = torch.zeros((O, 2), dtype=torch.float64, device="cuda")
    mean, rstd = torch.empty(O, device="cuda"), torch.empty(O, device="cuda")
    rm, rv = torch.zeros(O, device="cuda"), torch.ones(O, device="cuda")
    ops.dl6_forward_stats(x, idx, W, F, y_h, sums, binary=True)
    ops.dl6_forward_normalize(y_h, sums, mean, rstd, rm, rv, F, F, binary=True)
    assert float((y != y_h).float().mean()) < 1e-3
    assert torch.allclose(layer.mean, mean, atol=1e-6) and torch.allclose(layer.rstd, rstd, rtol=1e-4)
    ops.dl6_backward_stats(x, dy, idx, W, mean, rstd, F, sums, binary=True)
    dW_h = torch.zeros((O, 64), device="cuda")
    dx_h = torch.empty((I, F), device="cuda")
    ops.dl6_backward_apply(x, dy, dx_h, idx, W, dW_h, mean, rstd, sums, I, F, F, binary=True)
    amp = max(1.0, 0.3 * float(rstd.max()))
    assert float((dx - dx_h).abs().max()) <= 1e-4 * amp * max(1.0, float(dx_h.abs().max()))
    assert float((dW - dW_h).abs().max()) <= 1e-4 * amp * max(1.0, float(dW_h.abs().max()))


@pytest.mark.parametrize("binary", [True, False])
def test_two_frame_shards_equal_the_whole_batch(ops, binary):
    """The split operators on two frame shards, with the host adding the [O, 2] sums in between (what the all-reduce does), against the
    unsplit operators on the whole batch: binary mode takes the per-pattern table route in both halves, probability mode the tree
    kernels.  Also: an apply half that does not follow its own statistics half (other pointers) recomputes instead of reusing."""
    from gpu_util import dev, wiring
    rng = np.random.default_rng(43)
    I, O, F, H = 200, 300, 1024, 512
    idx, W = dev(wiring(rng, I, O)), dev(np.clip(rng.normal(0.5, 0.25, (O, 64)), 0, 1).astype(np.float32))
    x, dy = dev(rng.random((I, F), dtype=np.float32)), dev(rng.random((O, F), dtype=np.float32))
    rm, rv = torch.zeros(O, device="cuda"), torch.ones(O, device="cuda")
    y_w, mean_w, rstd_w = ops.differentiable_lut6_forward_training(x, idx, W, rm.clone(), rv.clone(), F, binary=binary)
    dW_w = torch.zeros((O, 64), device="cuda")
    dx_w = ops.differentiable_lut6_backward(x, dy, idx, W, dW_w, mean_w, rstd_w, I, F, binary=binary)
    xs = [x[:, :H].contiguous(), x[:, H:].contiguous()]
    dys = [dy[:, :H].contiguous(), dy[:, H:].contiguous()]
    ys = [torch.empty((O, H), device="cuda") for _ in range(2)]
    sums = [torch.zeros((O, 2), dtype=torch.float64, device="cuda") for _ in range(2)]
    for k in range(2):
        ops.dl6_forward_stats(xs[k], idx, W, H, ys[k], sums[k], binary=binary)
    total = sums[0] + sums[1]
    mean, rstd = torch.empty(O, device="cuda"), torch.empty(O, device="cuda")
    for k in range(2):
        ops.dl6_forward_normalize(ys[k], total.clone(), mean, rstd, rm.clone(), rv.clone(), H, F, binary=binary)
    assert torch.allclose(mean, mean_w, atol=1e-6) and torch.allclose(rstd, rstd_w, rtol=1e-4)
    assert float((torch.cat(ys, dim=1) != y_w).float().mean()) < (1e-3 if binary else 1.0)
    if not binary:
        assert float((torch.cat(ys, dim=1) - y_w).abs().max()) <= 1e-4 * max(1.0, 0.3 * float(rstd_w.max()))
    # backward: statistics of both shards first (as two ranks would), then the applies -- the second shard's statistics are the last
    # thing left in the stream's scratch, so shard 0's apply must notice that and recompute, shard 1's may reuse
    for k in range(2):
        ops.dl6_backward_stats(xs[k], dys[k], idx, W, mean_w, rstd_w, H, sums[k], binary=binary)
    total = sums[0] + sums[1]
    dW = torch.zeros((O, 64), device="cuda")
    dxs = [torch.empty((I, H), device="cuda") for _ in range(2)]
    for k in range(2):
        ops.dl6_backward_apply(xs[k], dys[k], dxs[k], idx, W, dW, mean_w, rstd_w, total.clone(), I, H, F, binary=binary)
    amp = max(1.0, 0.3 * float(rstd_w.max()))
    assert float((torch.cat(dxs, dim=1) - dx_w).abs().max()) <= 1e-4 * amp * max(1.0, float(dx_w.abs().max()))
    assert float((dW - dW_w).abs().max()) <= 1e-4 * amp * max(1.0, float(dW_w.abs().max()))
