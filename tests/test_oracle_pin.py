"""Pins the C oracle (oracle/lut6_oracle.c) to the reference.

1. Against tests/golden/lut6_golden.npz, which tests/golden/make_golden.py produced by running
   the unmodified reference headers (always runs).
2. Against oracle/_ref/libbbref.so directly on fresh seeded inputs, where that library exists.

Tolerances: bit-exact for BinaryLut6 and bit-packed outputs; 1e-5 of the value range for fp32
(y in [0,1]; dx, dW compared relative to their max magnitude).
"""
import numpy as np
import pytest

from conftest import golden_cases
from oracle import port, ref, pack_bits, unpack_bits

TOL = 1e-5


def close(a, b, tol=TOL):
    scale = max(1.0, float(np.abs(b).max()))
    return float(np.abs(a - b).max()) <= tol * scale


def flags(case):
    parts = case.split("_")
    d = {}
    for p in parts:
        if p[0] == "b" and p[1:].isdigit():
            d["binary"] = int(p[1:])
        if p[0] == "l" and p[1:].isdigit():
            d["lut_binarize"] = int(p[1:])
    return d


@pytest.mark.parametrize("case", golden_cases("sl6"))
def test_sl6_fp32_golden(golden, case):
    g = lambda n: golden[case + "_" + n]
    fl = flags(case)
    y = port.sl6_forward(g("x"), g("idx"), g("W"), **fl)
    dx, dW = port.sl6_backward(g("x"), g("dy"), g("idx"), g("W"), g("x").shape[0], dW=g("dW0"), **fl)
    assert close(y, g("y")) and close(dx, g("dx")) and close(dW, g("dW"))
    if case + "_y_simd" in golden.files:       # the AVX2 branch agrees with the generic branch to the same tolerance
        assert close(y, g("y_simd")) and close(dx, g("dx_simd")) and close(dW, g("dW_simd"))


@pytest.mark.parametrize("case", golden_cases("sl6bit"))
def test_sl6_bit_golden(golden, case):
    g = lambda n: golden[case + "_" + n]
    F = g("dy").shape[1]
    fl = flags(case)
    y = port.sl6_forward(g("x"), g("idx"), g("W"), frames=F, **fl)
    dx, dW = port.sl6_backward(g("x"), g("dy"), g("idx"), g("W"), g("x").shape[0], **fl)
    assert close(y, g("y")) and close(dx, g("dx")) and close(dW, g("dW"))


@pytest.mark.parametrize("case", golden_cases("dl6"))
def test_dl6_fp32_golden(golden, case):
    g = lambda n: golden[case + "_" + n]
    fl = flags(case)
    I = g("x").shape[0]
    p = port.dl6_forward_train(g("x"), g("idx"), g("W"), g("rm0"), g("rv0"), **fl)
    assert close(p["mean"], g("mean")) and close(p["rstd"] / g("rstd"), np.ones_like(g("rstd")))
    assert close(p["running_mean"], g("rm")) and close(p["running_var"], g("rv"))
    if fl["binary"]:
        bad = p["y"] != g("y")
        assert (np.abs(p["y_pre"][bad] - 0.5) < 1e-4).all() and bad.mean() < 1e-3
    else:
        assert close(p["y"], g("y"), 1e-5 * max(1.0, 0.3 * float(g("rstd").max())))
    dx, dW = port.dl6_backward(g("x"), g("dy"), g("idx"), g("W"), g("mean"), g("rstd"), I, **fl)
    assert close(dx, g("dx"), 2e-5) and close(dW, g("dW"), 2e-5)
    pi = port.dl6_forward_infer(g("x"), g("idx"), g("W"), g("rm0"), g("rv0"), **fl)
    if fl["binary"]:
        bad = pi["y"] != g("y_infer")
        assert (np.abs(pi["y_pre"][bad] - 0.5) < 1e-4).all()
    else:
        assert close(pi["y"], g("y_infer"))


@pytest.mark.parametrize("case", golden_cases("dl6bit"))
def test_dl6_bit_golden(golden, case):
    g = lambda n: golden[case + "_" + n]
    fl = flags(case)
    F = g("dy").shape[1]
    I = g("x").shape[0]
    O = g("idx").shape[0]
    p = port.dl6_forward_train(g("x"), g("idx"), g("W"), np.zeros(O), np.ones(O), frames=F, **fl)
    assert close(p["mean"], g("mean")) and close(p["rstd"] / g("rstd"), np.ones_like(g("rstd")))
    bad = unpack_bits(p["y_bits"], F) != unpack_bits(g("y"), F)
    assert (np.abs(p["y_pre"][bad] - 0.5) < 1e-4).all()
    dx, dW = port.dl6_backward(g("x"), g("dy"), g("idx"), g("W"), g("mean"), g("rstd"), I, **fl)
    assert close(dx, g("dx"), 2e-5) and close(dW, g("dW"), 2e-5)
    pi = port.dl6_forward_infer(g("x"), g("idx"), g("W"), g("rm"), g("rv"), frames=F, **fl)
    bad = unpack_bits(pi["y_bits"], F) != unpack_bits(g("y_infer"), F)
    assert (np.abs(pi["y_pre"][bad] - 0.5) < 1e-4).all()


def test_dl6_without_batch_norm_golden(golden):
    for binary in (0, 1):
        k = f"dl6nobn_14_16_40_b{binary}_"
        y, yb = port.sl6_forward(golden[k + "x"], golden[k + "idx"], golden[k + "W"], binary=binary, want_bits=True)
        if binary:   # DifferentiableLutN.h:987-998: binary mode binarises the output
            assert (unpack_bits(yb, 40) == golden[k + "y"]).all()
        else:
            assert close(y, golden[k + "y"])
        dx, dW = port.sl6_backward(golden[k + "x"], golden[k + "dy"], golden[k + "idx"], golden[k + "W"], 14, binary=binary)
        assert close(dx, golden[k + "dx"]) and close(dW, golden[k + "dW"])
    k = "dl6nobnbit_14_16_70_"
    y, yb = port.sl6_forward(golden[k + "x"], golden[k + "idx"], golden[k + "W"], frames=70, want_bits=True)
    assert (unpack_bits(yb, 70) == unpack_bits(golden[k + "y"], 70)).all()
    dx, dW = port.sl6_backward(golden[k + "x"], golden[k + "dy"], golden[k + "idx"], golden[k + "W"], 14)
    assert close(dx, golden[k + "dx"]) and close(dW, golden[k + "dW"])


@pytest.mark.parametrize("case", golden_cases("bl6"))
def test_binary_lut6_golden_bit_exact(golden, case):
    g = lambda n: golden[case + "_" + n]
    F = int(case.split("_")[-1])
    y = port.binary_lut6_forward(g("x"), g("idx"), g("table"), F)
    assert (unpack_bits(y, F) == unpack_bits(g("y"), F)).all()


def test_binary_lut6_truth_table_semantics():
    """Index bit k is input k and y = table[index] (the known-answer tests of BinaryLutTest.cpp:14-114)."""
    I = 6
    F = 64
    frames = np.arange(F)
    bits = ((frames[None, :] >> np.arange(I)[:, None]) & 1).astype(np.uint8)   # frame f presents index f
    x = pack_bits(bits)
    idx = np.arange(6, dtype=np.int32)[None, :]
    for t in (0x8000000000000000, 0xFFFFFFFFFFFFFFFE, 0x6996966996696996, 0x0123456789ABCDEF):
        table = np.array([[t & 0xFFFFFFFF, t >> 32]], dtype=np.uint64).astype(np.uint32).view(np.int32)
        y = unpack_bits(port.binary_lut6_forward(x, idx, table, F), F)[0]
        assert (y == [(t >> i) & 1 for i in range(64)]).all()


@pytest.mark.parametrize("O,F", [(3, 1), (16, 39), (8, 200)])
def test_sbn_golden(golden, O, F):
    k = f"sbn_{O}_{F}_"
    p = port.sbn_forward_train(golden[k + "x"], golden[k + "rm0"], golden[k + "rv0"])
    assert close(p["y"], golden[k + "y"]) and close(p["mean"], golden[k + "mean"])
    assert close(p["rstd"] / golden[k + "rstd"], np.ones(O))
    assert close(p["running_mean"], golden[k + "rm"]) and close(p["running_var"], golden[k + "rv"])
    assert close(port.sbn_reforward(golden[k + "x"], golden[k + "mean"], golden[k + "rstd"]), golden[k + "y_re"])
    if F > 1:   # with one frame var = 0 and rstd = 1e7: dx is rounding noise of cancelling 1e6-sized terms, not a value
        assert close(port.sbn_backward(golden[k + "x"], golden[k + "dy"], golden[k + "mean"], golden[k + "rstd"]), golden[k + "dx"])


def test_adam_100_steps_golden(golden):
    """100 x (forward, backward, Adam) on one DifferentiableLut6 layer: W within 1e-4 of the reference run."""
    idx, x, dy = golden["adam_idx"], golden["adam_x"], golden["adam_dy"]
    W = golden["adam_W0"].copy()
    O = idx.shape[0]
    m = np.zeros_like(W)
    v = np.zeros_like(W)
    st = np.ones(2, np.float32)
    rm, rv = np.zeros(O, np.float32), np.ones(O, np.float32)
    dW = np.zeros_like(W)
    for _ in range(100):
        np.clip(W, 0, 1, out=W)            # DifferentiableLutN.h:605-608 clamps W before the forward that follows a backward
        p = port.dl6_forward_train(x, idx, W, rm, rv, binary=False)
        rm, rv = p["running_mean"], p["running_var"]
        _, dW = port.dl6_backward(x, dy, idx, W, p["mean"], p["rstd"], x.shape[0], dW=dW, binary=False)
        port.adam_update(W, dW, m, v, st)
    assert np.abs(W - golden["adam_W100"]).max() < 1e-4
    assert np.abs(rm - golden["adam_rm100"]).max() < 1e-4
    # batch norm off, fresh-layer tables N(0.5, 0.01)
    W = golden["adamnobn_W0"].copy()
    m[:] = 0; v[:] = 0; st[:] = 1; dW[:] = 0
    for _ in range(100):
        np.clip(W, 0, 1, out=W)
        _, dW = port.sl6_backward(x, dy, idx, W, x.shape[0], dW=dW)
        port.adam_update(W, dW, m, v, st)
    assert np.abs(W - golden["adamnobn_W100"]).max() < 1e-4


@pytest.mark.skipif(not ref.available(), reason="oracle/_ref not built (needs a reference checkout)")
def test_port_against_reference_build_fresh_inputs():
    rng = np.random.default_rng(7)
    for (I, O, F) in [(13, 17, 1529), (14, 1024, 8)]:       # StochasticLutNTest.cpp:235-246
        idx = np.stack([rng.permutation(I)[:6] for _ in range(O)]).astype(np.int32)
        W = np.clip(rng.normal(0.5, 0.25, (O, 64)), 0, 1).astype(np.float32)
        x = rng.random((I, F), dtype=np.float32)
        dy = rng.random((O, F), dtype=np.float32)
        r = ref.stochastic_lut6(x, idx, W, dy=dy, host_simd=False)
        assert close(port.sl6_forward(x, idx, W), r["y"])
        dx, dW = port.sl6_backward(x, dy, idx, W, I)
        assert close(dx, r["dx"]) and close(dW, r["dW"])
        xb = pack_bits(x > 0.5)
        tbl = rng.integers(-2**31, 2**31, (O, 2)).astype(np.int32)
        assert (unpack_bits(port.binary_lut6_forward(xb, idx, tbl, F), F) == unpack_bits(ref.binary_lut6(xb, idx, tbl, F)["y"], F)).all()
