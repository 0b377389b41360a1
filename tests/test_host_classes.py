"""Host side above the C ABI: the C++ bb:: classes behind the pybind11 module `binarybrain_b200.core`.

CPU tests: library exports vs include/bbcu_b200.h, seeded wiring / table initialisation against the reference's
own draws (golden), FrameBuffer layout.  GPU tests: the layer classes end to end against the oracle, the way
the reference's tests drive them (create, set_input_shape, copy wiring and W, forward, backward, optimizer).
"""
import os
import re

import numpy as np
import pytest

from oracle import port, pack_bits

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def core():
    from binarybrain_b200 import build
    build.build_all()
    import binarybrain_b200.core as c
    return c


def test_library_exports_every_declared_symbol():
    """The C-ABI library loads and exports each function include/bbcu_b200.h declares (no compute call: works without a GPU)."""
    import ctypes
    from binarybrain_b200 import abi, build
    lib = ctypes.CDLL(build.build_library())
    text = open(os.path.join(ROOT, "include", "bbcu_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b(bbcu_[A-Za-z0-9_]+)\s*\(", text))
    assert len(names) >= 40
    missing = [n for n in sorted(names) if not hasattr(lib, n)]
    assert not missing, missing
    assert set(abi.SIGNATURES) == names          # the ctypes table covers the header, no more, no less
    assert lib.bbcu_b200_abi_version() == 1
    lib.bbcu_b200_error_string.restype = ctypes.c_char_p
    assert lib.bbcu_b200_error_string(-1).startswith(b"bbcu_b200")


def test_missing_library_fails_loudly(tmp_path):
    from binarybrain_b200 import abi
    with pytest.raises(ImportError):
        abi.load(str(tmp_path / "nope.so"))


def test_seeded_wiring_and_tables_match_the_reference(core, golden):
    lut = core.DifferentiableLut6_fp32_fp32.create([16], seed=1)
    lut.set_input_shape([32])
    assert (lut.get_connection() == golden["init_32_16_s1_idx"]).all()
    assert np.array_equal(lut.W().numpy(), golden["init_32_16_s1_W"])
    big = core.DifferentiableLut6_fp32_fp32.create([1024], seed=1)
    big.set_input_shape([784])
    idx = big.get_connection()
    assert (idx[:8] == golden["init_784_1024_s1_idx_head"]).all()
    assert int(idx.astype(np.int64).sum()) == int(golden["init_784_1024_s1_idx_sum"][0])
    assert np.array_equal(big.W().numpy()[:2], golden["init_784_1024_s1_W_head"])
    assert all(len(set(r)) == 6 for r in idx.tolist())            # six distinct inputs per node
    # the stochastic layer draws the same way; a different seed gives a different table
    sl = core.StochasticLut6_fp32_fp32.create([16], seed=1)
    sl.set_input_shape([32])
    assert (sl.get_connection() == golden["init_32_16_s1_idx"]).all()
    other = core.DifferentiableLut6_fp32_fp32.create([16], seed=2)
    other.set_input_shape([32])
    assert (other.get_connection() != golden["init_32_16_s1_idx"]).any()


def test_every_wiring_rule_draws_the_reference_tables(core):
    """random / serial / pointwise / depthwise / gauss (include/bb/ConnectionTable.h:150-284): the same seed gives the table the
    reference's layer draws, for 1-D and {c, h, w} node shapes (golden from the unmodified reference; live where it is built)."""
    import sys
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    from make_golden_wiring import CASES, key
    from oracle import ref
    z = np.load(os.path.join(ROOT, "tests", "golden", "wiring_golden.npz"))
    for rule, ins, outs, seed in CASES:
        layer = core.DifferentiableLut6_fp32_fp32.create(outs, connection=rule, seed=seed)
        assert layer.set_input_shape(ins) == outs
        got = layer.get_connection()
        assert np.array_equal(got, z[key(rule, ins, outs, seed)]), (rule, ins, outs)
        assert all(len(set(r)) == 6 for r in got.tolist()) or rule == "serial"
        if ref.available():
            assert np.array_equal(got, ref.init_connection(ins, outs, seed=seed, connection=rule))
    # structure: pointwise stays inside the pixel, depthwise inside the channel
    pw = core.DifferentiableLut6_fp32_fp32.create([9, 5, 4], connection="pointwise", seed=7)
    pw.set_input_shape([12, 5, 4])
    idx = pw.get_connection()
    assert ((idx % 20) == (np.arange(9 * 20) % 20)[:, None]).all()
    dw = core.DifferentiableLut6_fp32_fp32.create([7, 3, 4], connection="depthwise", seed=7)
    dw.set_input_shape([7, 6, 5])
    assert ((dw.get_connection() // 30) == (np.arange(7 * 12) // 12)[:, None]).all()
    with pytest.raises(Exception):
        bad = core.DifferentiableLut6_fp32_fp32.create([8], connection="no_such_rule")
        bad.set_input_shape([16])


def test_framebuffer_layout_and_numpy_round_trip(core):
    rng = np.random.default_rng(0)
    a = rng.random((39, 5), dtype=np.float32)                  # [frames, nodes]
    fb = core.FrameBuffer.from_numpy_fp32(a, core.TYPE_FP32)
    assert fb.get_frame_size() == 39 and fb.get_node_size() == 5
    assert fb.get_frame_stride() == 160 == core.FrameBuffer.calc_frame_stride(core.TYPE_FP32, 39)     # 40 floats: rows padded to 32 bytes
    assert np.array_equal(fb.numpy_fp32(), a)
    assert fb.get_fp32(7, 3) == a[7, 3]
    bits = (a > 0.5).astype(np.float32)
    fbb = core.FrameBuffer.from_numpy_fp32(a, core.TYPE_BIT)
    assert fbb.get_frame_stride() == 32 == core.FrameBuffer.calc_frame_stride(core.TYPE_BIT, 39)       # 256 bits
    assert np.array_equal(fbb.numpy_fp32(), bits)
    fbb.set_fp32(0, 0, 1.0 - bits[0, 0])
    assert fbb.get_fp32(0, 0) == 1.0 - bits[0, 0]
    shaped = core.FrameBuffer(8, [3, 4], core.TYPE_FP32)
    assert shaped.get_node_shape() == [3, 4] and shaped.get_node_size() == 12


def _framebuffer_views(core, on_device):
    """CopyTo / FrameRange / Range / Concatenate / ConvertTo / Clone against numpy slicing, on the host mirror or (on_device) with the
    source made current on the GPU first, which routes through bbcu_int32_FrameBufferCopy / bbcu_fp32_ConvBitToReal."""
    rng = np.random.default_rng(12)
    F, N = 200, 9
    a = rng.random((F, N), dtype=np.float32)
    for dtype, ref in ((core.TYPE_FP32, a), (core.TYPE_BIT, (a > 0.5).astype(np.float32))):
        def make():
            fb = core.FrameBuffer.from_numpy_fp32(a, dtype)
            if on_device:
                assert fb.lock_device() != 0
            return fb
        assert np.array_equal(make().clone().numpy_fp32(), ref)
        assert np.array_equal(make().range(4, 3).numpy_fp32(), ref[:, 3:7])
        assert np.array_equal(make().frame_range(64, 96).numpy_fp32(), ref[96:160])             # word-aligned: the device path for bit frames too
        assert np.array_equal(make().frame_range(50, 7).numpy_fp32(), ref[7:57])                # ragged bit ranges go through the host mirror
        cat = make().concatenate(make().range(2, 0))
        assert cat.get_node_size() == N + 2 and np.array_equal(cat.numpy_fp32(), np.concatenate([ref, ref[:, :2]], axis=1))
        dst = core.FrameBuffer(F, [N], dtype)
        dst.fill_zero()
        make().copy_to(dst, 32, 64, 128, 3, 1, 5)
        want = np.zeros_like(ref)
        want[128:160, 5:8] = ref[64:96, 1:4]
        assert np.array_equal(dst.numpy_fp32(), want)
    bits = core.FrameBuffer.from_numpy_fp32(a, core.TYPE_BIT)
    if on_device:
        bits.lock_device()
    real = bits.convert_to(core.TYPE_FP32)
    assert real.get_type() == core.TYPE_FP32 and np.array_equal(real.numpy_fp32(), (a > 0.5).astype(np.float32))       # 0 / 1, as the reference's CPU branch
    back = core.FrameBuffer.from_numpy_fp32(a, core.TYPE_FP32).convert_to(core.TYPE_BIT)
    assert np.array_equal(back.numpy_fp32(), (a > 0.5).astype(np.float32))


def test_framebuffer_copies_and_views_on_the_host(core):
    _framebuffer_views(core, on_device=False)


@pytest.mark.gpu
def test_framebuffer_copies_and_views_on_the_device(core):
    _framebuffer_views(core, on_device=True)
    big = core.FrameBuffer(40000, [4], core.TYPE_FP32)
    assert big.is_host_pinned()                               # 640 KB mirror: page-locked


@pytest.mark.gpu
def test_frame_buffer_copy_and_bit_to_real_operators():
    """bbcu_int32_FrameBufferCopy / bbcu_fp32_ConvBitToReal through the C ABI: odd offsets, strides that are not multiples of four words,
    rows longer than one CTA's segment."""
    import torch
    from binarybrain_b200 import abi
    g = torch.Generator(device="cuda").manual_seed(5)
    for (nodes, words, ss, ds, so, do_, n_off) in [(7, 9000, 9001, 9003, 1, 2, 1), (3, 4096, 4096, 8192, 0, 4096, 0), (5, 33, 40, 48, 3, 7, 2)]:
        src = torch.randint(-2**31, 2**31 - 1, (nodes + n_off, ss), dtype=torch.int32, device="cuda", generator=g)
        dst = torch.full((nodes + 1, ds), 17, dtype=torch.int32, device="cuda")
        abi.call("bbcu_int32_FrameBufferCopy", dst.data_ptr(), src.data_ptr(), nodes, 1, n_off, words - so, do_, so, ds, ss,
                 torch.cuda.current_stream().cuda_stream)
        want = torch.full_like(dst, 17)
        want[1:1 + nodes, do_:do_ + words - so] = src[n_off:n_off + nodes, so:words]
        assert torch.equal(dst, want)
    for (nodes, frames, xs, ys) in [(5, 1000, 32, 1000), (3, 8193, 264, 8200), (2, 31, 1, 33)]:
        x = torch.randint(-2**31, 2**31 - 1, (nodes, xs), dtype=torch.int32, device="cuda", generator=g)
        y = torch.full((nodes, ys), 9.0, device="cuda")
        abi.call("bbcu_fp32_ConvBitToReal", x.data_ptr(), y.data_ptr(), -1.0, 2.5, nodes, frames, xs, ys, torch.cuda.current_stream().cuda_stream)
        f = torch.arange(frames, device="cuda")
        bit = (x[:, (f >> 5)] >> (f & 31)[None, :]) & 1
        assert torch.equal(y[:, :frames], torch.where(bit.bool(), torch.tensor(2.5, device="cuda"), torch.tensor(-1.0, device="cuda")))
        assert (y[:, frames:] == 9.0).all()


def test_commands_and_defaults(core):
    lut = core.DifferentiableLut6_fp32_fp32.create([4])
    assert lut.get_model_name() == "DifferentiableLut6" and lut.get_gamma() == pytest.approx(0.3) and lut.get_beta() == 0.5
    lut.send_command("binary false")
    lut.send_command("lut_binarize true")
    lut.send_command("momentum 0.5")
    with pytest.raises(RuntimeError):
        lut.send_command("host_only true")                      # no CPU branch in this build
    with pytest.raises(RuntimeError):
        lut.set_input_shape([8])
        lut.set_node_connection_index(0, 0, 99)                 # out of range


# ------------------------------------------------------------------------------------------------ GPU
def _copy_layer(layer, idx, W):
    layer.set_connection(idx)
    layer.W().set_numpy(W)


@pytest.mark.gpu
@pytest.mark.parametrize("binary,lut_binarize", [(False, False), (True, True)])
def test_differentiable_lut6_layer_against_oracle(core, binary, lut_binarize):
    rng = np.random.default_rng(4)
    I, O, F = 64, 48, 200
    lut = core.DifferentiableLut6_fp32_fp32.create([O], momentum=0.9)
    lut.send_command("binary " + ("true" if binary else "false"))
    lut.send_command("lut_binarize " + ("true" if lut_binarize else "false"))
    lut.set_input_shape([I])
    idx = lut.get_connection()
    W = np.clip(rng.normal(0.5, 0.25, (O, 64)), 0, 1).astype(np.float32)
    lut.W().set_numpy(W)
    x = rng.random((F, I), dtype=np.float32)
    dy = rng.random((F, O), dtype=np.float32)
    p = port.dl6_forward_train(x.T.copy(), idx, W, np.zeros(O), np.ones(O), binary=int(binary), lut_binarize=int(lut_binarize))
    amp = max(1.0, 0.3 * float(p["rstd"].max()))
    # frames whose hard-tanh decision is within rounding of the pre-activation carry no gradient in this test (a masked and an
    # unmasked zero are the same), so that every other frame can be compared without exception
    pre = p["y_pre"]
    edge = (np.abs(pre) < 1e-4 * amp) | (np.abs(pre - 1) < 1e-4 * amp)
    dy = np.where(edge.T, np.float32(0), dy).astype(np.float32)
    y = lut.forward(core.FrameBuffer.from_numpy_fp32(x), True).numpy_fp32()
    dx = lut.backward(core.FrameBuffer.from_numpy_fp32(dy)).numpy_fp32()
    dx_w, dW_w = port.dl6_backward(x.T.copy(), dy.T.copy(), idx, W, p["mean"], p["rstd"], I, binary=int(binary), lut_binarize=int(lut_binarize))
    if binary:
        assert (y.T != p["y"]).mean() < 1e-3
    else:
        assert np.abs(y.T - p["y"]).max() <= 3e-5 * amp
    assert np.abs(lut.get_mean().numpy() - p["running_mean"]).max() <= 1e-5
    assert np.abs(dx.T - dx_w).max() <= 1e-4 * amp * max(1.0, np.abs(dx_w).max())
    assert np.abs(lut.dW().numpy() - dW_w).max() <= 1e-4 * amp * max(1.0, np.abs(dW_w).max())
    # inference uses the running statistics
    yi = lut.forward(core.FrameBuffer.from_numpy_fp32(x), False).numpy_fp32()
    pi = port.dl6_forward_infer(x.T.copy(), idx, W, p["running_mean"], p["running_var"], binary=int(binary), lut_binarize=int(lut_binarize))
    assert (np.abs(yi.T - pi["y"]) > 1e-4).mean() < 1e-3


@pytest.mark.gpu
def test_bit_layers_and_binary_lut_import(core):
    rng = np.random.default_rng(6)
    I, O, F = 40, 24, 333
    x = (rng.random((F, I)) > 0.5).astype(np.float32)
    xb = pack_bits(x.T)
    dl = core.DifferentiableLut6_bit_fp32.create([O], momentum=0.9)
    dl.set_input_shape([I])
    W = np.clip(rng.normal(0.5, 0.25, (O, 64)), 0, 1).astype(np.float32)
    dl.W().set_numpy(W)
    idx = dl.get_connection()
    y = dl.forward(core.FrameBuffer.from_numpy_fp32(x, core.TYPE_BIT), True).numpy_fp32()
    p = port.dl6_forward_train(xb, idx, W, np.zeros(O), np.ones(O), frames=F)
    assert (y.T != p["y"]).mean() < 1e-3
    dy = rng.random((F, O), dtype=np.float32)
    dx = dl.backward(core.FrameBuffer.from_numpy_fp32(dy)).numpy_fp32()
    dx_w, _ = port.dl6_backward(xb, dy.T.copy(), idx, W, p["mean"], p["rstd"], I)
    assert np.abs(dx.T - dx_w).max() <= 1e-3 * max(1.0, np.abs(dx_w).max())
    # StochasticLutN<6,Bit>: fp32 output
    sl = core.StochasticLut6_bit_fp32.create([O])
    sl.set_input_shape([I])
    sl.send_command("lut_binarize false")
    _copy_layer(sl, idx, W)
    ys = sl.forward(core.FrameBuffer.from_numpy_fp32(x, core.TYPE_BIT), True).numpy_fp32()
    assert np.abs(ys.T - port.sl6_forward(xb, idx, W, frames=F)).max() <= 1e-5
    # freeze the trained layer into truth tables (table[i] = W[i] >= 0.5) and run the bit-packed inference layer
    bl = core.BinaryLut6_bit_fp32.create([O])
    bl.import_layer(dl)
    table = np.zeros((O, 2), np.int32)
    tb = (W >= 0.5)
    for i in range(64):
        table[:, i >> 5] |= (tb[:, i].astype(np.int64) << (i & 31)).astype(np.uint32).view(np.int32)
        assert bl.get_lut_table(3, i) == bool(tb[3, i])
    yb = bl.forward(core.FrameBuffer.from_numpy_fp32(x, core.TYPE_BIT), False).numpy_fp32()
    want = port.binary_lut6_forward(xb, idx, table, F)
    from oracle import unpack_bits
    assert (yb.T == unpack_bits(want, F)).all()


@pytest.mark.gpu
def test_stochastic_layer_sbn_and_adam(core, golden):
    rng = np.random.default_rng(8)
    # StochasticLutN fp32 + OptimizerAdam: 100 steps against the reference's run (no batch norm, tables N(0.5, 0.01))
    idx, x, dy = golden["adam_idx"], golden["adam_x"], golden["adam_dy"]
    O = idx.shape[0]
    sl = core.DifferentiableLut6_fp32_fp32.create([O], batch_norm=False, binary=False)
    sl.set_input_shape([x.shape[0]])
    _copy_layer(sl, idx, golden["adamnobn_W0"])
    opt = core.OptimizerAdam_fp32.create()
    opt.set_variables(sl.W(), sl.dW())
    xb, dyb = core.FrameBuffer.from_numpy_fp32(x.T.copy()), core.FrameBuffer.from_numpy_fp32(dy.T.copy())
    for _ in range(100):
        sl.forward(xb, True)
        sl.backward(dyb)
        opt.update()
    assert np.abs(sl.W().numpy() - golden["adamnobn_W100"]).max() <= 1e-4
    # StochasticBatchNormalization
    a = rng.random((200, 8), dtype=np.float32)
    bn = core.StochasticBatchNormalization_fp32.create()
    y = bn.forward(core.FrameBuffer.from_numpy_fp32(a), True).numpy_fp32()
    p = port.sbn_forward_train(a.T.copy(), np.zeros(8), np.ones(8))
    assert np.abs(y.T - p["y"]).max() <= 2e-5
    g = rng.random((200, 8), dtype=np.float32)
    dx = bn.backward(core.FrameBuffer.from_numpy_fp32(g)).numpy_fp32()
    assert np.abs(dx.T - port.sbn_backward(a.T.copy(), g.T.copy(), p["mean"], p["rstd"])).max() <= 2e-5
    assert np.abs(bn.get_mean().numpy() - p["running_mean"]).max() <= 1e-6


@pytest.mark.gpu
def test_convolution2d_and_maxpooling_classes_against_oracle(core):
    """bb::Convolution2d (Im2Col -> Sequential of two StochasticLut6 layers -> Col2Im) followed by bb::MaxPooling, through the C++
    host classes; the oracle composes the same operators.  StochasticLut6 (no batch norm) keeps the comparison well conditioned."""
    from oracle import unpack_bits
    rng = np.random.default_rng(9)
    c, h, w, B = 3, 8, 8, 5
    seq = core.Sequential.create()
    l1 = core.StochasticLut6_fp32_fp32.create([24])
    l2 = core.StochasticLut6_fp32_fp32.create([8])
    for layer in (l1, l2):
        layer.send_command("lut_binarize false")
        seq.add(layer)
    conv = core.Convolution2d_fp32_fp32.create(seq, 3, 3, padding="same")
    pool = core.MaxPooling_fp32_fp32.create(2, 2)
    assert conv.set_input_shape([c, h, w]) == [8, h, w]
    assert pool.set_input_shape([8, h, w]) == [8, 4, 4]
    W1 = np.clip(rng.normal(0.5, 0.25, (24, 64)), 0, 1).astype(np.float32)
    W2 = np.clip(rng.normal(0.5, 0.25, (8, 64)), 0, 1).astype(np.float32)
    l1.W().set_numpy(W1)
    l2.W().set_numpy(W2)
    idx1, idx2 = l1.get_connection(), l2.get_connection()
    x = rng.random((B, c * h * w), dtype=np.float32)
    y = pool.forward(conv.forward(core.FrameBuffer.from_numpy_fp32(x.reshape(B, c, h, w)), True), True).numpy_fp32()
    cols = port.im2col_forward(x.T.copy(), c, h, w, 3, 3, padding="same")
    h1 = port.sl6_forward(cols, idx1, W1)
    h2 = port.sl6_forward(h1, idx2, W2)
    img = port.col2im_forward(h2, 8, h, w, B)
    y_w, am = port.maxpool_forward(img, 8, h, w, 2, 2)
    assert np.abs(y.reshape(B, -1).T - y_w).max() <= 1e-5
    dy = rng.random((B, 8 * 4 * 4), dtype=np.float32)
    dx = conv.backward(pool.backward(core.FrameBuffer.from_numpy_fp32(dy.reshape(B, 8, 4, 4)))).numpy_fp32()
    g = port.col2im_backward(port.maxpool_backward(am, dy.T.copy(), 8, h, w, 2, 2), 8, h, w)
    g1, dW2 = port.sl6_backward(h1, g, idx2, W2, 24)
    g0, dW1 = port.sl6_backward(cols, g1, idx1, W1, 27)
    dx_w = port.im2col_backward(g0, c, h, w, 3, 3, padding="same")
    assert np.abs(dx.reshape(B, -1).T - dx_w).max() <= 1e-5 * max(1.0, np.abs(dx_w).max())
    assert np.abs(l1.dW().numpy() - dW1).max() <= 1e-5 * max(1.0, np.abs(dW1).max())
    assert np.abs(l2.dW().numpy() - dW2).max() <= 1e-5 * max(1.0, np.abs(dW2).max())
    # bit frames: 2x2 pooling is an OR
    xb = (rng.random((B, c * h * w)) > 0.7).astype(np.float32)
    pb = core.MaxPooling_bit_fp32.create(2, 2)
    yb = pb.forward(core.FrameBuffer.from_numpy_fp32(xb.reshape(B, c, h, w), core.TYPE_BIT), True).numpy_fp32()
    want = unpack_bits(port.maxpool_forward(pack_bits(xb.T), c, h, w, 2, 2, frames=B), B)
    assert np.array_equal(yb.reshape(B, -1).T > 0.5, want.astype(bool))


@pytest.mark.gpu
@pytest.mark.parametrize("binary", [False, True])
def test_cpp_layer_frame_shards_equal_the_whole_batch(core, binary):
    """bb::DifferentiableLutN::SetFrameShard: two layer objects, each holding one half of the frames, with the exchange callback
    played by the host (it copies the per-shard sums out, adds them, and hands the totals back -- what an all-reduce does), against
    one object that sees the whole batch."""
    import torch
    from binarybrain_b200 import abi

    def dev_copy(dst, src, doubles):            # device -> device through the library's own block copy (2 words per double), default stream
        abi.call("bbcu_int32_FrameBufferCopy", dst, src, 1, 0, 0, 2 * doubles, 0, 0, 2 * doubles, 2 * doubles, None)

    def d2h(ptr, count):
        t = torch.empty(count, dtype=torch.float64, device="cuda")
        dev_copy(t.data_ptr(), ptr, count)
        return t.cpu().numpy()

    def h2d(ptr, a):
        t = torch.from_numpy(np.ascontiguousarray(a, np.float64)).cuda()
        dev_copy(ptr, t.data_ptr(), t.numel())
        torch.cuda.synchronize()

    rng = np.random.default_rng(8)
    I, O, F, H = 48, 40, 512, 256
    W = np.clip(rng.normal(0.5, 0.25, (O, 64)), 0, 1).astype(np.float32)
    x = rng.random((F, I), dtype=np.float32)
    dy = rng.random((F, O), dtype=np.float32)

    def make():
        layer = core.DifferentiableLut6_fp32_fp32.create([O], momentum=0.9)
        layer.send_command("binary " + ("true" if binary else "false"))
        layer.set_input_shape([I])
        layer.W().set_numpy(W)
        return layer

    whole = make()
    idx = whole.get_connection()
    y_w = whole.forward(core.FrameBuffer.from_numpy_fp32(x), True).numpy_fp32()
    dx_w = whole.backward(core.FrameBuffer.from_numpy_fp32(dy)).numpy_fp32()
    dW_w = whole.dW().numpy()
    shards = [make(), make()]
    for s_ in shards:
        s_.set_connection(idx)
    xs, dys = [x[:H], x[H:]], [dy[:H], dy[H:]]
    rec = {}
    for phase in ("record", "apply"):                      # forward: first collect every shard's sums, then run with their total
        ys = []
        for k, layer in enumerate(shards):
            if phase == "record":
                layer.set_frame_shard(F, lambda p, n, st, k=k: rec.__setitem__(k, d2h(p, n)))
            else:
                layer.set_frame_shard(F, lambda p, n, st: h2d(p, rec[0] + rec[1]))
            ys.append(layer.forward(core.FrameBuffer.from_numpy_fp32(xs[k]), True).numpy_fp32())
    y = np.concatenate(ys, axis=0)
    assert np.isfinite(shards[0].get_mean().numpy()).all()
    if binary:
        assert (y != y_w).mean() < 1e-3
    else:
        assert np.abs(y - y_w).max() <= 1e-4
    grads = {}
    for phase in ("record", "apply"):                      # backward, the same way (each forward above saved one copy of the input)
        dxs = []
        for k, layer in enumerate(shards):
            layer.dW().fill_zero()
            if phase == "record":
                layer.set_frame_shard(F, lambda p, n, st, k=k: rec.__setitem__(k, d2h(p, n)))
            else:
                layer.set_frame_shard(F, lambda p, n, st: h2d(p, rec[0] + rec[1]))
            dxs.append(layer.backward(core.FrameBuffer.from_numpy_fp32(dys[k])).numpy_fp32())
            grads[k] = layer.dW().numpy().copy()
    dx = np.concatenate(dxs, axis=0)
    assert np.abs(dx - dx_w).max() <= 1e-4 * max(1.0, float(np.abs(dx_w).max()))
    assert np.abs(grads[0] + grads[1] - dW_w).max() <= 1e-4 * max(1.0, float(np.abs(dW_w).max()))
    assert shards[0].get_total_frames() == F


# ------------------------------------------------------------------------------------------------ serialisation (CPU)
def _ser_state():
    from oracle import det_wiring, det_uniform
    return det_wiring(10, 3, 500), det_uniform((3, 64), 501)


def test_layers_load_the_reference_dumps_and_write_them_back(core, golden):
    """DumpObject bytes written by BinaryBrain's own classes (golden) load into the host classes here, every field arrives, and
    dumping again gives the same bytes."""
    idx, W = _ser_state()
    lut = core.DifferentiableLut6_fp32_fp32.create([3])
    data = golden["ser_dl6_fp32"].tobytes()
    lut.load_bytes(data)
    assert lut.get_input_shape() == [10] and lut.get_output_shape() == [3] and lut.get_object_name() == "DifferentiableLut6_fp32_fp32"
    assert np.array_equal(lut.W().numpy(), W) and np.array_equal(lut.get_connection(), idx)
    assert np.allclose(lut.get_mean().numpy(), [0.1, 0.2, 0.3]) and np.allclose(lut.get_var().numpy(), [1.5, 2.5, 3.5])
    assert lut.dump_bytes() == data
    for cls, key in ((core.DifferentiableLut6_bit_fp32, "ser_dl6_bit"), (core.StochasticLut6_fp32_fp32, "ser_sl6_fp32"),
                     (core.BinaryLut6_bit_fp32, "ser_binary_lut6")):
        layer = cls.create([3])
        layer.load_bytes(golden[key].tobytes())
        assert layer.dump_bytes() == golden[key].tobytes(), key
        assert [[layer.get_node_connection_index(n, k) for k in range(6)] for n in range(3)] == idx.tolist()
    bl = core.BinaryLut6_bit_fp32.create([3])
    bl.load_bytes(golden["ser_binary_lut6"].tobytes())
    assert [bl.get_lut_table(0, i) for i in range(3)] == [True, False, False] and bl.get_lut_table(0, 33) and bl.get_lut_table(2, 63)


def test_load_rejects_foreign_and_truncated_data(core, golden):
    data = golden["ser_dl6_fp32"].tobytes()
    lut = core.DifferentiableLut6_fp32_fp32.create([3])
    with pytest.raises(RuntimeError):
        lut.load_bytes(data[:200])                                            # truncated
    with pytest.raises(RuntimeError):
        lut.load_bytes(golden["ser_sl6_fp32"].tobytes())                      # another class's object
    with pytest.raises(RuntimeError):
        lut.load_bytes(b"not an object at all")


def test_reference_loads_what_the_host_classes_dump(core):
    """The other direction, where the reference build is present: a freshly initialised layer here, dumped, is read by BinaryBrain's
    LoadObject and written back unchanged."""
    from oracle import ref
    if not ref.available():
        pytest.skip("oracle/_ref not built")
    for cls, kind in ((core.DifferentiableLut6_fp32_fp32, "dl6_fp32"), (core.StochasticLut6_fp32_fp32, "sl6_fp32"),
                      (core.BinaryLut6_bit_fp32, "binary_lut6")):
        layer = cls.create([5])
        layer.set_input_shape([12])
        mine = np.frombuffer(layer.dump_bytes(), np.uint8)
        assert np.array_equal(ref.layer_redump(kind, mine, 5), mine), kind


def test_forward_node_against_oracle_inference(core):
    """ForwardNode (one node on the host, running statistics) equals the oracle's inference forward on the same six inputs."""
    rng = np.random.default_rng(11)
    I, O = 12, 7
    for binary in (True, False):
        lut = core.DifferentiableLut6_fp32_fp32.create([O], binary=binary)
        lut.set_input_shape([I])
        W = np.clip(rng.normal(0.5, 0.25, (O, 64)), 0, 1).astype(np.float32)
        lut.W().set_numpy(W)
        rm, rv = rng.normal(0.5, 0.05, O).astype(np.float32), rng.uniform(0.01, 0.1, O).astype(np.float32)
        lut.get_mean().set_numpy(rm)
        lut.get_var().set_numpy(rv)
        idx = lut.get_connection()
        x = rng.random((I, 9), dtype=np.float32)
        want = port.dl6_forward_infer(x, idx, W, rm, rv, binary=int(binary))
        for node in range(O):
            for f in range(9):
                got = lut.forward_node(node, [float(x[idx[node, k], f]) for k in range(6)])[0]
                if abs(want["y_pre"][node, f] - 0.5) > 1e-4 or not binary:
                    assert abs(got - want["y"][node, f]) <= 1e-5, (binary, node, f)
