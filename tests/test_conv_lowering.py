"""Convolution lowering around the per-pixel LUT layers of the LUT-CNN: ConvolutionIm2Col, ConvolutionCol2Im, MaxPooling,
fp32 and bit frames, forward and backward.  Golden values come from the reference's own classes (tests/golden/make_golden.py);
these operators only move or select values, so every comparison is exact (fp32 gradients of Im2Col, which add up to
filter_h * filter_w terms, to 1e-6)."""
import numpy as np
import pytest

from oracle import port, pack_bits, det_uniform

PADS, BORDERS = ["valid", "same"], ["constant", "reflect", "reflect_101", "replicate", "wrap"]


def _im2col_inputs(k, case):
    c, h, w, fh, fw, ys, xs, pad, bm, F = (int(v) for v in case)
    x = det_uniform((c * h * w, F), 300 + k)
    oh, ow, _, _ = port.im2col_geometry(h, w, fh, fw, ys, xs, PADS[pad])
    dy = det_uniform((c * fh * fw, F * oh * ow), 320 + k)
    return (c, h, w, fh, fw, ys, xs, PADS[pad], BORDERS[bm], F, oh, ow), x, dy


def _pool_inputs(k, case):
    c, h, w, fh, fw, F = (int(v) for v in case)
    x = np.floor(det_uniform((c * h * w, F), 360 + k) * 4).astype(np.float32) / 4
    oh, ow = (h + fh - 1) // fh, (w + fw - 1) // fw
    dy = det_uniform((c * oh * ow, F), 370 + k)
    xb = pack_bits(det_uniform((c * h * w, F), 380 + k) > 0.7)
    return (c, h, w, fh, fw, F), x, dy, xb


def test_conv_lowering_oracle_against_reference(golden):
    for k, case in enumerate(golden["im2col_cases"]):
        (c, h, w, fh, fw, ys, xs, pad, bm, F, oh, ow), x, dy = _im2col_inputs(k, case)
        assert np.array_equal(port.im2col_forward(x, c, h, w, fh, fw, ys, xs, pad, bm), golden[f"im2col{k}_y"])
        assert np.array_equal(port.im2col_forward(pack_bits(x > 0.5), c, h, w, fh, fw, ys, xs, pad, bm, frames=F), golden[f"im2col{k}_ybits"])
        assert np.array_equal(port.im2col_backward(dy, c, h, w, fh, fw, ys, xs, pad), golden[f"im2col{k}_dx"])
    for k, (c, h, w, Fo) in enumerate(golden["col2im_cases"].tolist()):
        x, dy = det_uniform((c, Fo * h * w), 340 + k), det_uniform((c * h * w, Fo), 350 + k)
        assert np.array_equal(port.col2im_forward(x, c, h, w, Fo), golden[f"col2im{k}_y"])
        assert np.array_equal(port.col2im_forward(pack_bits(x > 0.5), c, h, w, Fo), golden[f"col2im{k}_ybits"])
        assert np.array_equal(port.col2im_backward(dy, c, h, w), golden[f"col2im{k}_dx"])
    for k, case in enumerate(golden["pool_cases"]):
        (c, h, w, fh, fw, F), x, dy, xb = _pool_inputs(k, case)
        y, am = port.maxpool_forward(x, c, h, w, fh, fw)
        assert np.array_equal(y, golden[f"pool{k}_y"])
        assert np.array_equal(port.maxpool_backward(am, dy, c, h, w, fh, fw), golden[f"pool{k}_dx"])
        assert np.array_equal(port.maxpool_forward(xb, c, h, w, fh, fw, frames=F), golden[f"pool{k}_ybits"])
        assert np.array_equal(port.maxpool_backward(xb, dy, c, h, w, fh, fw), golden[f"pool{k}_dxbits"])


def test_im2col_col2im_round_trip_oracle():
    """A 1x1 'same' Im2Col followed by Col2Im is the identity on [c*h*w][frames] (the pair brackets the per-pixel LUT layers)."""
    c, h, w, F = 3, 5, 4, 6
    x = det_uniform((c * h * w, F), 390)
    cols = port.im2col_forward(x, c, h, w, 1, 1, padding="same")
    assert cols.shape == (c, F * h * w)
    assert np.array_equal(port.col2im_forward(cols, c, h, w, F), x)


@pytest.mark.gpu
def test_conv_lowering_gpu_against_golden(golden):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from binarybrain_b200 import ops
    from gpu_util import dev_fp32, dev_bits, host_fp32, host_bits, dev
    for k, case in enumerate(golden["im2col_cases"]):
        (c, h, w, fh, fw, ys, xs, pad, bm, F, oh, ow), x, dy = _im2col_inputs(k, case)
        Fo = F * oh * ow
        y = ops.im2col_forward(dev_fp32(x), F, c, h, w, fh, fw, ys, xs, pad, bm)
        assert np.array_equal(host_fp32(y, Fo), golden[f"im2col{k}_y"]), k
        yb = ops.im2col_forward(dev_bits(pack_bits(x > 0.5), F), F, c, h, w, fh, fw, ys, xs, pad, bm)
        assert np.array_equal(host_bits(yb, Fo), golden[f"im2col{k}_ybits"]), k
        dx = ops.im2col_backward(dev_fp32(dy), F, c, h, w, fh, fw, ys, xs, pad)
        assert np.abs(host_fp32(dx, F) - golden[f"im2col{k}_dx"]).max() <= 1e-6, k
    for k, (c, h, w, Fo) in enumerate(golden["col2im_cases"].tolist()):
        x, dy = det_uniform((c, Fo * h * w), 340 + k), det_uniform((c * h * w, Fo), 350 + k)
        assert np.array_equal(host_fp32(ops.col2im_forward(dev_fp32(x), c, h, w, Fo), Fo), golden[f"col2im{k}_y"]), k
        yb = ops.col2im_forward(dev_bits(pack_bits(x > 0.5), Fo * h * w), c, h, w, Fo)
        assert np.array_equal(host_bits(yb, Fo), golden[f"col2im{k}_ybits"]), k
        assert np.array_equal(host_fp32(ops.col2im_backward(dev_fp32(dy), c, h, w, Fo), Fo * h * w), golden[f"col2im{k}_dx"]), k
    for k, case in enumerate(golden["pool_cases"]):
        (c, h, w, fh, fw, F), x, dy, xb = _pool_inputs(k, case)
        y, am = ops.maxpool_forward(dev_fp32(x), F, c, h, w, fh, fw)
        assert np.array_equal(host_fp32(y, F), golden[f"pool{k}_y"]), k
        dx = ops.maxpool_backward(am, dev_fp32(dy), F, c, h, w, fh, fw)
        assert np.array_equal(host_fp32(dx, F), golden[f"pool{k}_dx"]), k
        xbd = dev_bits(xb, F)
        assert np.array_equal(host_bits(ops.maxpool_forward(xbd, F, c, h, w, fh, fw), F), golden[f"pool{k}_ybits"]), k
        dxb = ops.maxpool_backward(xbd, dev_fp32(dy), F, c, h, w, fh, fw, bit_input=True)
        assert np.array_equal(host_fp32(dxb, F), golden[f"pool{k}_dxbits"]), k


@pytest.mark.gpu
@pytest.mark.parametrize("c,h,w,fh,fw,ys,xs,pad,F", [
    (4, 32, 32, 3, 3, 1, 1, "same", 70),        # several bands of several rows, frame tail
    (2, 40, 24, 5, 5, 1, 1, "same", 33),        # halo of two rows each side
    (3, 33, 31, 3, 3, 2, 2, "same", 40),        # strides, odd sizes
    (2, 30, 20, 3, 2, 2, 1, "valid", 9),
    (1, 3, 600, 3, 3, 1, 1, "same", 8),         # a row too wide for a band in shared memory: the tile kernels
    (2, 28, 28, 3, 3, 1, 1, "same", 70),        # 784 pixels: bit words straddle frames (period of 49 words = 2 frames)
    (2, 28, 28, 5, 5, 1, 1, "valid", 33),
    (1, 27, 27, 3, 3, 1, 1, "same", 40),        # odd pixel count: the period is all 32 frames
    (1, 5, 4, 3, 3, 1, 1, "same", 40),          # tiny image: more windows per bit word than the table holds
    (1, 112, 112, 3, 3, 1, 1, "same", 33),      # 32 bit rows of the image exceed shared memory: the per-tap transpose kernel ...
    (1, 113, 111, 3, 3, 1, 1, "same", 33),      # ... and, for a pixel count that is no multiple of 32, the per-bit gather
])
def test_im2col_bands_and_bit_words_against_oracle(c, h, w, fh, fw, ys, xs, pad, F):
    """Im2Col fp32 forward (every border mode) and backward where the image splits into several bands, and where it does not fit
    a band at all; the forward moves values (exact), the backward adds at most filter_h * filter_w of them in the reference's order.
    Bit frames through the word-wise kernel on the same geometries (exact)."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from binarybrain_b200 import ops
    from gpu_util import dev_fp32, dev_bits, host_fp32, host_bits
    oh, ow, _, _ = port.im2col_geometry(h, w, fh, fw, ys, xs, pad)
    x = det_uniform((c * h * w, F), 410)
    xd = dev_fp32(x)
    xb = pack_bits(x > 0.5)
    xbd = dev_bits(xb, F)
    for border in BORDERS:
        y = ops.im2col_forward(xd, F, c, h, w, fh, fw, ys, xs, pad, border)
        assert np.array_equal(host_fp32(y, F * oh * ow), port.im2col_forward(x, c, h, w, fh, fw, ys, xs, pad, border)), border
        yb = ops.im2col_forward(xbd, F, c, h, w, fh, fw, ys, xs, pad, border)
        assert np.array_equal(host_bits(yb, F * oh * ow), port.im2col_forward(xb, c, h, w, fh, fw, ys, xs, pad, border, frames=F)), border
    dy = det_uniform((c * fh * fw, F * oh * ow), 411)
    dx = ops.im2col_backward(dev_fp32(dy), F, c, h, w, fh, fw, ys, xs, pad)
    assert np.array_equal(host_fp32(dx, F), port.im2col_backward(dy, c, h, w, fh, fw, ys, xs, pad))


@pytest.mark.gpu
@pytest.mark.parametrize("c,h,w,Fo", [(3, 28, 28, 70), (2, 27, 27, 40), (2, 7, 5, 1100), (1, 32, 32, 33)])
def test_col2im_bit_any_pixel_count_against_oracle(c, h, w, Fo):
    """Col2Im on bit frames: the bit vector of an output frame (h * w bits) starts on no particular word boundary."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from binarybrain_b200 import ops
    from gpu_util import dev_bits, host_bits
    xb = pack_bits(det_uniform((c, Fo * h * w), 420) > 0.5)
    yb = ops.col2im_forward(dev_bits(xb, Fo * h * w), c, h, w, Fo)
    assert np.array_equal(host_bits(yb, Fo), port.col2im_forward(xb, c, h, w, Fo))


@pytest.mark.gpu
def test_config3_block_shapes_gpu_against_oracle():
    """The lowering of the LUT-CNN's first conv block at full size: 3x32x32 images, batch 256, 3x3 'same' Im2Col (frames
    x1024, the bit-frame fast path with 32 pixel groups), Col2Im back from 32 channels and 2x2 MaxPooling, fp32 and bit frames."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from binarybrain_b200 import ops
    from gpu_util import dev_fp32, dev_bits, host_fp32, host_bits
    c, h, w, B = 3, 32, 32, 256
    x = det_uniform((c * h * w, B), 400)
    cols = ops.im2col_forward(dev_fp32(x), B, c, h, w, 3, 3, padding="same")
    want = port.im2col_forward(x, c, h, w, 3, 3, padding="same")
    assert np.array_equal(host_fp32(cols, B * h * w), want)
    xb = pack_bits(x > 0.5)
    colsb = ops.im2col_forward(dev_bits(xb, B), B, c, h, w, 3, 3, padding="same")
    assert np.array_equal(host_bits(colsb, B * h * w), port.im2col_forward(xb, c, h, w, 3, 3, padding="same", frames=B))
    dy = det_uniform((c * 9, B * h * w), 401)
    dx = ops.im2col_backward(dev_fp32(dy), B, c, h, w, 3, 3, padding="same")
    assert np.abs(host_fp32(dx, B) - port.im2col_backward(dy, c, h, w, 3, 3, padding="same")).max() <= 2e-6
    # the LUT tree's 32 output channels, still one pixel per frame, go back to images
    ch = 32
    z = det_uniform((ch, B * h * w), 402)
    img = ops.col2im_forward(dev_fp32(z), ch, h, w, B)
    img_w = port.col2im_forward(z, ch, h, w, B)
    assert np.array_equal(host_fp32(img, B), img_w)
    zb = pack_bits(z > 0.5)
    imgb = ops.col2im_forward(dev_bits(zb, B * h * w), ch, h, w, B)
    imgb_w = port.col2im_forward(zb, ch, h, w, B)
    assert np.array_equal(host_bits(imgb, B), imgb_w)
    g = det_uniform((ch * h * w, B), 403)
    assert np.array_equal(host_fp32(ops.col2im_backward(dev_fp32(g), ch, h, w, B), B * h * w), port.col2im_backward(g, ch, h, w))
    # 2x2 pooling to 16x16
    y, am = ops.maxpool_forward(img, B, ch, h, w, 2, 2)
    y_w, am_w = port.maxpool_forward(img_w, ch, h, w, 2, 2)
    assert np.array_equal(host_fp32(y, B), y_w) and np.array_equal(am[:, :B].cpu().numpy(), am_w)
    gp = det_uniform((ch * 16 * 16, B), 404)
    assert np.array_equal(host_fp32(ops.maxpool_backward(am, dev_fp32(gp), B, ch, h, w, 2, 2), B), port.maxpool_backward(am_w, gp, ch, h, w, 2, 2))
    yb = ops.maxpool_forward(imgb, B, ch, h, w, 2, 2)
    assert np.array_equal(host_bits(yb, B), port.maxpool_forward(imgb_w, ch, h, w, 2, 2, frames=B))
    dxb = ops.maxpool_backward(imgb, dev_fp32(gp), B, ch, h, w, 2, 2, bit_input=True)
    assert np.array_equal(host_fp32(dxb, B), port.maxpool_backward(imgb_w, gp, ch, h, w, 2, 2))


@pytest.mark.gpu
def test_conv_lowering_rejects_bad_arguments():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from binarybrain_b200 import abi
    x = torch.zeros((48, 8), device="cuda")
    y = torch.zeros((27, 8), device="cuda")
    p = lambda t: t.data_ptr()
    # output frame stride smaller than frames * oh * ow
    assert abi.lib().bbcu_fp32_Im2Col_Forward(p(x), p(y), 1, 1, 1, 1, 8, 8, 4, 4, 3, 4, 4, 8, 3, 3, 2, 0.0, None) == -3
    assert abi.lib().bbcu_fp32_Im2Col_Forward(None, p(y), 1, 1, 1, 1, 8, 8, 4, 4, 3, 4, 4, 128, 3, 3, 2, 0.0, None) == -1
    # pooling output size must be the rounded-up quotient
    assert abi.lib().bbcu_fp32_MaxPooling_Forward(p(x), p(y), None, 2, 2, 4, 4, 3, 2, 3, 8, 8, None) == -2


def _tables(shape, seed):
    """Well-spread tables (std ~0.25): batch norm then amplifies rounding differences by ~10 per layer instead of ~100."""
    return np.clip(0.5 + 0.25 * (det_uniform(shape, seed) - 0.5) * 3.46, 0, 1).astype(np.float32)


@pytest.mark.gpu
def test_convolution2d_layer_gpu_against_oracle():
    """bb::Convolution2d of two DifferentiableLut6 layers (27 -> 48 -> 16 per pixel) on 3x8x8 images, then 2x2 MaxPooling:
    forward and backward through the host-side classes against the same composition of oracle operators."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from binarybrain_b200.conv import Convolution2d, MaxPooling, Sequential
    from binarybrain_b200.dist import ShardedDifferentiableLut6
    from oracle import det_wiring
    from gpu_util import dev, dev_fp32, host_fp32, err
    c, h, w, B = 3, 8, 8, 6
    P = h * w
    widths = [27, 48, 16]
    idx = [det_wiring(widths[l], widths[l + 1], 410 + l) for l in range(2)]
    W = [_tables((widths[l + 1], 64), 420 + l) for l in range(2)]
    x = det_uniform((c * h * w, B), 430)
    dy = det_uniform((16 * 4 * 4, B), 431)
    # oracle composition
    cols = port.im2col_forward(x, c, h, w, 3, 3, padding="same")
    f1 = port.dl6_forward_train(cols, idx[0], W[0], np.zeros(48), np.ones(48), binary=False)
    f2 = port.dl6_forward_train(f1["y"], idx[1], W[1], np.zeros(16), np.ones(16), binary=False)
    img = port.col2im_forward(f2["y"], 16, h, w, B)
    y_w, am = port.maxpool_forward(img, 16, h, w, 2, 2)
    g = port.maxpool_backward(am, dy, 16, h, w, 2, 2)
    g = port.col2im_backward(g, 16, h, w)
    g1, dW1 = port.dl6_backward(f1["y"], g, idx[1], W[1], f2["mean"], f2["rstd"], 48, binary=False)
    g0, dW0 = port.dl6_backward(cols, g1, idx[0], W[0], f1["mean"], f1["rstd"], 27, binary=False)
    dx_w = port.im2col_backward(g0, c, h, w, 3, 3, padding="same")
    # device
    luts = [ShardedDifferentiableLut6(dev(idx[l]), dev(W[l]), widths[l]) for l in range(2)]
    net = Sequential([Convolution2d(luts, c, h, w, 3, 3, padding="same"), MaxPooling(16, h, w, 2, 2)])
    y = net.forward(dev_fp32(x), B)
    amp = max(1.0, 0.3 * float(f1["rstd"].max())) * max(1.0, 0.3 * float(f2["rstd"].max()))       # batch-norm gain of the two layers
    assert err(host_fp32(y, B), y_w) <= 1e-5 * amp
    dx = net.backward(dev_fp32(dy))
    assert err(host_fp32(dx, B), dx_w) <= 1e-4 * amp
    assert err(luts[1].dW.cpu().numpy(), dW1) <= 1e-4 * amp and err(luts[0].dW.cpu().numpy(), dW0) <= 1e-4 * amp
