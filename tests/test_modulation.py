"""Binary modulation around a LUT network: RealToBinary (frame modulation 7, seeded thresholds),
two StochasticLut6 layers on the modulated frames, BinaryToReal integration.  Golden values from the reference's own
RealToBinary / BinaryToReal (tests/golden/make_golden.py); bit outputs are compared bit for bit."""
import numpy as np
import pytest

from oracle import port, pack_bits, unpack_bits, det_uniform, det_wiring


def test_modulation_oracle_against_reference(golden):
    x = golden["r2b_x"]
    for ps in (1, 4):
        assert (port.real_to_binary(x, 7, 2, point_size=ps) == golden[f"r2b_p{ps}_det"]).all()
        assert (port.real_to_binary(x, 7, 2, thresholds=golden[f"r2b_p{ps}_th"], point_size=ps) == golden[f"r2b_p{ps}_seeded"]).all()
    assert np.array_equal(port.binary_to_real(golden["b2r_x"], 10, 8, 7), golden["b2r_y"])
    assert np.abs(port.binary_to_real_backward(golden["b2r_dy"], 60, 7) - golden["b2r_dx"]).max() <= 1e-7


@pytest.mark.gpu
def test_modulation_gpu_bit_exact(golden):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from binarybrain_b200 import ops
    from gpu_util import dev, dev_fp32, dev_bits, host_bits, host_fp32
    x = golden["r2b_x"]
    F = x.shape[1]
    for ps in (1, 4):
        y = ops.real_to_binary(dev_fp32(x), F, frame_mod=7, depth_mod=2, point_size=ps)
        assert (host_bits(y, F * 7) == golden[f"r2b_p{ps}_det"]).all()
        th = golden[f"r2b_p{ps}_th"]
        y = ops.real_to_binary(dev_fp32(x), F, frame_mod=7, depth_mod=2, thresholds=dev_fp32(th), point_size=ps)
        assert (host_bits(y, F * 7) == golden[f"r2b_p{ps}_seeded"]).all()
    xb = golden["b2r_x"]
    y = ops.binary_to_real(dev_bits(xb, 56), 60, 10, 8, frame_mux=7)
    assert np.array_equal(host_fp32(y, 8), golden["b2r_y"])
    dx = ops.binary_to_real_backward(dev_fp32(golden["b2r_dy"]), 60, 8, frame_mux=7)
    assert np.abs(host_fp32(dx, 56) - golden["b2r_dx"]).max() <= 1e-7


@pytest.mark.gpu
def test_config2_chain_gpu_against_oracle():
    """3x32x32 images, batch 256, RealToBinary x7 with seeded thresholds -> StochasticLut6<bit> 4096 -> StochasticLut6<fp32> 1020
    -> BinaryToReal to 10 outputs; forward and backward, every stage against the oracle (bit stages bit for bit)."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from binarybrain_b200 import ops
    from gpu_util import dev, dev_fp32, host_bits, host_fp32, err
    I, B, M = 3 * 32 * 32, 256, 7
    F = B * M
    x = det_uniform((I, B), 201)
    th = det_uniform((I, F), 202)
    idx1, idx2 = det_wiring(I, 4096, 203), det_wiring(4096, 1020, 204)
    W1 = (0.5 + 0.01 * (det_uniform((4096, 64), 205) - 0.5) * 3.46).astype(np.float32)
    W2 = (0.5 + 0.01 * (det_uniform((1020, 64), 206) - 0.5) * 3.46).astype(np.float32)
    # oracle
    xb = port.real_to_binary(x, M, 1, thresholds=th)
    h1 = port.sl6_forward(xb, idx1, W1, frames=F)
    h2 = port.sl6_forward(h1, idx2, W2)
    # device
    xbd = ops.real_to_binary(dev_fp32(x), B, frame_mod=M, thresholds=dev_fp32(th))
    assert (host_bits(xbd, F) == xb).all()
    h1d = ops.stochastic_lut6_forward(xbd, dev(idx1), dev(W1), F)
    assert err(host_fp32(h1d, F), h1) <= 1e-5
    h2d = ops.stochastic_lut6_forward(h1d, dev(idx2), dev(W2), F)
    assert err(host_fp32(h2d, F), h2) <= 1e-5
    yd = ops.binary_to_real(h2d, 1020, 10, B, frame_mux=M)                     # fp32 frames: counts values > 0
    want = np.zeros((10, B), np.float32)
    for n in range(1020):
        want[n % 10] += (h2[n].reshape(B, M) > 0).sum(1)
    want /= (102 * M)
    assert np.abs(host_fp32(yd, B) - want).max() <= 1e-6
    # backward through BinaryToReal and both LUT layers
    dy = det_uniform((10, B), 207)
    g = ops.binary_to_real_backward(dev_fp32(dy), 1020, B, frame_mux=M)
    g_w = port.binary_to_real_backward(dy, 1020, M)
    assert np.abs(host_fp32(g, F) - g_w).max() <= 1e-7
    dW2, dW1 = torch.zeros((1020, 64), device="cuda"), torch.zeros((4096, 64), device="cuda")
    g2 = ops.stochastic_lut6_backward(h1d, g, dev(idx2), dev(W2), dW2, 4096, F)
    g2_w, dW2_w = port.sl6_backward(h1, g_w, idx2, W2, 4096)
    assert err(host_fp32(g2, F), g2_w) <= 1e-5 and err(dW2.cpu().numpy(), dW2_w) <= 1e-5
    g1 = ops.stochastic_lut6_backward(xbd, g2, dev(idx1), dev(W1), dW1, I, F)
    g1_w, dW1_w = port.sl6_backward(xb, g2_w, idx1, W1, I)
    assert err(host_fp32(g1, F), g1_w) <= 1e-5 and err(dW1.cpu().numpy(), dW1_w) <= 1e-5
