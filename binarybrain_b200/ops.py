"""The bbcu_* operators on torch CUDA tensors.

torch only provides device memory and the current stream here; every operator is one call through
the C ABI (binarybrain_b200.abi).  Frame buffers are 2-D tensors ``[nodes, frame_stride]``: fp32
buffers hold one float per frame, bit buffers (dtype int32) 32 frames per element, LSB first -- the
FrameBuffer layout of the reference (include/bb/FrameBuffer.h:28-46).  ``frames`` is the number of
valid frames; the stride is taken from the tensor.
"""
import torch

from . import abi

BIAS = 0.25   # unbinarize_bias of the reference's layers (include/bb/DifferentiableLutN.h:63)


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _p(t):
    return 0 if t is None else t.data_ptr()


def _chk(t, dtype, name):
    if not t.is_cuda:
        raise ValueError(f"{name}: expected a CUDA tensor (the bbcu_* operators have no CPU path)")
    if t.dtype != dtype:
        raise ValueError(f"{name}: expected dtype {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name}: expected a contiguous tensor")
    return t


def fp32_stride(frames):
    """Row stride in floats: rows padded to 32 bytes (include/bb/FrameBuffer.h:414-417)."""
    return (frames + 7) // 8 * 8


def bit_stride(frames):
    """Row stride in 32-bit words: rows padded to 256 bits."""
    return (frames + 255) // 256 * 8


# ------------------------------------------------------------------------------------------ StochasticLut6
def stochastic_lut6_forward(x, idx, W, frames, y=None, binary=False, lut_binarize=False, bias=BIAS, bit_output=False):
    """fp32 or bit-packed x -> fp32 y (clip to [0,1]) or, with bit_output (bit x only), bit-packed y = lut > 0.5."""
    O = idx.shape[0]
    _chk(idx, torch.int32, "idx"); _chk(W, torch.float32, "W")
    if x.dtype == torch.float32:
        _chk(x, torch.float32, "x")
        if y is None:
            y = torch.empty((O, x.shape[1]), dtype=torch.float32, device=x.device)
        abi.call("bbcu_fp32_StochasticLut6_Forward", _p(x), _p(y), _p(idx), _p(W), O, frames, x.shape[1], int(binary), int(lut_binarize),
                 bias, _stream())
    elif bit_output:
        _chk(x, torch.int32, "x")
        if y is None:
            y = torch.zeros((O, x.shape[1]), dtype=torch.int32, device=x.device)
        abi.call("bbcu_bit_bit_fp32_StochasticLut6_Forward", _p(x), _p(y), _p(idx), _p(W), O, frames, x.shape[1], int(lut_binarize), bias,
                 _stream())
    else:
        _chk(x, torch.int32, "x")
        if y is None:
            y = torch.empty((O, fp32_stride(frames)), dtype=torch.float32, device=x.device)
        abi.call("bbcu_bit_fp32_StochasticLut6_Forward", _p(x), _p(y), _p(idx), _p(W), O, frames, y.shape[1], x.shape[1], int(lut_binarize),
                 bias, _stream())
    return y


def stochastic_lut6_backward(x, dy, idx, W, dW, n_in, frames, dx=None, binary=False, lut_binarize=False, bias=BIAS, dx_tmp=None):
    """dx is overwritten, dW accumulated into.  dx_tmp: optional fp32 scratch [6 * nodes, tmp_stride] as the reference's callers pass it."""
    O = idx.shape[0]
    _chk(dy, torch.float32, "dy"); _chk(dW, torch.float32, "dW")
    if dx is None:
        dx = torch.empty((n_in, dy.shape[1]), dtype=torch.float32, device=dy.device)
    if x.dtype == torch.float32:
        assert x.shape[1] == dy.shape[1], "x, dy and dx share one frame stride"
        abi.call("bbcu_fp32_StochasticLut6_Backward", _p(x), _p(dy), _p(dx), _p(dx_tmp), _p(idx), 0, _p(W), _p(dW), 0, n_in, O, frames, dy.shape[1],
                 0 if dx_tmp is None else dx_tmp.shape[1], 0 if dx_tmp is None else dx_tmp.shape[1], int(binary), int(lut_binarize), bias, _stream())
    else:
        _chk(x, torch.int32, "x")
        abi.call("bbcu_bit_fp32_StochasticLut6_Backward", _p(x), _p(dy), _p(dx), 0, _p(idx), 0, _p(W), _p(dW), 0, n_in, O, frames,
                 dy.shape[1], x.shape[1], 0, 0, int(lut_binarize), bias, _stream())
    return dx


# ------------------------------------------------------------------------------------------ DifferentiableLut6
def differentiable_lut6_forward_training(x, idx, W, running_mean, running_var, frames, y=None, gamma=0.3, beta=0.5, momentum=0.9,
                                         bias=BIAS, lut_binarize=False, binary=True):
    """Returns (y, mean, rstd); running_mean / running_var are updated in place.  Bit x gives bit y."""
    O = idx.shape[0]
    dev = x.device
    mean = torch.empty(O, dtype=torch.float32, device=dev)
    rstd = torch.empty(O, dtype=torch.float32, device=dev)
    if x.dtype == torch.float32:
        if y is None:
            y = torch.empty((O, x.shape[1]), dtype=torch.float32, device=dev)
        abi.call("bbcu_fp32_DifferentiableLut6_ForwardTraining", _p(x), _p(y), _p(idx), _p(W), _p(mean), _p(rstd), _p(running_mean),
                 _p(running_var), gamma, beta, momentum, bias, O, frames, x.shape[1], int(lut_binarize), int(binary), _stream())
    else:
        _chk(x, torch.int32, "x")
        if y is None:
            y = torch.zeros((O, x.shape[1]), dtype=torch.int32, device=dev)
        abi.call("bbcu_bit_fp32_DifferentiableLut6_ForwardTraining", _p(x), _p(y), _p(idx), _p(W), _p(mean), _p(rstd), _p(running_mean),
                 _p(running_var), gamma, beta, momentum, bias, O, frames, x.shape[1], int(lut_binarize), _stream())
    return y, mean, rstd


def differentiable_lut6_forward_inference(x, idx, W, running_mean, running_var, frames, y=None, gamma=0.3, beta=0.5, bias=BIAS,
                                          lut_binarize=False, binary=True):
    O = idx.shape[0]
    if x.dtype == torch.float32:
        if y is None:
            y = torch.empty((O, x.shape[1]), dtype=torch.float32, device=x.device)
        abi.call("bbcu_fp32_DifferentiableLut6_ForwardInference", _p(x), _p(y), _p(idx), _p(W), _p(running_mean), _p(running_var), gamma, beta,
                 bias, O, frames, x.shape[1], int(lut_binarize), int(binary), _stream())
    else:
        if y is None:
            y = torch.zeros((O, x.shape[1]), dtype=torch.int32, device=x.device)
        abi.call("bbcu_bit_fp32_DifferentiableLut6_ForwardInference", _p(x), _p(y), _p(idx), _p(W), _p(running_mean), _p(running_var), gamma,
                 beta, bias, O, frames, x.shape[1], int(lut_binarize), _stream())
    return y


def differentiable_lut6_backward(x, dy, idx, W, dW, mean, rstd, n_in, frames, dx=None, gamma=0.3, beta=0.5, bias=BIAS, lut_binarize=False,
                                 binary=True, dx_tmp=None):
    O = idx.shape[0]
    dev = dy.device
    if dx is None:
        dx = torch.empty((n_in, dy.shape[1]), dtype=torch.float32, device=dev)
    dmean = torch.empty(O, dtype=torch.float32, device=dev)
    dvar = torch.empty(O, dtype=torch.float32, device=dev)
    if x.dtype == torch.float32:
        assert x.shape[1] == dy.shape[1]
        abi.call("bbcu_fp32_DifferentiableLut6_Backward", _p(x), _p(dy), _p(dx), _p(dx_tmp), _p(idx), 0, _p(W), _p(dW), _p(mean), _p(rstd), _p(dmean),
                 _p(dvar), gamma, beta, bias, 0, n_in, O, frames, dy.shape[1], 0 if dx_tmp is None else dx_tmp.shape[1],
                 0 if dx_tmp is None else dx_tmp.shape[1], int(lut_binarize), int(binary), _stream())
    else:
        abi.call("bbcu_bit_fp32_DifferentiableLut6_Backward", _p(x), _p(dy), _p(dx), 0, _p(idx), 0, _p(W), _p(dW), _p(mean), _p(rstd),
                 _p(dmean), _p(dvar), gamma, beta, bias, 0, n_in, O, frames, dy.shape[1], x.shape[1], 0, 0, int(lut_binarize), _stream())
    return dx


# ------------------------------------------------------------------------------------------ StochasticBatchNormalization
def stochastic_bn_forward_training(x, running_mean, running_var, frames, gamma=0.2, beta=0.5, momentum=0.9):
    O = x.shape[0]
    y = torch.empty_like(x)
    mean = torch.empty(O, dtype=torch.float32, device=x.device)
    rstd = torch.empty(O, dtype=torch.float32, device=x.device)
    abi.call("bbcu_fp32_StochasticBatchNormalization_ForwardTraining", _p(x), _p(y), _p(mean), _p(rstd), _p(running_mean), _p(running_var),
             gamma, beta, momentum, O, frames, x.shape[1], _stream())
    return y, mean, rstd


def stochastic_bn_reforward(x, mean, rstd, frames, gamma=0.2, beta=0.5):
    y = torch.empty_like(x)
    abi.call("bbcu_fp32_StochasticBatchNormalization_ReForward", _p(x), _p(y), _p(mean), _p(rstd), gamma, beta, x.shape[0], frames, x.shape[1],
             _stream())
    return y


def stochastic_bn_forward_inference(x, running_mean, running_var, frames, gamma=0.2, beta=0.5):
    y = torch.empty_like(x)
    abi.call("bbcu_fp32_StochasticBatchNormalization_ForwardInference", _p(x), _p(y), _p(running_mean), _p(running_var), gamma, beta,
             x.shape[0], frames, x.shape[1], _stream())
    return y


def stochastic_bn_backward(x, dy, mean, rstd, frames, gamma=0.2):
    dx = torch.empty_like(dy)
    abi.call("bbcu_fp32_StochasticBatchNormalization_Backward", _p(x), _p(dy), _p(dx), _p(mean), _p(rstd), gamma, 1.0 / frames, dy.shape[0],
             frames, dy.shape[1], x.shape[1], _stream())
    return dx


# ------------------------------------------------------------------------------------------ BinaryLut6
def binary_lut6_forward(x, idx, table, frames, y=None, lop3_immediate=False):
    """Bit-packed inference forward; ``table`` is [nodes, 2] int32 (64-entry truth table per node).
    lop3_immediate: evaluate through the truth-table-immediate kernel (same results; aligned rows only)."""
    _chk(x, torch.int32, "x"); _chk(idx, torch.int32, "idx"); _chk(table, torch.int32, "table")
    O = idx.shape[0]
    if y is None:
        y = torch.empty((O, x.shape[1]), dtype=torch.int32, device=x.device)
    name = "bbcu_bit_BinaryLut6_Forward_Lop3Immediate" if lop3_immediate else "bbcu_bit_BinaryLut6_Forward"
    abi.call(name, _p(x), _p(y), _p(idx), _p(table), O, frames, x.shape[1], _stream())
    return y


def binary_lut6_forward_host(x, idx, table, frames, y=None):
    """BinaryLut6 forward on HOST tensors (int32, ideally pinned): chunked upload / kernel / download overlapped inside the library."""
    for t, n in ((x, "x"), (idx, "idx"), (table, "table")):
        if t.is_cuda or t.dtype != torch.int32 or not t.is_contiguous():
            raise ValueError(f"{n}: expected a contiguous int32 host tensor")
    O = idx.shape[0]
    if y is None:
        y = torch.empty((O, x.shape[1]), dtype=torch.int32).pin_memory()
    abi.call("bbcu_host_bit_BinaryLut6_Forward", _p(x), _p(y), _p(idx), _p(table), x.shape[0], O, frames, x.shape[1])
    return y


# ------------------------------------------------------------------------------------------ per-step neighbours
def clamp_(t, lo=0.0, hi=1.0):
    abi.call("bbcu_fp32_Vector_clamp", _p(t), _p(t), lo, hi, t.numel(), _stream())
    return t


def softmax_cross_entropy(y, t, frames, pix_size=1):
    """bb::LossSoftmaxCrossEntropy::CalculateLoss: returns (dy, loss) with loss = -sum(loss_buf) / t_sum (the mean over frames)."""
    dy = torch.empty_like(y)
    loss_buf = torch.zeros(frames, dtype=torch.float64, device=y.device)
    t_sum = float(t[:, :frames].sum().item())
    abi.call("bbcu_fp32_LossSoftmaxCrossEntropy", _p(y), _p(t), _p(dy), _p(loss_buf), t_sum, pix_size, y.shape[0] // pix_size, frames, y.shape[1],
             _stream())
    return dy, (-loss_buf.sum() / t_sum)


def mean_squared_error(y, t, frames, batch_size=None, loss_buf=None, dy=None):
    """bb::LossMeanSquaredError::CalculateLoss (mean reduction): returns (dy, loss_buf); loss = loss_buf.sum() / frames seen."""
    nodes = y.shape[0]
    batch_size = frames if batch_size is None else batch_size
    if dy is None:
        dy = torch.empty_like(y)
    if loss_buf is None:
        loss_buf = torch.zeros(1024, dtype=torch.float64, device=y.device)
    abi.call("bbcu_fp32_LossMeanSquaredError", _p(y), _p(t), _p(dy), _p(loss_buf), loss_buf.numel(), nodes, frames, y.shape[1],
             2.0 / (nodes * batch_size), 1.0 / nodes, _stream())
    return dy, loss_buf


def reduce_forward(x, out_nodes, frames, y=None):
    """bb::Reduce forward: y[o] = mean_i x[out_nodes * i + o]."""
    if y is None:
        y = torch.empty((out_nodes, x.shape[1]), dtype=torch.float32, device=x.device)
    abi.call("bbcu_fp32_Reduce_Forward", _p(x), _p(y), x.shape[0], out_nodes, frames, x.shape[1], y.shape[1], _stream())
    return y


def reduce_backward(dy, in_nodes, frames, dx=None):
    if dx is None:
        dx = torch.empty((in_nodes, dy.shape[1]), dtype=torch.float32, device=dy.device)
    abi.call("bbcu_fp32_Reduce_Backward", _p(dy), _p(dx), in_nodes, dy.shape[0], frames, dy.shape[1], dx.shape[1], _stream())
    return dx


def real_to_binary(x, frames, frame_mod=1, depth_mod=1, lo=0.0, hi=1.0, thresholds=None, point_size=None):
    """bb::RealToBinary forward to bit frames: [nodes, frames] fp32 -> [nodes * depth_mod, frames * frame_mod] bits.
    thresholds: optional fp32 [nodes, >= frames * frame_mod] (what a seeded value generator supplies in the reference)."""
    nodes = x.shape[0]
    point_size = nodes if point_size is None else point_size
    out_frames = frames * frame_mod
    y = torch.zeros((nodes * depth_mod, bit_stride(out_frames)), dtype=torch.int32, device=x.device)
    abi.call("bbcu_bit_fp32_RealToBinary_Forward", _p(x), _p(y), _p(thresholds), 0 if thresholds is None else thresholds.shape[1], depth_mod,
             frame_mod, lo, hi, point_size, nodes // point_size, frames, x.shape[1], y.shape[1], _stream())
    return y


def binary_to_real(x, x_nodes, y_nodes, y_frames, frame_mux=1):
    """bb::BinaryToReal forward: bit (int32) or fp32 frames -> fp32 [y_nodes, y_frames], averaging node_mux x frame_mux inputs."""
    y = torch.empty((y_nodes, fp32_stride(y_frames)), dtype=torch.float32, device=x.device)
    name = "bbcu_bit_fp32_BinaryToReal_Forward" if x.dtype == torch.int32 else "bbcu_fp32_BinaryToReal_Forward"
    abi.call(name, _p(x), _p(y), x_nodes // y_nodes, frame_mux, y_nodes, x.shape[1], y_frames, y.shape[1], _stream())
    return y


def binary_to_real_backward(dy, x_nodes, y_frames, frame_mux=1):
    y_nodes = dy.shape[0]
    dx = torch.empty((x_nodes, fp32_stride(y_frames * frame_mux)), dtype=torch.float32, device=dy.device)
    abi.call("bbcu_fp32_BinaryToReal_Backward", _p(dy), _p(dx), x_nodes // y_nodes, frame_mux, y_nodes, dx.shape[1], y_frames, dy.shape[1],
             _stream())
    return dx


BORDER_MODES = {"constant": 0, "reflect": 1, "reflect_101": 2, "replicate": 3, "wrap": 4}


def im2col_geometry(h, w, fh, fw, y_stride=1, x_stride=1, padding="valid"):
    """(out_h, out_w, y_offset, x_offset) of bb::ConvolutionIm2Col (include/bb/ConvolutionIm2Col.h:200-215)."""
    if padding == "valid":
        return ((h - fh + 1) + (y_stride - 1)) // y_stride, ((w - fw + 1) + (x_stride - 1)) // x_stride, 0, 0
    if padding == "same":
        return (h + y_stride - 1) // y_stride, (w + x_stride - 1) // x_stride, (fh - 1) // 2, (fw - 1) // 2
    raise ValueError(f"unknown padding {padding!r}")


def im2col_forward(x, frames, c, h, w, fh, fw, y_stride=1, x_stride=1, padding="valid", border_mode="reflect_101", border_value=0.0, y=None):
    """bb::ConvolutionIm2Col forward: [c*h*w, frames] (fp32, or int32 bit words) -> [c*fh*fw, frames*oh*ow].  `y`: an output buffer of
    that shape to write into (every word up to the last frame is written; nothing needs clearing)."""
    oh, ow, yo, xo = im2col_geometry(h, w, fh, fw, y_stride, x_stride, padding)
    of = frames * oh * ow
    if y is not None:
        abi.call("bbcu_bit_Im2Col_Forward" if x.dtype == torch.int32 else "bbcu_fp32_Im2Col_Forward", _p(x), _p(y), x_stride, y_stride, xo, yo, frames,
                 x.shape[1], w, h, c, ow, oh, y.shape[1], fw, fh, BORDER_MODES[border_mode], *(() if x.dtype == torch.int32 else (border_value,)), _stream())
        return y
    if x.dtype == torch.int32:
        y = torch.zeros((c * fh * fw, bit_stride(of)), dtype=torch.int32, device=x.device)
        abi.call("bbcu_bit_Im2Col_Forward", _p(x), _p(y), x_stride, y_stride, xo, yo, frames, x.shape[1], w, h, c, ow, oh, y.shape[1], fw, fh,
                 BORDER_MODES[border_mode], _stream())
    else:
        y = torch.empty((c * fh * fw, fp32_stride(of)), dtype=torch.float32, device=x.device)
        abi.call("bbcu_fp32_Im2Col_Forward", _p(x), _p(y), x_stride, y_stride, xo, yo, frames, x.shape[1], w, h, c, ow, oh, y.shape[1], fw, fh,
                 BORDER_MODES[border_mode], border_value, _stream())
    return y


def im2col_backward(dy, frames, c, h, w, fh, fw, y_stride=1, x_stride=1, padding="valid"):
    oh, ow, yo, xo = im2col_geometry(h, w, fh, fw, y_stride, x_stride, padding)
    dx = torch.empty((c * h * w, fp32_stride(frames)), dtype=torch.float32, device=dy.device)
    abi.call("bbcu_fp32_Im2Col_Backward", _p(dy), _p(dx), x_stride, y_stride, xo, yo, frames, dx.shape[1], w, h, c, ow, oh, dy.shape[1], fw, fh,
             _stream())
    return dx


def col2im_forward(x, c, h, w, out_frames):
    """bb::ConvolutionCol2Im forward: [c, out_frames*h*w] -> [c*h*w, out_frames] (fp32, or int32 bit words)."""
    if x.dtype == torch.int32:
        y = torch.zeros((c * h * w, bit_stride(out_frames)), dtype=torch.int32, device=x.device)
        abi.call("bbcu_bit_Col2Im_Forward", _p(x), _p(y), w, h, c, x.shape[1], out_frames, y.shape[1], _stream())
    else:
        y = torch.empty((c * h * w, fp32_stride(out_frames)), dtype=torch.float32, device=x.device)
        abi.call("bbcu_fp32_Col2Im_Forward", _p(x), _p(y), w, h, c, x.shape[1], out_frames, y.shape[1], _stream())
    return y


def col2im_backward(dy, c, h, w, out_frames):
    dx = torch.empty((c, fp32_stride(out_frames * h * w)), dtype=torch.float32, device=dy.device)
    abi.call("bbcu_fp32_Col2Im_Backward", _p(dy), _p(dx), w, h, c, dx.shape[1], out_frames, dy.shape[1], _stream())
    return dx


def maxpool_forward(x, frames, c, h, w, fh, fw, want_argmax=True):
    """bb::MaxPooling forward.  fp32: returns (y, argmax or None); int32 bit words: returns y."""
    oh, ow = (h + fh - 1) // fh, (w + fw - 1) // fw
    if x.dtype == torch.int32:
        y = torch.zeros((c * oh * ow, x.shape[1]), dtype=torch.int32, device=x.device)
        abi.call("bbcu_bit_MaxPooling_Forward", _p(x), _p(y), fh, fw, w, h, ow, oh, c, frames, x.shape[1], _stream())
        return y
    y = torch.empty((c * oh * ow, x.shape[1]), dtype=torch.float32, device=x.device)
    am = torch.empty((c * oh * ow, x.shape[1]), dtype=torch.int32, device=x.device) if want_argmax else None
    abi.call("bbcu_fp32_MaxPooling_Forward", _p(x), _p(y), _p(am), fh, fw, w, h, ow, oh, c, frames, x.shape[1], _stream())
    return y, am


def maxpool_backward(sel, dy, frames, c, h, w, fh, fw, bit_input=False):
    """sel: the forward's argmax (fp32 layer) or, with bit_input=True, the forward's bit-packed input."""
    oh, ow = (h + fh - 1) // fh, (w + fw - 1) // fw
    dx = torch.empty((c * h * w, dy.shape[1]), dtype=torch.float32, device=dy.device)
    if bit_input:
        abi.call("bbcu_bit_fp32_MaxPooling_Backward", _p(sel), _p(dy), _p(dx), fh, fw, w, h, ow, oh, c, frames, sel.shape[1], dy.shape[1], _stream())
    else:
        abi.call("bbcu_fp32_MaxPooling_Backward", _p(sel), _p(dy), _p(dx), fh, fw, w, h, ow, oh, c, frames, dy.shape[1], _stream())
    return dx


class Adam:
    """bb::OptimizerAdam over a list of (param, grad) CUDA tensors (include/bb/OptimizerAdam.h:142-184)."""

    def __init__(self, params, grads, lr=0.001, beta1=0.9, beta2=0.999):
        self.params, self.grads = list(params), list(grads)
        self.m = [torch.zeros_like(p) for p in self.params]
        self.v = [torch.zeros_like(p) for p in self.params]
        dev = self.params[0].device
        self._sizes = torch.tensor([p.numel() for p in self.params], dtype=torch.int32, device=dev)
        mk = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=dev)
        self._tabs = [mk(self.params), mk(self.grads), mk(self.m), mk(self.v)]
        self.lr, self.beta1, self.beta2 = lr, beta1, beta2
        self.b1, self.b2 = beta1, beta2

    def step(self):
        lr_t = self.lr * (1.0 - self.b2) ** 0.5 / (1.0 - self.b1)
        abi.call("bbcu_fp32_OptimizerAdam", len(self.params), _p(self._sizes), *[_p(t) for t in self._tabs], lr_t, self.beta1, self.beta2,
                 _stream())
        self.b1 *= self.beta1
        self.b2 *= self.beta2

    def zero_grad(self):
        for g in self.grads:
            g.zero_()

    def update(self):          # Optimizer::Update = Step + ZeroGrad (include/bb/Optimizer.h:29-33)
        self.step()
        self.zero_grad()


# ------------------------------------------------------------------------------------------ frame-sharded halves
def dl6_forward_stats(x, idx, W, frames, y, sums, bias=BIAS, lut_binarize=False, binary=True):
    """Pass 1 of the training forward on this rank's frames: raw LUT values into y, per-node (sum y, sum y^2) into sums [O,2] fp64."""
    abi.call("bbcu_fp32_DifferentiableLut6_ForwardStats", _p(x), _p(y), _p(idx), _p(W), _p(sums), bias, idx.shape[0], frames, x.shape[1],
             int(lut_binarize), int(binary), _stream())


def dl6_forward_normalize(y, sums, mean, rstd, running_mean, running_var, frames, total_frames, gamma=0.3, beta=0.5, momentum=0.9, binary=True):
    """Pass 2: statistics from the (all-reduced) sums over total_frames, then normalise y in place."""
    abi.call("bbcu_fp32_DifferentiableLut6_ForwardNormalize", _p(y), _p(sums), _p(mean), _p(rstd), _p(running_mean), _p(running_var), gamma, beta,
             momentum, y.shape[0], frames, y.shape[1], int(total_frames), int(binary), _stream())


def dl6_backward_stats(x, dy, idx, W, mean, rstd, frames, sums, gamma=0.3, beta=0.5, bias=BIAS, lut_binarize=False, binary=True):
    abi.call("bbcu_fp32_DifferentiableLut6_BackwardStats", _p(x), _p(dy), _p(idx), _p(W), _p(mean), _p(rstd), _p(sums), gamma, beta, bias,
             idx.shape[0], frames, x.shape[1], int(lut_binarize), int(binary), _stream())


def dl6_backward_stats_from_output(y, dy, rstd, frames, sums, gamma=0.3, beta=0.5):
    """The sums of dl6_backward_stats from the layer's training output y (non-binary mode): no second LUT evaluation."""
    abi.call("bbcu_fp32_DifferentiableLut6_BackwardStatsFromOutput", _p(y), _p(dy), _p(rstd), _p(sums), gamma, beta, y.shape[0], frames,
             y.shape[1], 0, _stream())


def dl6_backward_apply(x, dy, dx, idx, W, dW, mean, rstd, sums, n_in, frames, total_frames, gamma=0.3, beta=0.5, bias=BIAS, lut_binarize=False,
                       binary=True):
    O = idx.shape[0]
    dmean = torch.empty(O, dtype=torch.float32, device=dy.device)
    dvar = torch.empty(O, dtype=torch.float32, device=dy.device)
    abi.call("bbcu_fp32_DifferentiableLut6_BackwardApply", _p(x), _p(dy), _p(dx), _p(idx), _p(W), _p(dW), _p(mean), _p(rstd), _p(sums), _p(dmean),
             _p(dvar), gamma, beta, bias, n_in, O, frames, dy.shape[1], int(total_frames), int(lut_binarize), int(binary), _stream())
    return dx
