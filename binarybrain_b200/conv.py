"""Host-side mirrors of the reference's convolution wrappers over the lowering operators.

    Convolution2d  include/bb/Convolution2d.h:281-308   Im2Col -> per-pixel layers -> Col2Im (backward in reverse)
    MaxPooling     include/bb/MaxPooling.h:190-322, 600-629
    Sequential     include/bb/Sequential.h              forward in order, backward in reverse

Every layer here has the two methods the frame-sharded LUT layer (dist.ShardedDifferentiableLut6) has,
``forward(x, frames, total_frames)`` and ``backward(dy)``, on CUDA frame buffers [nodes, stride].  Lowering multiplies the
frame axis by the output pixels, so inside a Convolution2d the per-pixel layers see ``frames * oh * ow`` frames; batch
statistics there run over pixels and images alike, as in the reference.  The arithmetic back end is injected (``ops``),
by default the CUDA operators -- there is no CPU fallback behind them.
"""
import torch


def _default_ops(ops):
    if ops is None:
        from . import ops as cuda_ops
        return cuda_ops
    return ops


class Sequential:
    def __init__(self, layers):
        self.layers = list(layers)

    def forward(self, x, frames, total_frames=None):
        total_frames = frames if total_frames is None else total_frames
        for layer in self.layers:
            x = layer.forward(x, frames, total_frames)
        return x

    def backward(self, dy):
        for layer in reversed(self.layers):
            dy = layer.backward(dy)
        return dy

    def lut_layers(self):
        out = []
        for layer in self.layers:
            out.extend(layer.lut_layers() if hasattr(layer, "lut_layers") else ([layer] if hasattr(layer, "dW") else []))
        return out


class Convolution2d:
    """`layers` map {c, fh, fw} = c*fh*fw input nodes to c_out nodes, one pixel per frame."""

    def __init__(self, layers, c, h, w, fh, fw, y_stride=1, x_stride=1, padding="valid", border_mode="reflect_101", ops=None):
        self.ops = _default_ops(ops)
        self.inner = layers if isinstance(layers, Sequential) else Sequential(layers)
        self.c, self.h, self.w, self.fh, self.fw = c, h, w, fh, fw
        self.y_stride, self.x_stride, self.padding, self.border_mode = y_stride, x_stride, padding, border_mode
        self.oh, self.ow, _, _ = self.ops.im2col_geometry(h, w, fh, fw, y_stride, x_stride, padding)
        self.c_out = self.inner.layers[-1].n_out

    def lut_layers(self):
        return self.inner.lut_layers()

    def forward(self, x, frames, total_frames=None):
        total_frames = frames if total_frames is None else total_frames
        P = self.oh * self.ow
        cols = self.ops.im2col_forward(x, frames, self.c, self.h, self.w, self.fh, self.fw, self.y_stride, self.x_stride, self.padding,
                                       self.border_mode)
        z = self.inner.forward(cols, frames * P, total_frames * P)
        self._frames = frames
        return self.ops.col2im_forward(z, self.c_out, self.oh, self.ow, frames)

    def backward(self, dy):
        frames = self._frames
        g = self.ops.col2im_backward(dy, self.c_out, self.oh, self.ow, frames)
        g = self.inner.backward(g)
        return self.ops.im2col_backward(g, frames, self.c, self.h, self.w, self.fh, self.fw, self.y_stride, self.x_stride, self.padding)


class MaxPooling:
    def __init__(self, c, h, w, fh, fw, ops=None):
        self.ops = _default_ops(ops)
        self.c, self.h, self.w, self.fh, self.fw = c, h, w, fh, fw
        self.oh, self.ow = (h + fh - 1) // fh, (w + fw - 1) // fw

    def forward(self, x, frames, total_frames=None):
        self._frames = frames
        if x.dtype == torch.int32:                    # bit frames: the input is what backward needs
            self._sel, self._bit = x, True
            return self.ops.maxpool_forward(x, frames, self.c, self.h, self.w, self.fh, self.fw)
        y, self._sel = self.ops.maxpool_forward(x, frames, self.c, self.h, self.w, self.fh, self.fw)
        self._bit = False
        return y

    def backward(self, dy):
        dx = self.ops.maxpool_backward(self._sel, dy, self._frames, self.c, self.h, self.w, self.fh, self.fw, bit_input=self._bit)
        self._sel = None
        return dx
