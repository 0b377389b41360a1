"""TEST INFRASTRUCTURE ONLY: numpy front-ends of the CPU oracle.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may import
this package, and only as the checker.  The product (``binarybrain_b200``) never does.

``port``  : oracle/lut6_oracle.c, the plain-C restatement of the reference's CPU arithmetic.
``ref``   : oracle/_ref/libbbref.so, the unmodified reference headers behind oracle/ref_driver.cpp
            (present where it was built from a reference checkout; ``ref.available()`` tells).

Array conventions: fp32 frames ``[node, frame]`` C-contiguous; bit frames ``[node, words]`` uint32
with 32 frames per word, LSB first; wiring ``[out, 6]`` int32; ``W`` ``[out, 64]`` float32; binary
tables ``[out, 2]`` int32.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_PORT_SO = os.path.join(_HERE, "liblut6_oracle.so")
_REF_SO = os.path.join(_HERE, "_ref", "libbbref.so")

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")


def build():
    """Compile the oracle (and oracle/_ref when a reference checkout is present)."""
    subprocess.check_call(["make", "-s", "-C", _HERE, "all"])


def _vp(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def pack_bits(bits):
    """[node, frame] of {0,1} -> [node, ceil(frame/32)] uint32, frame f at bit f&31 of word f>>5."""
    bits = np.asarray(bits).astype(np.uint8)
    n, f = bits.shape
    words = (f + 31) // 32
    pad = np.zeros((n, words * 32), np.uint8)
    pad[:, :f] = bits
    return np.packbits(pad.reshape(n, words, 32), axis=2, bitorder="little").view(np.uint32).reshape(n, words).copy()


def unpack_bits(words, frames):
    words = np.ascontiguousarray(words, np.uint32)
    n = words.shape[0]
    b = np.unpackbits(words.view(np.uint8).reshape(n, -1), axis=1, bitorder="little")
    return b[:, :frames].copy()


def det_uniform(shape, seed):
    """Deterministic uniform[0,1) float32 array from integer hashing only (splitmix64 of the element index): the same values on
    every numpy version, so large test inputs need not be stored with the golden outputs."""
    n = int(np.prod(shape))
    z = np.arange(n, dtype=np.uint64) + np.uint64(((int(seed) + 1) * 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF)
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    z = z ^ (z >> np.uint64(31))
    return ((z >> np.uint64(40)).astype(np.float32) / np.float32(1 << 24)).reshape(shape)


def det_wiring(n_in, n_out, seed):
    """Deterministic [n_out, 6] wiring with six distinct inputs per node (argsort of hashed keys, row by row)."""
    keys = det_uniform((n_out, n_in), seed)
    return np.argsort(keys, axis=1, kind="stable")[:, :6].astype(np.int32)


class _Port:
    """oracle/lut6_oracle.c"""

    def __init__(self):
        self._lib = None

    @property
    def lib(self):
        if self._lib is None:
            if not os.path.exists(_PORT_SO):
                build()
            self._lib = C.CDLL(_PORT_SO)
        return self._lib

    # -- StochasticLut6 ---------------------------------------------------------------------
    def sl6_forward(self, x, idx, W, frames=None, binary=False, lut_binarize=False, bias=0.25, want_bits=False):
        bit_in = x.dtype == np.uint32
        x = np.ascontiguousarray(x)
        F = frames if frames is not None else x.shape[1]
        O = idx.shape[0]
        y = np.zeros((O, F), np.float32)
        yb = np.zeros((O, (F + 31) // 32), np.uint32) if want_bits else None
        self.lib.oracle_sl6_forward(
            C.c_int(bit_in), _vp(x), C.c_size_t(x.shape[1]), _vp(y), C.c_size_t(F), _vp(yb), C.c_size_t((F + 31) // 32),
            _vp(np.ascontiguousarray(idx, np.int32)), _vp(np.ascontiguousarray(W, np.float32)),
            C.c_int(O), C.c_int(F), C.c_int(binary), C.c_int(lut_binarize), C.c_float(bias))
        return (y, yb) if want_bits else y

    def sl6_backward(self, x, dy, idx, W, n_in, dW=None, frames=None, binary=False, lut_binarize=False, bias=0.25):
        bit_in = x.dtype == np.uint32
        x = np.ascontiguousarray(x)
        dy = np.ascontiguousarray(dy, np.float32)
        O, F = dy.shape
        dx = np.zeros((n_in, F), np.float32)
        dW = np.zeros((O, 64), np.float32) if dW is None else np.ascontiguousarray(dW, np.float32).copy()
        self.lib.oracle_sl6_backward(
            C.c_int(bit_in), _vp(x), C.c_size_t(x.shape[1]), _vp(dy), C.c_size_t(F), _vp(dx), C.c_size_t(F),
            _vp(np.ascontiguousarray(idx, np.int32)), _vp(np.ascontiguousarray(W, np.float32)), _vp(dW),
            C.c_int(n_in), C.c_int(O), C.c_int(F), C.c_int(binary), C.c_int(lut_binarize), C.c_float(bias))
        return dx, dW

    # -- DifferentiableLut6 -----------------------------------------------------------------
    def dl6_forward_train(self, x, idx, W, running_mean, running_var, frames=None, gamma=0.3, beta=0.5, momentum=0.9,
                          bias=0.25, lut_binarize=False, binary=True):
        bit_in = x.dtype == np.uint32
        x = np.ascontiguousarray(x)
        F = frames if frames is not None else x.shape[1]
        O = idx.shape[0]
        y = np.zeros((O, F), np.float32)
        ypre = np.zeros((O, F), np.float32)
        yb = np.zeros((O, (F + 31) // 32), np.uint32)
        mean = np.zeros(O, np.float32)
        rstd = np.zeros(O, np.float32)
        rm = np.ascontiguousarray(running_mean, np.float32).copy()
        rv = np.ascontiguousarray(running_var, np.float32).copy()
        self.lib.oracle_dl6_forward_train(
            C.c_int(bit_in), _vp(x), C.c_size_t(x.shape[1]), _vp(y), C.c_size_t(F), _vp(yb), C.c_size_t((F + 31) // 32), _vp(ypre),
            _vp(np.ascontiguousarray(idx, np.int32)), _vp(np.ascontiguousarray(W, np.float32)),
            _vp(mean), _vp(rstd), _vp(rm), _vp(rv),
            C.c_float(gamma), C.c_float(beta), C.c_float(momentum), C.c_float(bias),
            C.c_int(O), C.c_int(F), C.c_int(lut_binarize), C.c_int(1 if bit_in else binary))
        return dict(y=y, y_bits=yb, y_pre=ypre, mean=mean, rstd=rstd, running_mean=rm, running_var=rv)

    def dl6_forward_infer(self, x, idx, W, running_mean, running_var, frames=None, gamma=0.3, beta=0.5, bias=0.25,
                          lut_binarize=False, binary=True):
        bit_in = x.dtype == np.uint32
        x = np.ascontiguousarray(x)
        F = frames if frames is not None else x.shape[1]
        O = idx.shape[0]
        y = np.zeros((O, F), np.float32)
        ypre = np.zeros((O, F), np.float32)
        yb = np.zeros((O, (F + 31) // 32), np.uint32)
        self.lib.oracle_dl6_forward_infer(
            C.c_int(bit_in), _vp(x), C.c_size_t(x.shape[1]), _vp(y), C.c_size_t(F), _vp(yb), C.c_size_t((F + 31) // 32), _vp(ypre),
            _vp(np.ascontiguousarray(idx, np.int32)), _vp(np.ascontiguousarray(W, np.float32)),
            _vp(np.ascontiguousarray(running_mean, np.float32)), _vp(np.ascontiguousarray(running_var, np.float32)),
            C.c_float(gamma), C.c_float(beta), C.c_float(bias), C.c_int(O), C.c_int(F), C.c_int(lut_binarize),
            C.c_int(1 if bit_in else binary))
        return dict(y=y, y_bits=yb, y_pre=ypre)

    def dl6_backward(self, x, dy, idx, W, mean, rstd, n_in, dW=None, frames=None, gamma=0.3, beta=0.5, bias=0.25,
                     lut_binarize=False, binary=True):
        bit_in = x.dtype == np.uint32
        x = np.ascontiguousarray(x)
        dy = np.ascontiguousarray(dy, np.float32)
        O, F = dy.shape
        dx = np.zeros((n_in, F), np.float32)
        dW = np.zeros((O, 64), np.float32) if dW is None else np.ascontiguousarray(dW, np.float32).copy()
        self.lib.oracle_dl6_backward(
            C.c_int(bit_in), _vp(x), C.c_size_t(x.shape[1]), _vp(dy), C.c_size_t(F), _vp(dx), C.c_size_t(F),
            _vp(np.ascontiguousarray(idx, np.int32)), _vp(np.ascontiguousarray(W, np.float32)), _vp(dW),
            _vp(np.ascontiguousarray(mean, np.float32)), _vp(np.ascontiguousarray(rstd, np.float32)),
            C.c_float(gamma), C.c_float(beta), C.c_float(bias), C.c_int(n_in), C.c_int(O), C.c_int(F),
            C.c_int(lut_binarize), C.c_int(1 if bit_in else binary))
        return dx, dW

    # -- StochasticBatchNormalization ---------------------------------------------------------
    def sbn_forward_train(self, x, running_mean, running_var, gamma=0.2, beta=0.5, momentum=0.9):
        x = np.ascontiguousarray(x, np.float32)
        O, F = x.shape
        y = np.zeros_like(x)
        mean = np.zeros(O, np.float32)
        rstd = np.zeros(O, np.float32)
        rm = np.ascontiguousarray(running_mean, np.float32).copy()
        rv = np.ascontiguousarray(running_var, np.float32).copy()
        self.lib.oracle_sbn_forward_train(_vp(x), _vp(y), C.c_size_t(F), _vp(mean), _vp(rstd), _vp(rm), _vp(rv),
                                          C.c_float(gamma), C.c_float(beta), C.c_float(momentum), C.c_int(O), C.c_int(F))
        return dict(y=y, mean=mean, rstd=rstd, running_mean=rm, running_var=rv)

    def sbn_reforward(self, x, mean, rstd, gamma=0.2, beta=0.5):
        x = np.ascontiguousarray(x, np.float32)
        O, F = x.shape
        y = np.zeros_like(x)
        self.lib.oracle_sbn_reforward(_vp(x), _vp(y), C.c_size_t(F), _vp(np.ascontiguousarray(mean, np.float32)),
                                      _vp(np.ascontiguousarray(rstd, np.float32)), C.c_float(gamma), C.c_float(beta), C.c_int(O), C.c_int(F))
        return y

    def sbn_forward_infer(self, x, mean, var, gamma=0.2, beta=0.5):
        x = np.ascontiguousarray(x, np.float32)
        O, F = x.shape
        y = np.zeros_like(x)
        self.lib.oracle_sbn_forward_infer(_vp(x), _vp(y), C.c_size_t(F), _vp(np.ascontiguousarray(mean, np.float32)),
                                          _vp(np.ascontiguousarray(var, np.float32)), C.c_float(gamma), C.c_float(beta), C.c_int(O), C.c_int(F))
        return y

    def sbn_backward(self, x, dy, mean, rstd, gamma=0.2):
        x = np.ascontiguousarray(x, np.float32)
        dy = np.ascontiguousarray(dy, np.float32)
        O, F = x.shape
        dx = np.zeros_like(x)
        self.lib.oracle_sbn_backward(_vp(x), _vp(dy), _vp(dx), C.c_size_t(F), _vp(np.ascontiguousarray(mean, np.float32)),
                                     _vp(np.ascontiguousarray(rstd, np.float32)), C.c_float(gamma), C.c_int(O), C.c_int(F))
        return dx

    # -- BinaryLut6 ---------------------------------------------------------------------------
    def binary_lut6_forward(self, x_words, idx, table, frames):
        x_words = np.ascontiguousarray(x_words, np.uint32)
        O = idx.shape[0]
        y = np.zeros((O, x_words.shape[1]), np.uint32)
        self.lib.oracle_binary_lut6_forward(_vp(x_words), _vp(y), C.c_size_t(x_words.shape[1]),
                                            _vp(np.ascontiguousarray(idx, np.int32)), _vp(np.ascontiguousarray(table, np.int32)),
                                            C.c_int(O), C.c_int(frames))
        return y

    # -- Reduce and losses ----------------------------------------------------------------------
    def reduce_forward(self, x, out_nodes):
        x = np.ascontiguousarray(x, np.float32)
        y = np.zeros((out_nodes, x.shape[1]), np.float32)
        self.lib.oracle_reduce_forward(_vp(x), _vp(y), C.c_int(x.shape[0]), C.c_int(out_nodes), C.c_int(x.shape[1]))
        return y

    def reduce_backward(self, dy, in_nodes):
        dy = np.ascontiguousarray(dy, np.float32)
        dx = np.zeros((in_nodes, dy.shape[1]), np.float32)
        self.lib.oracle_reduce_backward(_vp(dy), _vp(dx), C.c_int(in_nodes), C.c_int(dy.shape[0]), C.c_int(dy.shape[1]))
        return dx

    def softmax_cross_entropy(self, y, t):
        y = np.ascontiguousarray(y, np.float32)
        t = np.ascontiguousarray(t, np.float32)
        dy = np.zeros_like(y)
        self.lib.oracle_softmax_cross_entropy.restype = C.c_double
        loss = self.lib.oracle_softmax_cross_entropy(_vp(y), _vp(t), _vp(dy), C.c_int(y.shape[0]), C.c_int(y.shape[1]))
        return dy, float(loss)

    def mean_squared_error(self, y, t, batch_size=None):
        y = np.ascontiguousarray(y, np.float32)
        t = np.ascontiguousarray(t, np.float32)
        dy = np.zeros_like(y)
        self.lib.oracle_mean_squared_error.restype = C.c_double
        loss = self.lib.oracle_mean_squared_error(_vp(y), _vp(t), _vp(dy), C.c_int(y.shape[0]), C.c_int(y.shape[1]),
                                                  C.c_int(y.shape[1] if batch_size is None else batch_size))
        return dy, float(loss)

    # -- binary modulation -------------------------------------------------------------------------
    def real_to_binary(self, x, frame_mod=1, depth_mod=1, thresholds=None, lo=0.0, hi=1.0, point_size=1):
        x = np.ascontiguousarray(x, np.float32)
        nodes, frames = x.shape
        words = (frames * frame_mod + 31) // 32
        y = np.zeros((nodes * depth_mod, words), np.uint32)
        th = None if thresholds is None else np.ascontiguousarray(thresholds, np.float32)
        self.lib.oracle_real_to_binary(_vp(x), _vp(y), C.c_size_t(words), _vp(th), C.c_int(nodes // point_size), C.c_int(point_size),
                                       C.c_int(frames), C.c_int(frame_mod), C.c_int(depth_mod), C.c_float(lo), C.c_float(hi))
        return y

    def binary_to_real(self, x_words, y_nodes, y_frames, frame_mux=1):
        x_words = np.ascontiguousarray(x_words, np.uint32)
        y = np.zeros((y_nodes, y_frames), np.float32)
        self.lib.oracle_binary_to_real_forward(_vp(x_words), C.c_size_t(x_words.shape[1]), _vp(y), C.c_int(x_words.shape[0]), C.c_int(y_nodes),
                                               C.c_int(y_frames), C.c_int(frame_mux))
        return y

    def binary_to_real_backward(self, dy, x_nodes, frame_mux=1):
        dy = np.ascontiguousarray(dy, np.float32)
        dx = np.zeros((x_nodes, dy.shape[1] * frame_mux), np.float32)
        self.lib.oracle_binary_to_real_backward(_vp(dy), _vp(dx), C.c_int(x_nodes), C.c_int(dy.shape[0]), C.c_int(dy.shape[1]), C.c_int(frame_mux))
        return dx

    # -- convolution lowering -------------------------------------------------------------------
    BORDER = {"constant": 0, "reflect": 1, "reflect_101": 2, "replicate": 3, "wrap": 4}

    @staticmethod
    def im2col_geometry(h, w, fh, fw, y_stride=1, x_stride=1, padding="valid"):
        """(out_h, out_w, y_offset, x_offset) of ConvolutionIm2Col (include/bb/ConvolutionIm2Col.h:200-215)."""
        if padding == "valid":
            return ((h - fh + 1) + (y_stride - 1)) // y_stride, ((w - fw + 1) + (x_stride - 1)) // x_stride, 0, 0
        if padding == "same":
            return (h + y_stride - 1) // y_stride, (w + x_stride - 1) // x_stride, (fh - 1) // 2, (fw - 1) // 2
        raise ValueError(padding)

    def im2col_forward(self, x, c, h, w, fh, fw, y_stride=1, x_stride=1, padding="valid", border_mode="reflect_101", border_value=0.0,
                       frames=None):
        """x: float32 [c*h*w][frames] or uint32 words [c*h*w][words] (then pass ``frames``)."""
        oh, ow, yo, xo = self.im2col_geometry(h, w, fh, fw, y_stride, x_stride, padding)
        bm = self.BORDER[border_mode]
        if x.dtype == np.uint32:
            x = np.ascontiguousarray(x)
            of = frames * oh * ow
            y = np.zeros((c * fh * fw, (of + 31) // 32), np.uint32)
            self.lib.oracle_im2col_forward_bit(_vp(x), C.c_size_t(x.shape[1]), _vp(y), C.c_size_t(y.shape[1]), C.c_int(x_stride), C.c_int(y_stride),
                                               C.c_int(xo), C.c_int(yo), C.c_int(frames), C.c_int(w), C.c_int(h), C.c_int(c), C.c_int(ow),
                                               C.c_int(oh), C.c_int(fw), C.c_int(fh), C.c_int(bm))
            return y
        x = np.ascontiguousarray(x, np.float32)
        frames = x.shape[1]
        y = np.zeros((c * fh * fw, frames * oh * ow), np.float32)
        self.lib.oracle_im2col_forward_f32(_vp(x), _vp(y), C.c_int(x_stride), C.c_int(y_stride), C.c_int(xo), C.c_int(yo), C.c_int(frames),
                                           C.c_int(w), C.c_int(h), C.c_int(c), C.c_int(ow), C.c_int(oh), C.c_int(fw), C.c_int(fh), C.c_int(bm),
                                           C.c_float(border_value))
        return y

    def im2col_backward(self, dy, c, h, w, fh, fw, y_stride=1, x_stride=1, padding="valid"):
        oh, ow, yo, xo = self.im2col_geometry(h, w, fh, fw, y_stride, x_stride, padding)
        dy = np.ascontiguousarray(dy, np.float32)
        frames = dy.shape[1] // (oh * ow)
        dx = np.zeros((c * h * w, frames), np.float32)
        self.lib.oracle_im2col_backward_f32(_vp(dy), _vp(dx), C.c_int(x_stride), C.c_int(y_stride), C.c_int(xo), C.c_int(yo), C.c_int(frames),
                                            C.c_int(w), C.c_int(h), C.c_int(c), C.c_int(ow), C.c_int(oh), C.c_int(fw), C.c_int(fh))
        return dx

    def col2im_forward(self, x, c, h, w, out_frames):
        if x.dtype == np.uint32:
            x = np.ascontiguousarray(x)
            y = np.zeros((c * h * w, (out_frames + 31) // 32), np.uint32)
            self.lib.oracle_col2im_forward_bit(_vp(x), C.c_size_t(x.shape[1]), _vp(y), C.c_size_t(y.shape[1]), C.c_int(w), C.c_int(h), C.c_int(c),
                                               C.c_int(out_frames))
            return y
        x = np.ascontiguousarray(x, np.float32)
        y = np.zeros((c * h * w, out_frames), np.float32)
        self.lib.oracle_col2im_forward_f32(_vp(x), _vp(y), C.c_int(w), C.c_int(h), C.c_int(c), C.c_int(out_frames))
        return y

    def col2im_backward(self, dy, c, h, w):
        dy = np.ascontiguousarray(dy, np.float32)
        out_frames = dy.shape[1]
        dx = np.zeros((c, out_frames * h * w), np.float32)
        self.lib.oracle_col2im_backward_f32(_vp(dy), _vp(dx), C.c_int(w), C.c_int(h), C.c_int(c), C.c_int(out_frames))
        return dx

    def maxpool_forward(self, x, c, h, w, fh, fw, frames=None):
        """float32: returns (y, argmax); uint32 words: returns y."""
        oh, ow = (h + fh - 1) // fh, (w + fw - 1) // fw
        if x.dtype == np.uint32:
            x = np.ascontiguousarray(x)
            y = np.zeros((c * oh * ow, x.shape[1]), np.uint32)
            self.lib.oracle_maxpool_forward_bit(_vp(x), _vp(y), C.c_size_t(x.shape[1]), C.c_int(fh), C.c_int(fw), C.c_int(w), C.c_int(h), C.c_int(c),
                                                C.c_int(frames))
            return y
        x = np.ascontiguousarray(x, np.float32)
        frames = x.shape[1]
        y = np.zeros((c * oh * ow, frames), np.float32)
        am = np.zeros((c * oh * ow, frames), np.int32)
        self.lib.oracle_maxpool_forward_f32(_vp(x), _vp(y), _vp(am), C.c_int(fh), C.c_int(fw), C.c_int(w), C.c_int(h), C.c_int(c), C.c_int(frames))
        return y, am

    def maxpool_backward(self, argmax_or_xbits, dy, c, h, w, fh, fw):
        """argmax int32 [c*oh*ow][frames] (fp32 layer) or the forward input as uint32 words (bit layer)."""
        dy = np.ascontiguousarray(dy, np.float32)
        frames = dy.shape[1]
        dx = np.zeros((c * h * w, frames), np.float32)
        a = np.ascontiguousarray(argmax_or_xbits)
        if a.dtype == np.uint32:
            self.lib.oracle_maxpool_backward_bit_f32(_vp(a), C.c_size_t(a.shape[1]), _vp(dy), _vp(dx), C.c_int(fh), C.c_int(fw), C.c_int(w),
                                                     C.c_int(h), C.c_int(c), C.c_int(frames))
        else:
            self.lib.oracle_maxpool_backward_f32(_vp(a.astype(np.int32)), _vp(dy), _vp(dx), C.c_int(fh), C.c_int(fw), C.c_int(w), C.c_int(h),
                                                 C.c_int(c), C.c_int(frames))
        return dx

    # -- Adam ---------------------------------------------------------------------------------
    def adam_update(self, p, g, m, v, state, lr=0.001, beta1=0.9, beta2=0.999):
        """In place on float32 arrays p, g, m, v; ``state`` is a 2-element float32 array [b1^t, b2^t] starting at 1."""
        self.lib.oracle_adam_update(_vp(p), _vp(g), _vp(m), _vp(v), C.c_size_t(p.size), C.c_float(lr), C.c_float(beta1),
                                    C.c_float(beta2), C.c_void_p(state.ctypes.data), C.c_void_p(state.ctypes.data + 4))


class _Ref:
    """oracle/_ref/libbbref.so: the unmodified reference CPU path."""

    def __init__(self):
        self._lib = None

    def available(self):
        return os.path.exists(_REF_SO)

    @property
    def lib(self):
        if self._lib is None:
            self._lib = C.CDLL(_REF_SO)
        return self._lib

    def num_threads(self):
        return int(self.lib.bbref_num_threads())

    def use_all_cores(self):
        """OpenMP team = every core this process may run on, whatever OMP_NUM_THREADS the launcher exported; returns the count."""
        n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
        if hasattr(self.lib, "bbref_set_num_threads"):
            self.lib.bbref_set_num_threads(C.c_int(n))
        return self.num_threads()

    def stochastic_lut6(self, x, idx, W, frames=None, binary=False, lut_binarize=False, host_simd=True, dy=None, dW=None):
        bit_in = x.dtype == np.uint32
        x = np.ascontiguousarray(x)
        F = frames if frames is not None else x.shape[1]
        O, I = idx.shape[0], x.shape[0]
        y = np.zeros((O, F), np.float32)
        t = np.zeros(2, np.float64)
        dx = dWo = None
        if dy is not None:
            dy = np.ascontiguousarray(dy, np.float32)
            dx = np.zeros((I, F), np.float32)
            dWo = np.zeros((O, 64), np.float32) if dW is None else np.ascontiguousarray(dW, np.float32).copy()
        self.lib.bbref_stochastic_lut6(
            C.c_int(bit_in), _vp(x), C.c_int(I), C.c_int(O), C.c_int(F), _vp(np.ascontiguousarray(idx, np.int32)),
            _vp(np.ascontiguousarray(W, np.float32)), C.c_int(binary), C.c_int(lut_binarize), C.c_int(host_simd),
            _vp(y), _vp(dy), _vp(dx), _vp(dWo), _vp(t))
        return dict(y=y, dx=dx, dW=dWo, t_fwd=t[0], t_bwd=t[1])

    def differentiable_lut6(self, x, idx, W, frames=None, batch_norm=True, binary=True, lut_binarize=False, gamma=0.3, beta=0.5,
                            momentum=0.9, running_mean=None, running_var=None, train=True, dy=None, dW=None):
        bit_io = x.dtype == np.uint32
        x = np.ascontiguousarray(x)
        F = frames if frames is not None else x.shape[1]
        O, I = idx.shape[0], x.shape[0]
        y = np.zeros((O, (F + 31) // 32), np.uint32) if bit_io else np.zeros((O, F), np.float32)
        mean = np.zeros(O, np.float32)
        rstd = np.zeros(O, np.float32)
        rm = np.zeros(O, np.float32) if running_mean is None else np.ascontiguousarray(running_mean, np.float32).copy()
        rv = np.ones(O, np.float32) if running_var is None else np.ascontiguousarray(running_var, np.float32).copy()
        t = np.zeros(2, np.float64)
        dx = dWo = None
        if dy is not None:
            dy = np.ascontiguousarray(dy, np.float32)
            dx = np.zeros((I, F), np.float32)
            dWo = np.zeros((O, 64), np.float32) if dW is None else np.ascontiguousarray(dW, np.float32).copy()
        self.lib.bbref_differentiable_lut6(
            C.c_int(bit_io), _vp(x), C.c_int(I), C.c_int(O), C.c_int(F), _vp(np.ascontiguousarray(idx, np.int32)),
            _vp(np.ascontiguousarray(W, np.float32)), C.c_int(batch_norm), C.c_int(binary), C.c_int(lut_binarize),
            C.c_float(gamma), C.c_float(beta), C.c_float(momentum), _vp(rm), _vp(rv), C.c_int(train),
            _vp(y), _vp(mean), _vp(rstd), _vp(dy), _vp(dx), _vp(dWo), _vp(t))
        return dict(y=y, mean=mean, rstd=rstd, running_mean=rm, running_var=rv, dx=dx, dW=dWo, t_fwd=t[0], t_bwd=t[1])

    def binary_lut6(self, x_words, idx, table, frames, host_simd=True):
        x_words = np.ascontiguousarray(x_words, np.uint32)
        assert x_words.shape[1] == (frames + 31) // 32
        O, I = idx.shape[0], x_words.shape[0]
        y = np.zeros((O, x_words.shape[1]), np.uint32)
        t = np.zeros(2, np.float64)
        self.lib.bbref_binary_lut6(_vp(x_words), C.c_int(I), C.c_int(O), C.c_int(frames), _vp(np.ascontiguousarray(idx, np.int32)),
                                   _vp(np.ascontiguousarray(table, np.int32)), C.c_int(host_simd), _vp(y), _vp(t))
        return dict(y=y, t_fwd=t[0])

    def stochastic_bn(self, x, mode=0, gamma=0.2, beta=0.5, momentum=0.9, running_mean=None, running_var=None, dy=None):
        x = np.ascontiguousarray(x, np.float32)
        O, F = x.shape
        y = np.zeros_like(x)
        mean = np.zeros(O, np.float32)
        rstd = np.zeros(O, np.float32)
        rm = np.zeros(O, np.float32) if running_mean is None else np.ascontiguousarray(running_mean, np.float32).copy()
        rv = np.ones(O, np.float32) if running_var is None else np.ascontiguousarray(running_var, np.float32).copy()
        dx = None
        if dy is not None:
            dy = np.ascontiguousarray(dy, np.float32)
            dx = np.zeros_like(x)
        self.lib.bbref_stochastic_bn(_vp(x), C.c_int(O), C.c_int(F), C.c_float(gamma), C.c_float(beta), C.c_float(momentum),
                                     _vp(rm), _vp(rv), C.c_int(mode), _vp(y), _vp(mean), _vp(rstd), _vp(dy), _vp(dx))
        return dict(y=y, mean=mean, rstd=rstd, running_mean=rm, running_var=rv, dx=dx)

    def init_layer(self, n_in, n_out, seed=1, connection=""):
        idx = np.zeros((n_out, 6), np.int32)
        W = np.zeros((n_out, 64), np.float32)
        self.lib.bbref_init_layer(C.c_int(n_in), C.c_int(n_out), C.c_uint64(seed), C.c_char_p(connection.encode()), _vp(idx), _vp(W))
        return idx, W

    def init_connection(self, in_shape, out_shape, seed=1, connection=""):
        """[out_nodes, 6] wiring of a fresh reference layer with these node shapes under a connection rule."""
        ins, outs = np.asarray(in_shape, np.int32), np.asarray(out_shape, np.int32)
        idx = np.zeros((int(np.prod(outs)), 6), np.int32)
        self.lib.bbref_init_connection(C.c_int(len(ins)), _vp(ins), _vp(outs), C.c_uint64(seed), C.c_char_p(connection.encode()), _vp(idx))
        return idx

    def differentiable_lut6_adam(self, x, idx, W, dy, steps, batch_norm=True, binary=False, lut_binarize=False, gamma=0.3, beta=0.5,
                                 momentum=0.9, lr=0.001, beta1=0.9, beta2=0.999):
        x = np.ascontiguousarray(x, np.float32)
        dy = np.ascontiguousarray(dy, np.float32)
        I, F = x.shape
        O = idx.shape[0]
        Wo = np.ascontiguousarray(W, np.float32).copy()
        y = np.zeros((O, F), np.float32)
        rm = np.zeros(O, np.float32)
        rv = np.zeros(O, np.float32)
        self.lib.bbref_differentiable_lut6_adam(
            _vp(x), C.c_int(I), C.c_int(O), C.c_int(F), _vp(np.ascontiguousarray(idx, np.int32)), _vp(Wo),
            C.c_int(batch_norm), C.c_int(binary), C.c_int(lut_binarize), C.c_float(gamma), C.c_float(beta), C.c_float(momentum),
            _vp(dy), C.c_int(steps), C.c_float(lr), C.c_float(beta1), C.c_float(beta2), _vp(y), _vp(rm), _vp(rv))
        return dict(W=Wo, y=y, running_mean=rm, running_var=rv)


    def real_to_binary(self, x, frame_mod=1, depth_mod=1, seed=0, point_size=1):
        x = np.ascontiguousarray(x, np.float32)
        nodes, frames = x.shape
        of = frames * frame_mod
        y = np.zeros((nodes * depth_mod, (of + 31) // 32), np.uint32)
        th = np.zeros((nodes, of), np.float32)
        self.lib.bbref_real_to_binary(_vp(x), C.c_int(nodes // point_size), C.c_int(point_size), C.c_int(frames), C.c_int(frame_mod),
                                      C.c_int(depth_mod), C.c_uint64(seed), _vp(y), _vp(th))
        return y, (th if seed else None)

    def binary_to_real(self, x_words, y_nodes, y_frames, frame_mux=1, dy=None):
        x_words = np.ascontiguousarray(x_words, np.uint32)
        x_nodes = x_words.shape[0]
        y = np.zeros((y_nodes, y_frames), np.float32)
        dx = None
        if dy is not None:
            dy = np.ascontiguousarray(dy, np.float32)
            dx = np.zeros((x_nodes, y_frames * frame_mux), np.float32)
        self.lib.bbref_binary_to_real(_vp(x_words), C.c_int(x_nodes), C.c_int(y_nodes), C.c_int(y_frames), C.c_int(frame_mux), _vp(y), _vp(dy), _vp(dx))
        return y, dx

    def im2col(self, x, c, h, w, fh, fw, y_stride=1, x_stride=1, padding="valid", border_mode="reflect_101", dy=None, frames=None):
        """Returns (y, dx); x float32 [c*h*w][frames] or uint32 words (then pass ``frames``; forward only)."""
        bit = x.dtype == np.uint32
        x = np.ascontiguousarray(x) if bit else np.ascontiguousarray(x, np.float32)
        frames = frames if bit else x.shape[1]
        hw = C.c_int(0)
        args = lambda y, dyv, dxv: self.lib.bbref_im2col(C.c_int(int(bit)), _vp(x), C.c_int(c), C.c_int(h), C.c_int(w), C.c_int(frames), C.c_int(fh),
                                                         C.c_int(fw), C.c_int(y_stride), C.c_int(x_stride), padding.encode(), border_mode.encode(),
                                                         _vp(y), _vp(dyv), _vp(dxv), C.byref(hw))
        args(None, None, None)                       # first pass: output geometry
        of = frames * hw.value
        y = np.zeros((c * fh * fw, (of + 31) // 32), np.uint32) if bit else np.zeros((c * fh * fw, of), np.float32)
        dx = None
        if dy is not None and not bit:
            dy = np.ascontiguousarray(dy, np.float32)
            dx = np.zeros((c * h * w, frames), np.float32)
        args(y, dy, dx)
        return y, dx

    def col2im(self, x, c, h, w, out_frames, dy=None):
        bit = x.dtype == np.uint32
        x = np.ascontiguousarray(x) if bit else np.ascontiguousarray(x, np.float32)
        y = np.zeros((c * h * w, (out_frames + 31) // 32), np.uint32) if bit else np.zeros((c * h * w, out_frames), np.float32)
        dx = None
        if dy is not None and not bit:
            dy = np.ascontiguousarray(dy, np.float32)
            dx = np.zeros((c, out_frames * h * w), np.float32)
        self.lib.bbref_col2im(C.c_int(int(bit)), _vp(x), C.c_int(c), C.c_int(h), C.c_int(w), C.c_int(out_frames), _vp(y), _vp(dy), _vp(dx))
        return y, dx

    def maxpool(self, x, c, h, w, fh, fw, dy=None, frames=None):
        bit = x.dtype == np.uint32
        x = np.ascontiguousarray(x) if bit else np.ascontiguousarray(x, np.float32)
        frames = frames if bit else x.shape[1]
        oh, ow = (h + fh - 1) // fh, (w + fw - 1) // fw
        y = np.zeros((c * oh * ow, (frames + 31) // 32), np.uint32) if bit else np.zeros((c * oh * ow, frames), np.float32)
        dx = None
        if dy is not None:
            dy = np.ascontiguousarray(dy, np.float32)
            dx = np.zeros((c * h * w, frames), np.float32)
        self.lib.bbref_maxpool(C.c_int(int(bit)), _vp(x), C.c_int(c), C.c_int(h), C.c_int(w), C.c_int(frames), C.c_int(fh), C.c_int(fw), _vp(y),
                               _vp(dy), _vp(dx))
        return y, dx

    LAYER_KINDS = {"dl6_fp32": 0, "dl6_bit": 1, "sl6_fp32": 2, "binary_lut6": 3}

    def layer_dump(self, kind, n_in, idx, tables, running_mean=None, running_var=None, batch_norm=True, binary=True, lut_binarize=False,
                   gamma=0.3, beta=0.5, momentum=0.9):
        """DumpObject bytes (uint8 array) of a reference layer holding the given wiring and tables."""
        k = self.LAYER_KINDS[kind]
        idx = np.ascontiguousarray(idx, np.int32)
        O = idx.shape[0]
        tables = np.ascontiguousarray(tables, np.int32 if k == 3 else np.float32)
        rm = np.zeros(O, np.float32) if running_mean is None else np.ascontiguousarray(running_mean, np.float32)
        rv = np.ones(O, np.float32) if running_var is None else np.ascontiguousarray(running_var, np.float32)
        buf = np.zeros(4096 + O * 1024, np.uint8)
        self.lib.bbref_layer_dump.restype = C.c_longlong
        n = self.lib.bbref_layer_dump(C.c_int(k), C.c_int(n_in), C.c_int(O), _vp(idx), _vp(tables), _vp(rm), _vp(rv), C.c_int(batch_norm),
                                      C.c_int(binary), C.c_int(lut_binarize), C.c_float(gamma), C.c_float(beta), C.c_float(momentum), _vp(buf),
                                      C.c_longlong(buf.size))
        assert n > 0, n
        return buf[:n].copy()

    def layer_load(self, kind, data, n_in, n_out):
        """LoadObject `data` into a reference layer and read its state back: dict(idx, tables, running_mean, running_var, flags, params)."""
        k = self.LAYER_KINDS[kind]
        data = np.ascontiguousarray(data, np.uint8)
        idx = np.zeros((n_out, 6), np.int32)
        tables = np.zeros((n_out, 2), np.int32) if k == 3 else np.zeros((n_out, 64), np.float32)
        rm, rv = np.zeros(n_out, np.float32), np.zeros(n_out, np.float32)
        flags, params = np.zeros(3, np.int32), np.zeros(3, np.float32)
        rc = self.lib.bbref_layer_load(C.c_int(k), _vp(data), C.c_longlong(data.size), C.c_int(n_in), C.c_int(n_out), _vp(idx), _vp(tables),
                                       _vp(rm), _vp(rv), _vp(flags), _vp(params))
        assert rc == 0, rc
        return dict(idx=idx, tables=tables, running_mean=rm, running_var=rv, lut_binarize=bool(flags[0]), binary=bool(flags[1]),
                    batch_norm=bool(flags[2]), gamma=float(params[0]), beta=float(params[1]))

    def layer_redump(self, kind, data, n_out):
        """LoadObject then DumpObject through the reference: the bytes it writes back."""
        data = np.ascontiguousarray(data, np.uint8)
        out = np.zeros(data.size + 4096, np.uint8)
        self.lib.bbref_layer_redump.restype = C.c_longlong
        n = self.lib.bbref_layer_redump(C.c_int(self.LAYER_KINDS[kind]), _vp(data), C.c_longlong(data.size), C.c_int(n_out), _vp(out),
                                        C.c_longlong(out.size))
        assert n > 0, n
        return out[:n].copy()

    def _lut_mlp_step(self, x, t, widths, classes, idx_list, W_list, use_mse, lr):
        x = np.ascontiguousarray(x, np.float32)
        t = np.ascontiguousarray(t, np.float32)
        F = x.shape[1]
        idx = np.ascontiguousarray(np.concatenate([np.asarray(i, np.int32).reshape(-1) for i in idx_list]))
        W = np.ascontiguousarray(np.concatenate([np.asarray(w, np.float32).reshape(-1) for w in W_list]))
        wd = np.ascontiguousarray(widths, np.int32)
        y = np.zeros((classes, F), np.float32)
        dx = np.zeros((widths[0], F), np.float32)
        loss = C.c_double(0)
        self.lib.bbref_lut_mlp_step(_vp(x), _vp(t), C.c_int(F), C.c_int(len(widths) - 1), _vp(wd), C.c_int(classes), _vp(idx), _vp(W),
                                    C.c_int(use_mse), C.c_float(lr), _vp(y), C.byref(loss), _vp(dx))
        out, o = [], 0
        for n in widths[1:]:
            out.append(W[o:o + n * 64].reshape(n, 64).copy())
            o += n * 64
        return dict(y=y, loss=loss.value, dx=dx, W=out)

    def lut_mlp_step(self, x, t, widths, classes, idx_list, W_list, use_mse=False, lr=0.001):
        """One training step (forward, loss, backward, Adam) of stacked DifferentiableLut6 layers + Reduce through the reference's Sequential."""
        return self._lut_mlp_step(x, t, list(widths), classes, idx_list, W_list, int(use_mse), lr)


    CNN_WIDTHS = (216, 36, 32, 216, 36, 32, 384, 64, 384, 64, 1024, 420, 70, 10)

    @staticmethod
    def cnn_input_widths(hw=32):
        """Input node counts of the 14 LUT layers of the LUT-CNN on {3, hw, hw} images (the first dense layer reads 64 * (hw/4)^2 nodes)."""
        return (27, 216, 36, 288, 216, 36, 288, 384, 576, 384, 64 * (hw // 4) ** 2, 1024, 420, 70)

    def lut_cnn_step(self, x, dy, idx_list, W_list, hw=32):
        """Forward (training) + backward of the LUT-CNN through the reference's Sequential / Convolution2d / MaxPooling / DifferentiableLutN.
        x [3*hw*hw, B] fp32, dy [10, B]; returns y [10, B], dx, and the table gradients of the 14 LUT layers."""
        x = np.ascontiguousarray(x, np.float32)
        dy = np.ascontiguousarray(dy, np.float32)
        B = x.shape[1]
        idx = np.ascontiguousarray(np.concatenate([np.asarray(i, np.int32).reshape(-1) for i in idx_list]))
        W = np.ascontiguousarray(np.concatenate([np.asarray(w, np.float32).reshape(-1) for w in W_list]))
        y = np.zeros((10, B), np.float32)
        dx = np.zeros((3 * hw * hw, B), np.float32)
        dW = np.zeros_like(W)
        self.lib.bbref_lut_cnn_step(_vp(x), _vp(dy), C.c_int(B), C.c_int(hw), _vp(idx), _vp(W), _vp(y), _vp(dx), _vp(dW))
        out, o = [], 0
        for n in self.CNN_WIDTHS:
            out.append(dW[o:o + n * 64].reshape(n, 64).copy())
            o += n * 64
        return dict(y=y, dx=dx, dW=out)


port = _Port()
ref = _Ref()
