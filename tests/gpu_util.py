"""Helpers shared by the GPU parity tests: numpy <-> padded CUDA frame buffers."""
import numpy as np
import torch

from binarybrain_b200 import ops


def dev_fp32(a, stride=None, fill=0.0):
    """Dense [nodes, frames] float32 -> CUDA [nodes, stride] (stride defaults to the 32-byte row rule)."""
    a = np.ascontiguousarray(a, np.float32)
    n, f = a.shape
    s = ops.fp32_stride(f) if stride is None else stride
    t = torch.full((n, s), fill, dtype=torch.float32)
    t[:, :f] = torch.from_numpy(a)
    return t.cuda()


def dev_bits(words, frames, stride=None):
    """[nodes, ceil(frames/32)] uint32 -> CUDA int32 [nodes, stride]."""
    words = np.ascontiguousarray(words, np.uint32)
    n, w = words.shape
    s = ops.bit_stride(frames) if stride is None else stride
    t = torch.zeros((n, s), dtype=torch.int32)
    t[:, :w] = torch.from_numpy(words.view(np.int32))
    return t.cuda()


def host_fp32(t, frames):
    return t[:, :frames].cpu().numpy()


def host_bits(t, frames):
    w = (frames + 31) // 32
    return np.ascontiguousarray(t[:, :w].cpu().numpy()).view(np.uint32)


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def wiring(rng, n_in, n_out):
    """6 distinct random inputs per node."""
    if n_in >= 64:
        idx = rng.integers(0, n_in, (n_out, 6))
        for _ in range(8):           # re-draw rows with a repeated index
            s = np.sort(idx, axis=1)
            bad = (s[:, 1:] == s[:, :-1]).any(axis=1)
            if not bad.any():
                break
            idx[bad] = rng.integers(0, n_in, (int(bad.sum()), 6))
        return idx.astype(np.int32)
    return np.stack([rng.permutation(n_in)[:6] for _ in range(n_out)]).astype(np.int32)


def err(a, b):
    """max |a-b| relative to the value range of b (at least 1)."""
    return float(np.abs(a - b).max()) / max(1.0, float(np.abs(b).max()))
