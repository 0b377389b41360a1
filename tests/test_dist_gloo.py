"""Frame sharding over 2 ranks (gloo, CPU): the orchestration of binarybrain_b200.dist with a host stand-in for the
operators.  What is under test is the host logic -- shard arithmetic, which sums are exchanged, with which frame
counts, and that dW is complete after wait_grad() -- not the CUDA kernels (those are covered by the -m gpu tests).
The stand-in splits the oracle's batch-norm layer at the same two points the CUDA operators are split at.
"""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


class HostOps:
    """CPU stand-in with the signatures of ops.dl6_* (test double; uses the oracle's LUT arithmetic)."""

    def __init__(self):
        from oracle import port
        self.port = port

    def _raw(self, x, idx, W, frames, lut_binarize, binary):
        # raw LUT value = the no-batch-norm forward without the final clip: take it from dl6 inference with mean 0, var 1, gamma 1, beta 0
        O = idx.shape[0]
        r = self.port.dl6_forward_infer(x[:, :frames].numpy().copy(), idx.numpy(), W.numpy(), np.zeros(O, np.float32), np.ones(O, np.float32),
                                        gamma=1.0, beta=0.0, lut_binarize=int(lut_binarize), binary=int(binary))
        return r["y_pre"]

    def dl6_forward_stats(self, x, idx, W, frames, y, sums, bias=0.25, lut_binarize=False, binary=True):
        raw = self._raw(x, idx, W, frames, lut_binarize, binary)
        y[:, :frames] = torch.from_numpy(raw)
        sums[:, 0] = torch.from_numpy(raw.astype(np.float64).sum(1))
        sums[:, 1] = torch.from_numpy((raw.astype(np.float64) ** 2).sum(1))

    def dl6_forward_normalize(self, y, sums, mean, rstd, running_mean, running_var, frames, total_frames, gamma=0.3, beta=0.5, momentum=0.9,
                              binary=True):
        rF = np.float32(1.0) / np.float32(total_frames)
        m = sums[:, 0].numpy().astype(np.float32) * rF
        v = np.maximum(np.float32(1e-5), sums[:, 1].numpy().astype(np.float32) * rF - m * m)
        r = (np.float32(1.0) / np.sqrt(v)).astype(np.float32)
        mean[:] = torch.from_numpy(m)
        rstd[:] = torch.from_numpy(r)
        running_mean.mul_(momentum).add_(torch.from_numpy(m) * (1 - momentum))
        running_var.mul_(momentum).add_(torch.from_numpy(v) * (1 - momentum))
        t = (y[:, :frames] - mean[:, None]) * rstd[:, None] * gamma + beta
        y[:, :frames] = (t > 0.5).float() if binary else t.clamp(0, 1)

    def dl6_backward_stats(self, x, dy, idx, W, mean, rstd, frames, sums, gamma=0.3, beta=0.5, bias=0.25, lut_binarize=False, binary=True):
        raw = torch.from_numpy(self._raw(x, idx, W, frames, lut_binarize, binary))
        t = (raw - mean[:, None]) * rstd[:, None] * gamma + beta
        g = torch.where((t <= 0) | (t >= 1), torch.zeros(()), dy[:, :frames]) * gamma
        sums[:, 0] = -(g * (raw - mean[:, None]) * (rstd * rstd)[:, None]).double().sum(1)
        sums[:, 1] = -(g * rstd[:, None]).double().sum(1)

    def dl6_backward_apply(self, x, dy, dx, idx, W, dW, mean, rstd, sums, n_in, frames, total_frames, gamma=0.3, beta=0.5, bias=0.25,
                           lut_binarize=False, binary=True):
        raw = torch.from_numpy(self._raw(x, idx, W, frames, lut_binarize, binary))
        rF = 1.0 / total_frames
        dvar = sums[:, 0].float() * rstd
        dmean = (sums[:, 1].float() - mean * dvar) * rF
        t = (raw - mean[:, None]) * rstd[:, None] * gamma + beta
        g = torch.where((t <= 0) | (t >= 1), torch.zeros(()), dy[:, :frames])
        g = g * gamma * rstd[:, None] + dmean[:, None] + raw * (dvar * rF)[:, None]
        dxo, dWo = self.port.sl6_backward(x[:, :frames].numpy().copy(), g.numpy().copy(), idx.numpy(), W.numpy(), n_in, dW=dW.numpy(),
                                          binary=int(binary), lut_binarize=int(lut_binarize))
        dx[:, :frames] = torch.from_numpy(dxo)
        dW.copy_(torch.from_numpy(dWo))
        return dx


def _case():
    rng = np.random.default_rng(12)
    I, O, F = 24, 16, 128
    idx = np.stack([rng.permutation(I)[:6] for _ in range(O)]).astype(np.int32)
    W = np.clip(rng.normal(0.5, 0.25, (O, 64)), 0, 1).astype(np.float32)
    x = rng.random((I, F), dtype=np.float32)
    dy = rng.random((O, F), dtype=np.float32)
    return I, O, F, idx, W, x, dy


def _worker(rank, world, port_no, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port_no)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from binarybrain_b200.dist import ShardedDifferentiableLut6, frame_shard
    I, O, F, idx, W, x, dy = _case()
    b, e = frame_shard(F, rank, world)
    layer = ShardedDifferentiableLut6(torch.from_numpy(idx), torch.from_numpy(W), I, ops=HostOps(), binary=False)
    y = layer.forward(torch.from_numpy(x[:, b:e].copy()), e - b, F)
    dx = layer.backward(torch.from_numpy(dy[:, b:e].copy()))
    dW = layer.wait_grad()
    np.savez(out.format(rank), y=y.numpy(), dx=dx.numpy(), dW=dW.numpy(), mean=layer.mean.numpy(), rstd=layer.rstd.numpy(),
             rm=layer.running_mean.numpy(), b=b, e=e)
    dist.barrier()
    dist.destroy_process_group()


def test_frame_shard_partition():
    from binarybrain_b200.dist import frame_shard
    for total, world in [(1 << 20, 8), (4096, 3), (96, 4), (32, 2), (77, 1)]:
        parts = [frame_shard(total, r, world) for r in range(world)]
        assert parts[0][0] == 0 and parts[-1][1] == total
        assert all(parts[i][1] == parts[i + 1][0] for i in range(world - 1))
        if world > 1:
            assert all(b % 32 == 0 and e % 32 == 0 for b, e in parts)
        sizes = [e - b for b, e in parts]
        assert max(sizes) - min(sizes) <= 32
    with pytest.raises(ValueError):
        frame_shard(100, 0, 2)


def test_two_ranks_equal_one_rank(tmp_path):
    from oracle import port
    I, O, F, idx, W, x, dy = _case()
    out = str(tmp_path / "r{}.npz")
    mp.spawn(_worker, args=(2, 29000 + os.getpid() % 2000, out), nprocs=2, join=True)
    p = port.dl6_forward_train(x, idx, W, np.zeros(O), np.ones(O), binary=0)
    dx_w, dW_w = port.dl6_backward(x, dy, idx, W, p["mean"], p["rstd"], I, binary=0)
    rs = [np.load(out.format(r)) for r in range(2)]
    assert (rs[0]["b"], rs[0]["e"], rs[1]["b"], rs[1]["e"]) == (0, 64, 64, 128)
    y = np.concatenate([r["y"] for r in rs], axis=1)
    dx = np.concatenate([r["dx"] for r in rs], axis=1)
    amp = max(1.0, 0.3 * float(p["rstd"].max()))
    for r in rs:                                    # every rank ends with the global statistics and the complete dW
        assert np.abs(r["mean"] - p["mean"]).max() <= 1e-6
        assert np.abs(r["rstd"] / p["rstd"] - 1).max() <= 1e-4
        assert np.abs(r["rm"] - p["running_mean"]).max() <= 1e-6
        assert np.abs(r["dW"] - dW_w).max() <= 1e-4 * amp * max(1.0, np.abs(dW_w).max())
    assert np.abs(y - p["y"]).max() <= 1e-4 * amp
    assert np.abs(dx - dx_w).max() <= 1e-4 * amp * max(1.0, np.abs(dx_w).max())


def _local_worker(rank, world, port_no, out):
    """Rank 0 alone runs a layer marked sharded=False while a 2-rank group exists; rank 1 goes straight to the barrier.  A layer
    that entered a collective here would leave rank 0 waiting for a partner that never comes (the group's timeout is 20 s)."""
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port_no)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    from binarybrain_b200.dist import ShardedDifferentiableLut6
    if rank == 0:
        I, O, F, idx, W, x, dy = _case()
        layer = ShardedDifferentiableLut6(torch.from_numpy(idx), torch.from_numpy(W), I, ops=HostOps(), binary=False, sharded=False)
        assert layer.world == 1
        y = layer.forward(torch.from_numpy(x.copy()), F, F)
        layer.backward(torch.from_numpy(dy.copy()))
        np.savez(out.format(rank), y=y.numpy(), dW=layer.wait_grad().numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_unsharded_layer_on_one_rank_enters_no_collective(tmp_path):
    from oracle import port
    I, O, F, idx, W, x, dy = _case()
    out = str(tmp_path / "l{}.npz")
    mp.spawn(_local_worker, args=(2, 31000 + os.getpid() % 2000, out), nprocs=2, join=True)
    p = port.dl6_forward_train(x, idx, W, np.zeros(O), np.ones(O), binary=0)
    r = np.load(out.format(0))
    assert np.abs(r["y"] - p["y"]).max() <= 1e-4 * max(1.0, 0.3 * float(p["rstd"].max()))
