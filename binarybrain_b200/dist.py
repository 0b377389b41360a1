"""Frame-sharded data parallelism for the DifferentiableLut6 path (one process per GPU).

The reference has no multi-device path (include/bb/Memory.h:215-216 leaves it for the future); this layer is
new.  Every rank holds a contiguous shard of the frames of a step and a full replica of wiring, tables and
optimizer state.  Per layer and step exactly three exchanges are needed:

  forward : per-node (sum y, sum y^2) over ALL frames      -> all-reduce of [O, 2] fp64, on the critical path
  backward: per-node (dstd, dmeanx)   over ALL frames      -> all-reduce of [O, 2] fp64, on the critical path
  backward: dW [O, 64] fp32                                -> all-reduce, issued asynchronously so that it overlaps
                                                              the backward of the layer below

The compute halves are the bbcu_fp32_DifferentiableLut6_{Forward,Backward}{Stats,Normalize,Apply} operators; the
exchanges go through torch.distributed (NCCL over NVLink on GPUs).  The arithmetic back end is injected (`ops`),
which is how the CPU tests drive the same orchestration over gloo with a host stand-in.
"""
import torch
import torch.distributed as dist


def frame_shard(total_frames, rank, world, align=32):
    """Contiguous frame range [begin, end) of `rank`: equal shares, multiples of `align` frames (bit words / 32-byte rows)."""
    if total_frames % align != 0 and world > 1:
        raise ValueError(f"total_frames must be a multiple of {align} to shard it")
    units = total_frames // align if world > 1 else total_frames
    unit = align if world > 1 else 1
    base, extra = divmod(units, world)
    begin = rank * base + min(rank, extra)
    end = begin + base + (1 if rank < extra else 0)
    return begin * unit, end * unit


class ShardedDifferentiableLut6:
    """One DifferentiableLut6 layer (fp32, batch norm on) whose frames are sharded over the ranks of `group`."""

    def __init__(self, idx, W, n_in, ops=None, group=None, gamma=0.3, beta=0.5, momentum=0.9, binary=False, lut_binarize=False, sharded=True):
        if ops is None:
            from . import ops as cuda_ops          # the CUDA operators; there is no CPU fallback behind them
            ops = cuda_ops
        self.ops, self.group = ops, group
        self.sharded = sharded          # False: a purely local layer that never enters a collective, whatever process group exists
        self.idx, self.W, self.n_in = idx, W, n_in
        self.n_out = idx.shape[0]
        dev = W.device
        self.dW = torch.zeros_like(W)
        self.running_mean = torch.zeros(self.n_out, dtype=torch.float32, device=dev)
        self.running_var = torch.ones(self.n_out, dtype=torch.float32, device=dev)
        self.mean = torch.empty(self.n_out, dtype=torch.float32, device=dev)
        self.rstd = torch.empty(self.n_out, dtype=torch.float32, device=dev)
        self.sums = torch.zeros((self.n_out, 2), dtype=torch.float64, device=dev)
        self.gamma, self.beta, self.momentum, self.binary, self.lut_binarize = gamma, beta, momentum, binary, lut_binarize
        self._x = self._y = None
        self._pending = None

    @property
    def world(self):
        if not self.sharded:
            return 1
        return dist.get_world_size(self.group) if dist.is_available() and dist.is_initialized() else 1

    def _allreduce(self, t, async_op=False):
        if self.world == 1:
            return None
        return dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group, async_op=async_op)

    def forward(self, x, frames, total_frames, y=None):
        """x: this rank's [n_in, stride] shard with `frames` valid frames; total_frames: frames of the whole step."""
        if y is None:
            y = torch.empty((self.n_out, x.shape[1]), dtype=torch.float32, device=x.device)
        self._fused = self.world == 1 and self.binary and hasattr(self.ops, "differentiable_lut6_forward_training")
        if self._fused:
            # one rank, binary mode: the unsplit operators, which take the per-pattern table route (no exchange point is needed)
            _, mean, rstd = self.ops.differentiable_lut6_forward_training(x, self.idx, self.W, self.running_mean, self.running_var, frames, y=y,
                                                                         gamma=self.gamma, beta=self.beta, momentum=self.momentum,
                                                                         lut_binarize=self.lut_binarize, binary=True)
            self.mean, self.rstd = mean, rstd
            self._x, self._frames, self._total, self._y = x, frames, total_frames, None
            return y
        self.ops.dl6_forward_stats(x, self.idx, self.W, frames, y, self.sums, lut_binarize=self.lut_binarize, binary=self.binary)
        self._allreduce(self.sums)
        self.ops.dl6_forward_normalize(y, self.sums, self.mean, self.rstd, self.running_mean, self.running_var, frames, total_frames,
                                       gamma=self.gamma, beta=self.beta, momentum=self.momentum, binary=self.binary)
        self._x, self._frames, self._total = x, frames, total_frames
        # the output doubles as the saved pre-activation (non-binary mode): in a stack of layers it is the next layer's input
        # and stays alive until that layer's backward, i.e. past this layer's
        self._y = y if (not self.binary and hasattr(self.ops, "dl6_backward_stats_from_output")) else None
        return y

    def backward(self, dy, dx=None):
        """Returns dx for this rank's frames; dW (local partial) is all-reduced asynchronously -- call wait_grad() before using it."""
        x, frames, total = self._x, self._frames, self._total
        if dx is None:
            dx = torch.empty((self.n_in, dy.shape[1]), dtype=torch.float32, device=dy.device)
        kw = dict(gamma=self.gamma, beta=self.beta, lut_binarize=self.lut_binarize, binary=self.binary)
        if getattr(self, "_fused", False):
            self.ops.differentiable_lut6_backward(x, dy, self.idx, self.W, self.dW, self.mean, self.rstd, self.n_in, frames, dx=dx, **kw)
            self._x = None
            return dx
        if self._y is not None and self._y.shape[1] == dy.shape[1]:
            self.ops.dl6_backward_stats_from_output(self._y, dy, self.rstd, frames, self.sums, gamma=self.gamma, beta=self.beta)
        else:
            self.ops.dl6_backward_stats(x, dy, self.idx, self.W, self.mean, self.rstd, frames, self.sums, **kw)
        self._allreduce(self.sums)
        self.ops.dl6_backward_apply(x, dy, dx, self.idx, self.W, self.dW, self.mean, self.rstd, self.sums, self.n_in, frames, total, **kw)
        self._pending = self._allreduce(self.dW, async_op=True)
        self._x = self._y = None
        return dx

    def wait_grad(self):
        if self._pending is not None:
            self._pending.wait()
            self._pending = None
        return self.dW
