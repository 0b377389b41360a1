"""The allocation-free training forward against the regular one.

bbcu_fp32_DifferentiableLut6_ForwardTraining_NoAlloc exists for callers that cannot let an operator call
cudaMalloc (all device memory planned up front, or a path where cudaMalloc's implicit synchronisation is not
acceptable).  It must give what bbcu_fp32_DifferentiableLut6_ForwardTraining gives.  Two calls in a row check
that nothing of the first call survives in the shared scratch array.  This file sorts last on purpose, so a run
that stops at the first failure has already been through every other test; it also passes on its own in a
fresh process (the first call on a device does the entry point's one-time set-up).
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(abi, name, x, idx, W, frames, binary, seed_stats):
    O = idx.shape[0]
    y = torch.full((O, x.shape[1]), -7.0, dtype=torch.float32, device="cuda")
    mean = torch.empty(O, device="cuda")
    rstd = torch.empty(O, device="cuda")
    rm, rv = seed_stats[0].clone(), seed_stats[1].clone()
    abi.call(name, x.data_ptr(), y.data_ptr(), idx.data_ptr(), W.data_ptr(), mean.data_ptr(), rstd.data_ptr(), rm.data_ptr(), rv.data_ptr(),
             0.3, 0.5, 0.9, 0.25, O, frames, x.shape[1], 0, int(binary), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return y[:, :frames].cpu().numpy(), mean.cpu().numpy(), rstd.cpu().numpy(), rm.cpu().numpy(), rv.cpu().numpy()


def test_no_alloc_forward_matches_regular_forward_twice():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from binarybrain_b200 import abi
    g = torch.Generator(device="cuda").manual_seed(11)
    for call, (I, O, F, binary) in enumerate([(300, 700, 1100, False), (64, 33, 257, True)]):   # two calls in a row, different sizes
        S = (F + 7) // 8 * 8
        x = torch.rand((I, S), device="cuda", generator=g)
        idx = torch.randint(0, I, (O, 6), device="cuda", generator=g).to(torch.int32)
        W = (torch.randn((O, 64), device="cuda", generator=g) * 0.25 + 0.5).clamp_(0, 1)
        stats = (torch.rand(O, device="cuda", generator=g), torch.rand(O, device="cuda", generator=g) + 0.5)
        want = _run(abi, "bbcu_fp32_DifferentiableLut6_ForwardTraining", x, idx, W, F, binary, stats)
        got = _run(abi, "bbcu_fp32_DifferentiableLut6_ForwardTraining_NoAlloc", x, idx, W, F, binary, stats)
        amp = max(1.0, 0.3 * float(want[2].max()))
        for name, a, b in zip(("mean", "rstd", "running_mean", "running_var"), got[1:], want[1:]):
            assert np.abs(a - b).max() <= 1e-5 * max(1.0, float(np.abs(b).max())), (call, name)
        if binary:      # a binarised output may only differ where the two runs' sums differ in the last bit
            assert (got[0] != want[0]).mean() <= 1e-4
        else:
            assert np.abs(got[0] - want[0]).max() <= 1e-5 * amp, call


def test_no_alloc_forward_rejects_more_nodes_than_its_scratch_holds():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from binarybrain_b200 import abi
    L = abi.lib()
    limit = L.bbcu_fp32_DifferentiableLut6_ForwardTraining_NoAlloc_MaxNodes()
    assert limit == 65536
    t = torch.zeros(64, device="cuda")
    p = t.data_ptr()
    rc = L.bbcu_fp32_DifferentiableLut6_ForwardTraining_NoAlloc(p, p, p, p, p, p, p, p, 0.3, 0.5, 0.9, 0.25, limit + 1, 8, 8, 0, 0, None)
    assert rc == -6 and b"exceeds" in L.bbcu_b200_error_string(rc)
    torch.cuda.synchronize()
