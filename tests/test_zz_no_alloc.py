"""The allocation-free training forward against the regular one.

bbcu_fp32_DifferentiableLut6_ForwardTraining_NoAlloc exists for callers that cannot let an operator call
cudaMalloc (all device memory planned up front, or a path where cudaMalloc's implicit synchronisation is not
acceptable).  It must give what bbcu_fp32_DifferentiableLut6_ForwardTraining gives.  Two calls in a row check
that nothing of the first call survives in the shared scratch array.  This file sorts last on purpose, so a run
that stops at the first failure has already been through every other test; it also passes on its own in a
fresh process (the first call on a device does the entry point's one-time set-up).
"""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Runs in a process of its own, where the allocation-free entry point is the FIRST call into the library: nothing an earlier
# operator may have set up (heap scratch, the per-device fault word) exists yet.  The device heap is capped at one byte, so any
# request the call made of it would fail; torch allocates the tensors before the call, and the free device memory is read
# around a second call (the first one loads the library's device code, which the driver accounts as device memory).
_FRESH_PROCESS = r"""
import sys
import numpy as np
import torch
sys.path.insert(0, ROOT)
from binarybrain_b200 import abi
from oracle import port

L = abi.lib()
L.bbcu_LocalHeap_SetByteLimit(1)
rng = np.random.default_rng(21)
I, O, F = 300, 700, 1100
S = (F + 7) // 8 * 8
idx = np.stack([rng.permutation(I)[:6] for _ in range(O)]).astype(np.int32)
W = np.clip(rng.normal(0.5, 0.25, (O, 64)), 0, 1).astype(np.float32)
x = rng.random((I, F), dtype=np.float32)
rm0, rv0 = rng.random(O, dtype=np.float32), rng.random(O, dtype=np.float32) + 0.5
xd = torch.zeros((I, S)); xd[:, :F] = torch.from_numpy(x); xd = xd.cuda()
idx_d, W_d = torch.from_numpy(idx).cuda(), torch.from_numpy(W).cuda()
y = torch.full((O, S), -7.0, device="cuda")
mean, rstd = torch.empty(O, device="cuda"), torch.empty(O, device="cuda")
rm, rv = torch.from_numpy(rm0).cuda(), torch.from_numpy(rv0).cuda()
rm2, rv2 = rm.clone(), rv.clone()
torch.cuda.synchronize()

def call(rm_t, rv_t):
    rc = L.bbcu_fp32_DifferentiableLut6_ForwardTraining_NoAlloc(xd.data_ptr(), y.data_ptr(), idx_d.data_ptr(), W_d.data_ptr(), mean.data_ptr(),
                                                                rstd.data_ptr(), rm_t.data_ptr(), rv_t.data_ptr(), 0.3, 0.5, 0.9, 0.25, O, F, S, 0, 0,
                                                                torch.cuda.current_stream().cuda_stream)
    assert rc == 0, L.bbcu_b200_error_string(rc)
    torch.cuda.synchronize()

call(rm, rv)
assert L.bbcu_LocalHeap_GetAllocatedSize() == 0 and L.bbcu_LocalHeap_GetMaxAllocSize() == 0
free_before = torch.cuda.mem_get_info()[0]
call(rm2, rv2)
assert torch.cuda.mem_get_info()[0] == free_before, "device memory changed across a call"
assert L.bbcu_LocalHeap_GetAllocatedSize() == 0 and L.bbcu_LocalHeap_GetMaxAllocSize() == 0
assert L.bbcu_b200_device_fault() == 0
p = port.dl6_forward_train(x, idx, W, rm0, rv0, binary=False)
amp = max(1.0, 0.3 * float(p["rstd"].max()))
assert np.abs(mean.cpu().numpy() - p["mean"]).max() <= 1e-5
assert np.abs(rm.cpu().numpy() - p["running_mean"]).max() <= 1e-5 and np.abs(rv.cpu().numpy() - p["running_var"]).max() <= 1e-5
assert np.abs(y[:, :F].cpu().numpy() - p["y"]).max() <= 3e-5 * amp
print("fresh-process no-alloc ok")
"""


def test_no_alloc_forward_first_call_of_a_fresh_process_allocates_nothing_and_matches_the_oracle():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    r = subprocess.run([sys.executable, "-c", _FRESH_PROCESS.replace("ROOT", repr(ROOT))], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "fresh-process no-alloc ok" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


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
