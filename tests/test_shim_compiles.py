"""The reference-side shim, proven by compilation (no GPU).

include/bbcu_b200_shim.h defines BinaryBrain's operator declarations (include/bbcu/bbcu.h) as inline forwarders to the C ABI.
This test compiles BinaryBrain's unmodified layer headers, with BB_WITH_CUDA, against bbcu.h + the shim (tests/shim_call_sites.cpp
instantiates every member function, hence every call site) and reads the object's undefined symbols:
  * every operator of the path must have resolved to a plain C symbol that libbbcu_b200.so exports;
  * no C++-mangled (i.e. BinaryBrain-declared, still undefined) operator of the path may be left over -- the only bbcu_* names
    still undefined are the tensor arithmetic and conversion helpers outside the path, which stay with BinaryBrain's own sources.
Skipped where no BinaryBrain checkout or no CUDA headers are present.
"""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE = os.environ.get("BB_REFERENCE", "/root/reference")
CUDA_INC = os.environ.get("CUDA_INC", "/usr/local/cuda/include")
NOT_ON_THE_PATH = ("bbcu_fp32_Vector_sqrt", "bbcu_fp32_Vector_add_ex", "bbcu_fp32_Vector_sub_ex", "bbcu_fp32_Vector_mul_ex", "bbcu_fp32_Vector_div_ex")


@pytest.fixture(scope="module")
def undefined_symbols(tmp_path_factory):
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else shutil.which("g++")
    if not os.path.isdir(os.path.join(REFERENCE, "include", "bb")) or not os.path.exists(os.path.join(CUDA_INC, "cuda_runtime.h")) or not cxx:
        pytest.skip("needs a BinaryBrain checkout, the CUDA headers and g++")
    obj = str(tmp_path_factory.mktemp("shim") / "call_sites.o")
    # the reference's own flags (samples/cpp/mnist/Makefile:24,49), -O0 to keep every inline forwarder's call in the object
    cmd = [cxx, "-std=c++14", "-mavx2", "-mfma", "-fopenmp", "-O0", "-DBB_WITH_CUDA", "-c", os.path.join(ROOT, "tests", "shim_call_sites.cpp"), "-o", obj,
           "-I" + os.path.join(REFERENCE, "include"), "-I" + os.path.join(ROOT, "include"), "-I" + CUDA_INC]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-4000:]
    nm = subprocess.run(["nm", "-C", "--undefined-only", obj], capture_output=True, text=True, check=True).stdout
    return [l.split(None, 1)[1].strip() for l in nm.splitlines() if "bbcu" in l]


def test_every_call_site_resolves_to_the_c_abi(undefined_symbols):
    from binarybrain_b200 import abi
    plain = {s for s in undefined_symbols if "(" not in s}
    assert plain <= set(abi.SIGNATURES), plain - set(abi.SIGNATURES)
    must = {"bbcu_fp32_StochasticLut6_Forward", "bbcu_bit_fp32_StochasticLut6_Forward", "bbcu_bit_bit_fp32_StochasticLut6_Forward",
            "bbcu_fp32_StochasticLut6_Backward", "bbcu_bit_fp32_StochasticLut6_Backward",
            "bbcu_fp32_DifferentiableLut6_ForwardTraining", "bbcu_bit_fp32_DifferentiableLut6_ForwardTraining",
            "bbcu_fp32_DifferentiableLut6_ForwardInference", "bbcu_bit_fp32_DifferentiableLut6_ForwardInference",
            "bbcu_fp32_DifferentiableLut6_Backward", "bbcu_bit_fp32_DifferentiableLut6_Backward",
            "bbcu_fp32_StochasticBatchNormalization_ForwardTraining", "bbcu_fp32_StochasticBatchNormalization_ReForward",
            "bbcu_fp32_StochasticBatchNormalization_ForwardInference", "bbcu_fp32_StochasticBatchNormalization_Backward",
            "bbcu_bit_BinatyLut6_Forward", "bbcu_LocalHeap_Malloc", "bbcu_LocalHeap_Free", "bbcu_GetDevice", "bbcu_IsHostOnly",
            "bbcu_fp32_OptimizerAdam", "bbcu_fp32_Vector_clamp", "bbcu_fp32_ConvBitToReal", "bbcu_fp32_Im2Col_Forward", "bbcu_fp32_Col2Im_Forward", "bbcu_fp32_MaxPooling_Forward"}
    assert must <= plain, must - plain


def test_no_operator_of_the_path_is_left_to_the_reference(undefined_symbols):
    mangled = [s for s in undefined_symbols if "(" in s]
    left = [s for s in mangled if not any(n in s for n in NOT_ON_THE_PATH)]
    assert not left, left
