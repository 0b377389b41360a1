"""ctypes view of the C ABI declared in include/bbcu_b200.h.

This is the one place the library is loaded; there is no fallback: a missing or unloadable
``libbbcu_b200.so`` raises ImportError here, and a non-zero status from any entry point raises
``BbcuError``.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("BBCU_B200_LIB") or os.path.join(_HERE, "lib", "libbbcu_b200.so")

_vp, _i, _f, _ll, _sz = C.c_void_p, C.c_int, C.c_float, C.c_longlong, C.c_size_t

# name -> (restype, argtypes); pointers are passed as integers (device addresses)
SIGNATURES = {
    "bbcu_b200_error_string": (C.c_char_p, [_i]),
    "bbcu_b200_abi_version": (_i, []),
    "bbcu_b200_device_fault": (_i, []),
    "bbcu_b200_selftest_wait_expiry": (_i, [_vp]),
    "bbcu_GetDeviceCount": (_i, []),
    "bbcu_GetDevice": (_i, []),
    "bbcu_SetDevice": (None, [_i]),
    "bbcu_SetHostOnly": (None, [_i]),
    "bbcu_IsHostOnly": (_i, []),
    "bbcu_IsDeviceAvailable": (_i, []),
    "bbcu_LocalHeap_Malloc": (_vp, [_sz]),
    "bbcu_LocalHeap_Free": (None, [_vp]),
    "bbcu_LocalHeap_GetMaxAllocSize": (_sz, []),
    "bbcu_LocalHeap_GetAllocatedSize": (_sz, []),
    "bbcu_LocalHeap_GarbageCollect": (None, []),
    "bbcu_LocalHeap_SetByteLimit": (None, [_sz]),
    "bbcu_fp32_StochasticLut6_Forward": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _vp]),
    "bbcu_bit_fp32_StochasticLut6_Forward": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _vp]),
    "bbcu_bit_bit_fp32_StochasticLut6_Forward": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _vp]),
    "bbcu_fp32_StochasticLut6_Backward": (_i, [_vp] * 8 + [_i] * 9 + [_f, _vp]),
    "bbcu_bit_fp32_StochasticLut6_Backward": (_i, [_vp] * 8 + [_i] * 9 + [_f, _vp]),
    "bbcu_fp32_DifferentiableLut6_ForwardTraining": (_i, [_vp] * 8 + [_f] * 4 + [_i] * 5 + [_vp]),
    "bbcu_bit_fp32_DifferentiableLut6_ForwardTraining": (_i, [_vp] * 8 + [_f] * 4 + [_i] * 4 + [_vp]),
    "bbcu_fp32_DifferentiableLut6_ForwardInference": (_i, [_vp] * 6 + [_f] * 3 + [_i] * 5 + [_vp]),
    "bbcu_bit_fp32_DifferentiableLut6_ForwardInference": (_i, [_vp] * 6 + [_f] * 3 + [_i] * 4 + [_vp]),
    "bbcu_fp32_DifferentiableLut6_Backward": (_i, [_vp] * 12 + [_f] * 3 + [_i] * 9 + [_vp]),
    "bbcu_bit_fp32_DifferentiableLut6_Backward": (_i, [_vp] * 12 + [_f] * 3 + [_i] * 9 + [_vp]),
    "bbcu_fp32_StochasticBatchNormalization_ForwardTraining": (_i, [_vp] * 6 + [_f] * 3 + [_i] * 3 + [_vp]),
    "bbcu_fp32_StochasticBatchNormalization_ReForward": (_i, [_vp] * 4 + [_f] * 2 + [_i] * 3 + [_vp]),
    "bbcu_fp32_StochasticBatchNormalization_ForwardInference": (_i, [_vp] * 4 + [_f] * 2 + [_i] * 3 + [_vp]),
    "bbcu_fp32_StochasticBatchNormalization_Backward": (_i, [_vp] * 5 + [_f] * 2 + [_i] * 4 + [_vp]),
    "bbcu_bit_BinaryLut6_Forward": (_i, [_vp] * 4 + [_i] * 3 + [_vp]),
    "bbcu_bit_BinatyLut6_Forward": (_i, [_vp] * 4 + [_i] * 3 + [_vp]),
    "bbcu_bit_BinaryLut6_Forward_Lop3Immediate": (_i, [_vp] * 4 + [_i] * 3 + [_vp]),
    "bbcu_host_bit_BinaryLut6_Forward": (_i, [_vp] * 4 + [_i] * 4),
    "bbcu_b200_host_alloc": (_vp, [_sz]),
    "bbcu_b200_host_free": (None, [_vp]),
    "bbcu_int32_FrameBufferCopy": (_i, [_vp, _vp] + [_i] * 8 + [_vp]),
    "bbcu_fp32_ConvBitToReal": (_i, [_vp, _vp, _f, _f] + [_i] * 4 + [_vp]),
    "bbcu_fp32_Vector_clamp": (_i, [_vp, _vp, _f, _f, _i, _vp]),
    "bbcu_fp32_Vector_set": (_i, [_vp, _f, _i, _vp]),
    "bbcu_fp32_OptimizerAdam": (_i, [_i] + [_vp] * 5 + [_f] * 3 + [_vp]),
    "bbcu_fp32_LossSoftmaxCrossEntropy": (_i, [_vp] * 4 + [_f] + [_i] * 4 + [_vp]),
    "bbcu_fp32_LossMeanSquaredError": (_i, [_vp] * 4 + [_i] * 4 + [_f, C.c_double, _vp]),
    "bbcu_fp32_Reduce_Forward": (_i, [_vp] * 2 + [_i] * 5 + [_vp]),
    "bbcu_fp32_Reduce_Backward": (_i, [_vp] * 2 + [_i] * 5 + [_vp]),
    "bbcu_bit_fp32_RealToBinary_Forward": (_i, [_vp, _vp, _vp, _i, C.c_uint, C.c_uint, _f, _f] + [C.c_uint] * 5 + [_vp]),
    "bbcu_bit_fp32_BinaryToReal_Forward": (_i, [_vp, _vp] + [_i] * 6 + [_vp]),
    "bbcu_fp32_BinaryToReal_Forward": (_i, [_vp, _vp] + [_i] * 6 + [_vp]),
    "bbcu_fp32_BinaryToReal_Backward": (_i, [_vp, _vp] + [_i] * 6 + [_vp]),
    "bbcu_fp32_Im2Col_Forward": (_i, [_vp, _vp] + [_i] * 15 + [_f, _vp]),
    "bbcu_bit_Im2Col_Forward": (_i, [_vp, _vp] + [_i] * 15 + [_vp]),
    "bbcu_fp32_Im2Col_Backward": (_i, [_vp, _vp] + [_i] * 14 + [_vp]),
    "bbcu_fp32_Col2Im_Forward": (_i, [_vp, _vp] + [_i] * 6 + [_vp]),
    "bbcu_bit_Col2Im_Forward": (_i, [_vp, _vp] + [_i] * 6 + [_vp]),
    "bbcu_fp32_Col2Im_Backward": (_i, [_vp, _vp] + [_i] * 6 + [_vp]),
    "bbcu_fp32_MaxPooling_Forward": (_i, [_vp] * 3 + [_i] * 9 + [_vp]),
    "bbcu_bit_MaxPooling_Forward": (_i, [_vp] * 2 + [_i] * 9 + [_vp]),
    "bbcu_fp32_MaxPooling_Backward": (_i, [_vp] * 3 + [_i] * 9 + [_vp]),
    "bbcu_bit_fp32_MaxPooling_Backward": (_i, [_vp] * 3 + [_i] * 10 + [_vp]),
    "bbcu_fp32_DifferentiableLut6_ForwardStats": (_i, [_vp] * 5 + [_f] + [_i] * 5 + [_vp]),
    "bbcu_fp32_DifferentiableLut6_ForwardNormalize": (_i, [_vp] * 6 + [_f] * 3 + [_i] * 3 + [_ll, _i, _vp]),
    "bbcu_fp32_DifferentiableLut6_BackwardStats": (_i, [_vp] * 7 + [_f] * 3 + [_i] * 5 + [_vp]),
    "bbcu_fp32_DifferentiableLut6_ForwardTraining_NoAlloc": (_i, [_vp] * 8 + [_f] * 4 + [_i] * 5 + [_vp]),
    "bbcu_fp32_DifferentiableLut6_ForwardTraining_NoAlloc_MaxNodes": (_i, []),
    "bbcu_fp32_DifferentiableLut6_BackwardStatsFromOutput": (_i, [_vp] * 4 + [_f] * 2 + [_i] * 4 + [_vp]),
    "bbcu_fp32_DifferentiableLut6_BackwardApply": (_i, [_vp] * 11 + [_f] * 3 + [_i] * 4 + [_ll, _i, _i, _vp]),
}


class BbcuError(RuntimeError):
    def __init__(self, name, status, text):
        super().__init__(f"{name} failed with status {status}: {text}")
        self.status = status


def load(path=LIB_PATH):
    if not os.path.exists(path):
        raise ImportError(f"{path} is missing: build it with `python -m binarybrain_b200.build` "
                          "(there is no CPU fallback for the bbcu_* operators)")
    lib = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        if not hasattr(lib, name):
            continue                      # optional symbols are checked by their callers
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = load()
    return _lib


def call(name, *args):
    """Calls an int-returning entry point and raises BbcuError on a non-zero status."""
    L = lib()
    status = getattr(L, name)(*args)
    if status != 0:
        raise BbcuError(name, status, L.bbcu_b200_error_string(status).decode())
    return status
