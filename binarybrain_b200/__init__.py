"""B200-native implementation of BinaryBrain's 6-input LUT layer hot path.

``binarybrain_b200.abi``   ctypes view of the C ABI (include/bbcu_b200.h -> lib/libbbcu_b200.so)
``binarybrain_b200.ops``   the bbcu_* operators on torch CUDA tensors (device memory + streams only)
``binarybrain_b200.core``  pybind11 module: bb::FrameBuffer, bb::DifferentiableLutN<6>, ... host classes in C++
``binarybrain_b200.dist``  frame-sharded data-parallel layer over torch.distributed
"""
__version__ = "0.1.0"
