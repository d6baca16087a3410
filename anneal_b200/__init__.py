"""anneal_b200: a B200-native device backend for the anneal tensor compiler.

``csrc/`` holds the CUDA runtime, code generator and kernels behind the C ABI in
``include/anneal_cuda.h``; the Python modules are the caller side (tensor graph,
autodiff, scheduler) that produces the kernels the device executes, and the
``ctypes`` binding of the device.
"""
