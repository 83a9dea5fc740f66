"""darknet_b200: the XNOR-Net binarized-convolution forward path of Darknet, rebuilt for NVIDIA B200 (sm_100a).

Layout:
  csrc/      hand-written CUDA kernels and the C ABI (include/xnor_b200.h) -> libxnor_b200.so
  build.py   in-tree nvcc build of that library
  capi.py    ctypes declarations of the C ABI
  layer.py   host-side mirror of Darknet's xnor conv-layer calls over the C ABI

There is no CPU or PyTorch implementation of the path in this package: if libxnor_b200.so is
missing, every call raises.
"""
__all__ = ["capi", "layer", "build"]
