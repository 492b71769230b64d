"""B200-native (sm_100a) backend for the ternary expert GEMM of Vedant-Sood/DeepSeekTernarized.

Layout:
  csrc/            hand-written CUDA kernels and the C-ABI library (see include/dst_b200.h)
  _lib.py          in-tree nvcc build and ctypes loader
  kernels/         drop-in for the reference's boilerplate/kernels/ternary_cuda.py call surface
  ternary/         drop-in for boilerplate/ternary/pack.py and ops.py (PackedTerm, TernaryLinear)
  moe.py           the MoE routed-expert layer (single GPU and expert-parallel)
"""

__version__ = "0.1.0"
