"""B200-native backend for SharpMind's quantized vec-dot / matmul hot path.

The compute lives in `csrc/` (hand-written sm_100a CUDA behind a C ABI declared in
`include/sharpmind_cuda.h`); this package is the host-side mirror of the reference's operator
interface for that path and loads the shared library through ctypes.
"""
__version__ = "0.1.0"
