"""B200-native speculative-decoding verify path for yuuka (qwen35 / qwen35moe).

The product is libyuuka_cuda.so (hand-written sm_100a kernels behind the C ABI
declared in include/yuuka_cuda.h). This package holds its in-tree build, a
ctypes mirror of the ABI and the host-side runtime that mirrors the reference's
engine.SpeculativeRuntime for the verify path.
"""
__all__ = ["build", "synth"]
