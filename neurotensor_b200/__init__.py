"""neurotensor_b200 -- B200-native engine for NeuroTensor's matmult / Linear / conv2d hot path.

`neurotensor_b200.api` mirrors the reference's functional interface (matmult, linear, conv2d, unfold2d, ...)
on device buffers; `neurotensor_b200._lib` is the raw C ABI.  Everything computes in hand-written CUDA for
sm_100a inside libntb200.so; PyTorch only supplies device memory, streams and torch.distributed.
"""
from . import _lib  # noqa: F401

__all__ = ["_lib", "api", "partition"]
