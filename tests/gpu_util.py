"""Helpers shared by the GPU parity tests: seeded inputs, host<->device moves, dtype plumbing."""
import numpy as np
import torch

NP_TO_TORCH = {np.dtype(np.float32): torch.float32, np.dtype(np.float16): torch.float16, np.dtype(np.int8): torch.int8,
               np.dtype(np.int16): torch.int16, np.dtype(np.int32): torch.int32, np.dtype(np.int64): torch.int64,
               np.dtype(np.float64): torch.float64, np.dtype(np.uint8): torch.uint8}


def dev(arr, bf16=False):
    """numpy -> cuda tensor.  bf16 operands travel as uint16 bit patterns on the numpy side."""
    if bf16:
        return torch.from_numpy(arr.view(np.int16).copy()).cuda().view(torch.bfloat16)
    return torch.from_numpy(np.ascontiguousarray(arr)).cuda()


def host(t):
    """cuda tensor -> numpy (bf16 comes back as uint16 bit patterns)."""
    torch.cuda.synchronize()
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    return t.contiguous().cpu().numpy()


def normal(rng, shape, dtype, scale=1.0):
    return (rng.standard_normal(shape) * scale).astype(dtype)


def integers(rng, shape, dtype, lo, hi):
    return rng.integers(lo, hi, size=shape, endpoint=True).astype(dtype)
