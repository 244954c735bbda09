"""quantizeQ4 / quantizeQ8 / matmulQ4 / matmulQ8 -- the operators of src/ops/quantize.js.

Same names, arguments, return records and error text as the reference
(src/ops/quantize.js:14-68, 71-90, 99-118).  What changes is where the work
runs: ``quantizeQ4`` no longer packs on the host in a scalar loop but dispatches
the ``quantize_q4`` kernel, which produces the identical bytes on the device
and leaves them in device memory, where the matmul kernels stream them.
``quantizeQ8`` is new: the reference consumes the Q8 layout
(shaders/matmul_q8.metal) but never produces it.
"""
import numpy as np

from .. import device
from .. import tensor as T
from ..dispatch import run

GROUP_SIZE = 32        # src/ops/quantize.js:9
GROUP_BYTES = 24       # src/ops/quantize.js:10
Q8_BLOCK_SIZE = 32     # src/ops/quantize.js:94
Q8_BLOCK_BYTES = 34    # src/ops/quantize.js:95


class Quantized(dict):
    """The record {buffer, K, N, groups, totalBytes} (src/ops/quantize.js:67),
    readable both as a mapping and through attributes."""
    __getattr__ = dict.__getitem__


def _field(obj, name):
    return obj[name] if isinstance(obj, dict) else getattr(obj, name)


def _quantize(weight, kernel, groupSize, blockBytes):
    K, N = weight.shape
    groups = -(-K // groupSize)
    totalBytes = groups * N * blockBytes
    # Un-pooled, like the reference's device.alloc at src/ops/quantize.js:63,
    # but device-only: the packed weights are written and read on the device.
    buffer = device.alloc(totalBytes, device.PRIVATE)
    params = np.array([K, N], dtype=np.uint32)
    run(kernel, [
        {"buffer": weight.buffer, "index": 0},
        {"buffer": buffer, "index": 1},
    ], {"x": N, "y": groups}, {"x": min(N, 256), "y": 1}, {"data": params, "index": 2})
    return Quantized(buffer=buffer, K=K, N=N, groups=groups, totalBytes=totalBytes)


def quantizeQ4(weight):
    """Pack a 2-D f32 weight [K, N] into 24-byte Q4 blocks (src/ops/quantize.js:14-68)."""
    return _quantize(weight, "quantize_q4", GROUP_SIZE, GROUP_BYTES)


def quantizeQ8(weight):
    """Pack a 2-D f32 weight [K, N] into the 34-byte blocks matmulQ8 reads."""
    return _quantize(weight, "quantize_q8", Q8_BLOCK_SIZE, Q8_BLOCK_BYTES)


def _matmul(name, kernel, a, bQuant):
    M = a.shape[0]
    N, K, groups, bBuffer = (_field(bQuant, f) for f in ("N", "K", "groups", "buffer"))
    if a.shape[1] != K:
        raise ValueError(f"{name}: inner dims don't match: {a.shape[1]} vs {K}")
    out = T.create([M, N], a.dtype)
    params = np.array([M, N, K, groups], dtype=np.uint32)
    run(kernel, [
        {"buffer": a.buffer, "index": 0},
        {"buffer": bBuffer, "index": 1},
        {"buffer": out.buffer, "index": 2},
    ], {"x": N, "y": M}, {"x": min(N, 16), "y": min(M, 16)}, {"data": params, "index": 3})
    return out


def matmulQ4(a, bQuant):
    """C[M,N] = A[M,K](f32) @ B[K,N](q4)  (src/ops/quantize.js:71-90)."""
    return _matmul("matmulQ4", "matmul_q4", a, bQuant)


def matmulQ8(a, bQuant):
    """C[M,N] = A[M,K](f32) @ B[K,N](q8)  (src/ops/quantize.js:99-118)."""
    return _matmul("matmulQ8", "matmul_q8", a, bQuant)
