"""Device-backed tensors -- the part of src/tensor.js the quantized path uses.

A tensor is the reference's plain record (src/tensor.js:62-71): ``buffer`` (an
opaque bridge handle), ``data`` (a typed view of the buffer's host memory, None
for PRIVATE tensors), ``shape``, ``strides``, ``dtype``, ``size``, ``offset``,
``mode``.  Creation goes through the pool and registers with the lifecycle
scopes exactly as src/tensor.js:55-74 does.
"""
import numpy as np

from . import device
from .dtype import dtypeArray, dtypeBytes, fromFloat16, toFloat16
from .lifecycle import setReleaseFn, trackAllocation
from .pool import poolAlloc, poolFree

setReleaseFn(lambda t: poolFree(t.buffer, t.size * dtypeBytes(t.dtype), t.mode))

_rng = np.random.default_rng()


def seed(n):
    """Seed rand/randn (the reference draws from unseeded Math.random)."""
    global _rng
    _rng = np.random.default_rng(n)


class Tensor:
    __slots__ = ("buffer", "data", "shape", "strides", "dtype", "size", "offset", "mode",
                 "_refCount", "_disposed")

    def __repr__(self):
        return f"tensor(shape={self.shape}, dtype={self.dtype})"


def computeStrides(shape):
    strides = [0] * len(shape)
    stride = 1
    for i in range(len(shape) - 1, -1, -1):
        strides[i] = stride
        stride *= shape[i]
    return strides


def shapeSize(shape):
    s = 1
    for d in shape:
        s *= d
    return s


def create(shape, dtype="f32", mode=device.SHARED):
    """src/tensor.js:55-74"""
    size = shapeSize(shape)
    nbytes = size * dtypeBytes(dtype)
    t = Tensor()
    t._refCount = None
    t._disposed = False
    t.buffer = poolAlloc(nbytes, mode)
    t.data = device.viewBuffer(t.buffer, nbytes, dtypeArray(dtype)) if mode == device.SHARED else None
    t.shape = list(shape)
    t.strides = computeStrides(shape)
    t.dtype = dtype
    t.size = size
    t.offset = 0
    t.mode = mode
    trackAllocation(t)
    return t


def tensor(values, shape, dtype="f32"):
    """src/tensor.js:77-86"""
    t = create(shape, dtype)
    flat = np.asarray(values).reshape(-1)
    if dtype == "f16":
        for i in range(t.size):
            t.data[i] = toFloat16(flat[i] if i < flat.size else 0)
    else:
        n = min(flat.size, t.size)
        t.data[:n] = flat[:n]
        t.data[n:] = 0
    return t


def zeros(shape, dtype="f32"):
    t = create(shape, dtype)
    if t.data is not None:
        t.data[:] = 0
    return t


def full(shape, value, dtype="f32"):
    t = create(shape, dtype)
    t.data[:] = toFloat16(value) if dtype == "f16" else value
    return t


def ones(shape, dtype="f32"):
    return full(shape, 1.0, dtype)


def rand(shape, dtype="f32"):
    """Uniform [0,1) on the host (src/tensor.js:115-124)."""
    t = create(shape, dtype)
    v = _rng.random(t.size)
    if dtype == "f16":
        for i in range(t.size):
            t.data[i] = toFloat16(v[i])
    else:
        t.data[:] = v
    return t


def randn(shape, dtype="f32"):
    """Standard normal on the host (src/tensor.js:126-146)."""
    t = create(shape, dtype)
    v = _rng.standard_normal(t.size)
    if dtype == "f16":
        for i in range(t.size):
            t.data[i] = toFloat16(v[i])
    else:
        t.data[:] = v
    return t


def toArray(t):
    """Nested lists of Python floats (src/tensor.js:163-184)."""
    if t.data is None:
        raise RuntimeError("Cannot read from private (GPU-only) tensor")
    if t.dtype == "f16":
        flat = np.array([fromFloat16(int(h)) for h in t.data[:t.size]])
    else:
        flat = np.asarray(t.data[:t.size])
    if len(t.shape) == 0:
        return flat[0].item()
    return flat.reshape(t.shape).tolist()


def toNumpy(t):
    """The tensor's values as a numpy array of its shape (a copy)."""
    if t.data is None:
        raise RuntimeError("Cannot read from private (GPU-only) tensor")
    return np.array(t.data[:t.size]).reshape(t.shape)


def byteSize(t):
    return t.size * dtypeBytes(t.dtype)


def release(t):
    """src/tensor.js:192-198"""
    if t.buffer:
        poolFree(t.buffer, t.size * dtypeBytes(t.dtype), t.mode)
        t.buffer = None
        t.data = None


def isContiguous(t):
    return list(t.strides) == computeStrides(t.shape)
