"""matmul / matmul2d / matmulBatched -- the operators of src/ops/matmul.js.

Same names, arguments, choice of kernel and error text as the reference
(src/ops/matmul.js:13-107).  ``matmul2d`` dispatches the tiled kernel's name
(``matmul_f32`` / ``matmul_f16``) when M, N and K are all at least 64 and the
simple kernel's name otherwise (src/ops/matmul.js:10,28-52); ``matmulBatched``
dispatches ``matmul_batched[_f16]`` (src/ops/matmul.js:60-87).  What changes
is behind the names: the tiled name runs on the tensor cores (f32 storage as
three bf16 planes and six partial products per k-block), the simple and batched
names on a CUDA-core kernel that keeps the shaders' order of operations bit
for bit.
"""
import numpy as np

from .. import tensor as T
from ..dispatch import run

TILE_THRESHOLD = 64    # src/ops/matmul.js:10


def k(baseName, dtype):
    """src/dispatch.js:92-94"""
    return baseName + "_f16" if dtype == "f16" else baseName


def matmulParams(M, N, K):
    """src/dispatch.js:57-59"""
    return np.array([M, N, K], dtype=np.uint32)


def batchMatmulParams(M, N, K, batch):
    """src/dispatch.js:61-63"""
    return np.array([M, N, K, batch], dtype=np.uint32)


def _contiguous(t):
    # the reference copies strided views (src/ops/matmul.js:15-16); tensors of this package have no views
    if not T.isContiguous(t):
        raise ValueError("matmul: tensors must be contiguous")
    return t


def matmul2d(a_, b_):
    """C[M,N] = A[M,K] @ B[K,N]  (src/ops/matmul.js:13-58)."""
    a, b = _contiguous(a_), _contiguous(b_)
    M, K = a.shape[-2], a.shape[-1]
    N = b.shape[-1]
    if K != b.shape[-2]:
        raise ValueError(f"matmul: inner dims don't match: {K} vs {b.shape[-2]}")
    out = T.create([M, N], a.dtype)
    params = matmulParams(M, N, K)
    bufs = [{"buffer": a.buffer, "index": 0}, {"buffer": b.buffer, "index": 1}, {"buffer": out.buffer, "index": 2}]
    if M >= TILE_THRESHOLD and N >= TILE_THRESHOLD and K >= TILE_THRESHOLD:
        groupsX, groupsY = -(-N // 32), -(-M // 32)
        run("matmul_f16" if a.dtype == "f16" else "matmul_f32", bufs, {"x": groupsX * 64, "y": groupsY},
            {"x": 64, "y": 1}, {"data": params, "index": 3})
    else:
        run(k("matmul_simple", a.dtype), bufs, {"x": N, "y": M}, {"x": min(N, 16), "y": min(M, 16)},
            {"data": params, "index": 3})
    return out


def matmulBatched(a_, b_, batchSize):
    """C[B,M,N] = A[B,M,K] @ B[B,K,N]  (src/ops/matmul.js:60-87)."""
    a, b = _contiguous(a_), _contiguous(b_)
    M, K = a.shape[-2], a.shape[-1]
    N = b.shape[-1]
    out = T.create(list(a.shape[:-2]) + [M, N], a.dtype)
    params = batchMatmulParams(M, N, K, batchSize)
    run(k("matmul_batched", a.dtype), [
        {"buffer": a.buffer, "index": 0},
        {"buffer": b.buffer, "index": 1},
        {"buffer": out.buffer, "index": 2},
    ], {"x": N, "y": M, "z": batchSize}, {"x": min(N, 16), "y": min(M, 16), "z": 1}, {"data": params, "index": 3})
    return out


def _broadcastShapes(a, b):
    """src/tensor.js:32-44"""
    out = []
    for i in range(max(len(a), len(b))):
        da = a[len(a) - 1 - i] if i < len(a) else 1
        db = b[len(b) - 1 - i] if i < len(b) else 1
        if da != db and da != 1 and db != 1:
            raise ValueError(f"Cannot broadcast shapes [{','.join(map(str, a))}] and [{','.join(map(str, b))}]")
        out.insert(0, max(da, db))
    return out


def matmul(a, b):
    """2-D or batched matmul (src/ops/matmul.js:90-107); batch dims must match, as in the reference."""
    if len(a.shape) < 2 or len(b.shape) < 2:
        raise ValueError(f"matmul requires at least 2D tensors, got {len(a.shape)}D and {len(b.shape)}D")
    if len(a.shape) == 2 and len(b.shape) == 2:
        return matmul2d(a, b)
    batchShape = _broadcastShapes(list(a.shape[:-2]), list(b.shape[:-2]))
    return matmulBatched(a, b, T.shapeSize(batchShape))
