"""GGUF weight tensors on the quantized path -- what src/gguf.js and src/gguf_loader.js do through f32.

The reference de-quantises every GGUF tensor to f32 on the host (src/gguf.js:343-400), transposes
weight matrices from GGUF's [outDim, inDim] to [inDim, outDim] (src/gguf_loader.js:236-252) and runs
the f32 matmul.  For Q8_0 and Q4_0 tensors the blocks can instead go to the device as they lie in the
file and be re-tiled there into the layouts matmulQ8 / matmulQ4 read (smith_gguf_repack): Q8_0 blocks
are byte for byte matmul_q8's blocks; a Q4_0 block is matmul_q4's block with zero = 8.
"""
import numpy as np

from . import device
from .ops.quantize import GROUP_BYTES, Q8_BLOCK_BYTES, Quantized

GGML_Q4_0, GGML_Q8_0 = device.GGML_Q4_0, device.GGML_Q8_0    # src/gguf.js:17-19
_BLOCK = {GGML_Q4_0: (18, GROUP_BYTES, "q4"), GGML_Q8_0: (34, Q8_BLOCK_BYTES, "q8")}   # src/gguf.js:32-34


def quantizedFromGGUF(blocks, ggmlType, shape):
    """``blocks``: the tensor's raw bytes from the file (uint8), ``shape`` = [outDim, inDim] as GGUF
    gives it.  Returns (kind, record) with record = {buffer, K = inDim, N = outDim, groups, totalBytes}
    ready for matmulQ4 / matmulQ8: y[M, outDim] = x[M, inDim] @ W^T, the product the reference
    computes after transposing."""
    if ggmlType not in _BLOCK:
        raise ValueError(f"quantizedFromGGUF: ggml type {ggmlType} is not read directly by the quantized kernels "
                         "(Q4_0 = 2 and Q8_0 = 8 are)")
    outDim, inDim = int(shape[0]), int(shape[1])
    if inDim % 32:
        raise ValueError(f"quantizedFromGGUF: inDim = {inDim} is not a multiple of 32")
    srcBytes, dstBytes, kind = _BLOCK[ggmlType]
    groups = inDim // 32
    raw = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    if raw.size != outDim * groups * srcBytes:
        raise ValueError(f"quantizedFromGGUF: {raw.size} bytes, expected {outDim * groups * srcBytes}")
    src = device.alloc(raw.size, device.PRIVATE)
    device.upload(src, raw)
    total = groups * outDim * dstBytes
    dst = device.alloc(total, device.PRIVATE)
    device.ggufRepack(ggmlType, src, dst, outDim, inDim)
    device.synchronize()
    device.releaseBuffer(src)
    return kind, Quantized(buffer=dst, K=inDim, N=outDim, groups=groups, totalBytes=total)
