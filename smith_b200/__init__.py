"""smith_b200 -- the quantized-inference path of Smith on NVIDIA B200.

Flat namespace in the manner of the reference's src/index.js: tensor creation,
the four quantization operators, profiling and device info.  Everything runs
through libsmith_cuda.so; importing this package without the built library
raises ImportError.
"""
from . import checkpoint, device, dispatch, dtype, gguf, lifecycle, pool, profile, tensor
from .checkpoint import loadQuantized, saveQuantized
from .gguf import quantizedFromGGUF
from .device import PRIVATE, SHARED, SmithError
from .lifecycle import dispose, isDisposed, retain, using, withNoAlloc
from .ops.matmul import matmul, matmul2d, matmulBatched
from .ops.quantize import (GROUP_BYTES, GROUP_SIZE, Q8_BLOCK_BYTES, Q8_BLOCK_SIZE, matmulQ4, matmulQ8,
                           quantizeQ4, quantizeQ8)
from .pool import poolDrain, poolFlush, poolStats
from .profile import benchmark, disableProfiling, enableProfiling, report, resetProfile, setPeaks
from .profile import profile as profileFn
from .tensor import create, full, ones, rand, randn, toArray, toNumpy, zeros
from .tensor import tensor as tensorFrom


def info():
    """src/index.js:117-124"""
    return {
        "device": device.deviceName(),
        "maxThreadgroupMemory": device.maxThreadgroupMemory(),
        "maxThreadsPerThreadgroup": device.maxThreadsPerThreadgroup(),
        "pool": poolStats(),
    }
