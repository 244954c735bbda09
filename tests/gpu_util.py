"""Helpers for the -m gpu tests: thin wrappers that move numpy arrays through
the C ABI (PRIVATE buffers + upload/download) and call the direct entries."""
import numpy as np

from smith_b200 import device


class DevBuf:
    """A PRIVATE bridge buffer that releases itself."""

    def __init__(self, nbytes):
        self.nbytes = int(nbytes)
        self.handle = device.alloc(max(self.nbytes, 1), device.PRIVATE)

    @classmethod
    def of(cls, array):
        a = np.ascontiguousarray(array)
        b = cls(a.nbytes)
        if a.nbytes:
            device.upload(b.handle, a)
        return b

    def get(self, dtype=np.uint8, nbytes=None):
        return device.download(self.handle, self.nbytes if nbytes is None else nbytes, dtype)

    def free(self):
        if self.handle:
            device.releaseBuffer(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def pack_on_device(w, kind):
    """f32 [K,N] -> packed bytes produced by the CUDA packer."""
    K, N = w.shape
    bb = 24 if kind == "q4" else 34
    wb = DevBuf.of(w.astype(np.float32))
    ob = DevBuf(((K + 31) // 32) * N * bb)
    (device.q4Pack if kind == "q4" else device.q8Pack)(wb.handle, ob.handle, K, N)
    device.synchronize()
    out = ob.get()
    wb.free()
    ob.free()
    return out


def matmul_on_device(a, packed, K, N, kind, path=device.PATH_AUTO, groups=None):
    """C = A x dequant(packed) through smith_qmatmul on device-resident buffers."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    M = a.shape[0]
    groups = (K + 31) // 32 if groups is None else groups
    ab, bb, cb = DevBuf.of(a), DevBuf.of(packed), DevBuf(M * N * 4)
    device.qmatmul(4 if kind == "q4" else 8, ab.handle, bb.handle, cb.handle, M, N, K, groups, path)
    device.synchronize()
    assert device.kernelStatus() == 0, "a bounded device-side wait gave up"
    out = cb.get(np.float32).reshape(M, N)
    for b in (ab, bb, cb):
        b.free()
    return out
