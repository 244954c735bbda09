"""-m gpu, collected last: the entry point that allocates nothing.

smith_qmatmul_static serves callers that cannot allocate device memory when
they call (all memory already handed to their own arena, a loop or callback
where cudaMalloc is off limits, or only raw device pointers and no smith
context).  It must give what smith_qmatmul gives on the tensor-core path, call
after call, although every call reuses the same built-in scratch array and
finds the previous call's contents in it."""
import numpy as np
import pytest

from gpu_util import DevBuf
from helpers import within_tolerance
from oracle import oracle as O
from smith_b200 import device

pytestmark = pytest.mark.gpu
REL = 1e-3


def _existing(kind, a, packed, K, N):
    M = a.shape[0]
    ab, bb, cb = DevBuf.of(a), DevBuf.of(packed), DevBuf(M * N * 4)
    device.qmatmul(kind, ab.handle, bb.handle, cb.handle, M, N, K, K // 32, device.PATH_TENSOR)
    device.synchronize()
    out = cb.get(np.float32).reshape(M, N)
    for b in (ab, bb, cb):
        b.free()
    return out


def _static(kind, a, packed, K, N, stream="context", check_memory=False):
    import torch
    M = a.shape[0]
    ab, bb, cb = DevBuf.of(a), DevBuf.of(packed), DevBuf(M * N * 4)
    device.upload(cb.handle, np.full(M * N, np.nan, np.float32))
    device.synchronize()
    free_before = torch.cuda.mem_get_info()[0] if check_memory else None
    device.qmatmulStatic(kind, device.devicePtr(ab.handle), device.devicePtr(bb.handle), device.devicePtr(cb.handle),
                         M, N, K, K // 32, device.stream() if stream == "context" else None)
    if stream != "context":
        torch.cuda.synchronize()                          # the legacy default stream
    device.synchronize()
    if check_memory:                                      # the call took no device memory
        assert torch.cuda.mem_get_info()[0] == free_before
    assert device.kernelStatus() == 0
    out = cb.get(np.float32).reshape(M, N)
    for b in (ab, bb, cb):
        b.free()
    return out


@pytest.mark.parametrize("kind", [4, 8])
def test_static_entry_matches_existing_entry_on_consecutive_calls(kind):
    rng = np.random.default_rng(100 + kind)
    knd = "q4" if kind == 4 else "q8"
    # two calls in a row, the second smaller so that it runs over the first one's leftovers
    for M, K, N in [(200, 2048, 384), (64, 1024, 256)]:
        w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
        a = rng.standard_normal((M, K)).astype(np.float32)
        packed = O.quantize_q4(w) if kind == 4 else O.quantize_q8(w)
        want = _existing(kind, a, packed, K, N)
        first = M == 200
        # the first call of a kernel variant sets its attributes; the free-memory check is on the second
        got = _static(kind, a, packed, K, N, check_memory=not first)
        ok, worst = within_tolerance(got, want, a, packed, K, N, knd, REL)
        assert ok, f"M={M} K={K} N={N}: worst err/bound against the existing entry point = {worst}"
        ok, worst = within_tolerance(got, O.matmul(a, packed, K, N, knd, threads=O.max_threads()), a, packed, K, N,
                                     knd, REL)
        assert ok, f"M={M} K={K} N={N}: worst err/bound against the oracle = {worst}"


def test_static_entry_on_the_default_stream():
    """stream = NULL: the legacy default stream, as a caller without a stream of its own would pass."""
    rng = np.random.default_rng(9)
    M, K, N = 96, 1024, 256
    w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    a = rng.standard_normal((M, K)).astype(np.float32)
    packed = O.quantize_q8(w)
    got = _static(8, a, packed, K, N, stream=None, check_memory=True)
    ok, worst = within_tolerance(got, O.matmul(a, packed, K, N, "q8", threads=O.host_threads()), a, packed, K, N, "q8", REL)
    assert ok, worst


def test_static_entry_refuses_what_does_not_fit():
    small = DevBuf(256)
    p = device.devicePtr(small.handle)
    with pytest.raises(device.SmithError, match="exceeds the built-in scratch"):
        device.qmatmulStatic(8, p, p, p, 4096, 64, 4096, 128, device.stream())   # 32 MiB of 16-bit activations
    with pytest.raises(device.SmithError, match="not taken"):
        device.qmatmulStatic(8, p, p, p, 64, 60, 1024, 32, device.stream())      # N % 8 != 0
    with pytest.raises(device.SmithError, match="null"):
        device.qmatmulStatic(8, None, p, p, 64, 64, 1024, 32, device.stream())
    with pytest.raises(device.SmithError):                                       # a and b must be 16-byte aligned
        device.qmatmulStatic(8, p + 4, p, p, 64, 64, 1024, 32, device.stream())
    with pytest.raises(device.SmithError):
        device.qmatmulStatic(8, p, p + 8, p, 64, 64, 1024, 32, device.stream())
    small.free()
