"""CPU tests of the host layer: the C ABI's symbol table, and the host-side
mirror of the reference interface (pool, lifecycle, dtype, operator argument
checks).  Nothing here computes on a device."""
import ctypes
import os
import re

import numpy as np
import pytest

import smith_b200 as smith
from smith_b200 import device, lifecycle, pool
from smith_b200.ops import quantize as Q

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "smith_cuda_bridge.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(smith_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = _declared_symbols()
    assert len(names) >= 27
    lib = ctypes.CDLL(device.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/smith_cuda_bridge.h but not exported"


def test_binding_table_covers_the_header():
    assert sorted(device.SYMBOLS) == _declared_symbols()


def test_reference_ffi_names_are_all_present():
    # the 26 names bound by src/device.js:10-50, plus smith_dispatch_sync (native/gpu_bridge.h:104)
    ref = """smith_init smith_destroy smith_device_name smith_max_threadgroup_memory
    smith_max_threads_per_threadgroup smith_alloc smith_buffer_contents smith_buffer_length
    smith_release_buffer smith_load_library smith_compile_source smith_create_pipeline smith_begin
    smith_set_buffer smith_set_bytes smith_set_threadgroup_memory smith_set_pipeline smith_dispatch
    smith_end_sync smith_end_async smith_wait smith_end_timed smith_allocated_size smith_test_release
    smith_test_release_after_use smith_buffer_retain_count smith_dispatch_sync""".split()
    assert len(ref) == 27
    for n in ref:
        assert n in device.SYMBOLS


def test_calls_without_a_device_fail_cleanly():
    if device.deviceCount() > 0:
        pytest.skip("a device is present")
    assert device.lib.smith_init() is None
    assert "no CUDA device" in device.lastError()
    assert device.lib.smith_buffer_length(None) == 0
    assert device.lib.smith_buffer_retain_count(None) == -1
    assert device.lib.smith_allocated_size(None) == 0
    with pytest.raises(device.SmithError):
        device.ctx()


def test_constants_match_reference():
    assert (Q.GROUP_SIZE, Q.GROUP_BYTES, Q.Q8_BLOCK_SIZE, Q.Q8_BLOCK_BYTES) == (32, 24, 32, 34)
    assert (smith.SHARED, smith.PRIVATE) == (0, 1)


class _FakeTensor:
    def __init__(self, shape):
        self.shape, self.dtype, self.buffer = list(shape), "f32", None


@pytest.mark.parametrize("fn,name", [(Q.matmulQ4, "matmulQ4"), (Q.matmulQ8, "matmulQ8")])
def test_inner_dimension_mismatch_message(fn, name):
    # src/ops/quantize.js:75-77 and :103-105 -- raised before anything touches the device
    with pytest.raises(ValueError) as e:
        fn(_FakeTensor([2, 48]), {"buffer": None, "K": 64, "N": 8, "groups": 2})
    assert str(e.value) == f"{name}: inner dims don't match: 48 vs 64"
    with pytest.raises(ValueError):
        fn(_FakeTensor([2, 48]), Q.Quantized(buffer=None, K=64, N=8, groups=2, totalBytes=0))


def test_pool_bucketing_and_recycling():
    assert [pool.bucketSize(n) for n in (0, 1, 256, 257, 1000, 1024, 1025, 23_000_000)] == \
        [256, 256, 256, 512, 1024, 1024, 2048, 1 << 25]
    pool.poolDrain()
    made = []
    pool.setAllocFn(lambda nbytes, mode: made.append((nbytes, mode)) or ("buf", len(made)))
    try:
        a = pool.poolAlloc(1000)
        b = pool.poolAlloc(1000, smith.PRIVATE)
        assert made == [(1024, 0), (1024, 1)]
        pool.poolFree(a, 1000)
        assert pool.poolStats()["shared"] == {"count": 1, "bytes": 1024}
        assert pool.poolAlloc(700) is a          # same bucket, recycled
        assert pool.poolAlloc(700) != a          # bin empty again -> new allocation
        s = pool.poolStats()
        assert (s["hits"], s["misses"], s["totalAllocated"]) == (1, 3, 3072)
        pool.poolFree(b, 1000, smith.PRIVATE)
        assert pool.poolStats()["private"]["count"] == 1
        pool.poolFree(None, 10)                  # ignored
    finally:
        pool.setAllocFn(None)
        pool.poolDrain()


class _T:
    def __init__(self):
        self.buffer, self.data = object(), object()


def test_lifecycle_scopes_and_refcounts():
    released = []
    lifecycle.setReleaseFn(lambda t: released.append(t))
    try:
        kept = {}

        def body():
            a, b = _T(), _T()
            lifecycle.trackAllocation(a)
            lifecycle.trackAllocation(b)
            kept["b"] = lifecycle.retain(b)
            assert lifecycle.activeScopeDepth() == 1
            return a

        a = lifecycle.using(body)
        assert lifecycle.isDisposed(a) and a.buffer is None and released == [a]
        assert not lifecycle.isDisposed(kept["b"]) and kept["b"]._refCount == 1
        lifecycle.dispose(kept["b"])
        assert lifecycle.isDisposed(kept["b"]) and len(released) == 2
        lifecycle.dispose(kept["b"])             # idempotent
        assert len(released) == 2
        with pytest.raises(RuntimeError):
            lifecycle.withNoAlloc(lambda: lifecycle.trackAllocation(_T()))
        lifecycle.trackAllocation(_T())          # guard is lifted afterwards
    finally:
        from smith_b200 import tensor  # restores the pool hook
        from smith_b200.dtype import dtypeBytes
        lifecycle.setReleaseFn(lambda t: pool.poolFree(t.buffer, t.size * dtypeBytes(t.dtype), t.mode))


def test_profile_stats_shape():
    from smith_b200.profile import computeStats
    s = computeStats(sorted([1.0, 2.0, 3.0, 4.0]))
    assert s == {"mean": 2.5, "median": 2.5, "min": 1.0, "max": 4.0, "p95": 4.0, "stddev": 1.118}
    assert computeStats([])["mean"] == 0


def test_profile_algorithmic_cost_and_roofline_fields():
    """The additions to src/profile.js's report: bytes / flops per dispatch and the roofline fraction."""
    from smith_b200 import profile as P
    assert P.algorithmicCost("matmul_q4", [1, 14336, 4096, 128]) == (128 * 14336 * 24 + 4 * 4096 + 4 * 14336, 2 * 4096 * 14336)
    assert P.algorithmicCost("matmul_q8", [512, 11008, 4096, 128]) == (128 * 11008 * 34 + 4 * 512 * 4096 + 4 * 512 * 11008,
                                                                        2 * 512 * 4096 * 11008)
    assert P.algorithmicCost("quantize_q4", [100, 40]) == (4 * 100 * 40 + 4 * 40 * 24, 0)
    assert P.algorithmicCost("relu_forward", [3]) is None and P.algorithmicCost("matmul_q4", None) is None
    saved = dict(P._kernelStats), P._totalDispatches, P._totalGpuMs
    try:
        P._kernelStats.clear()
        P._totalDispatches, P._totalGpuMs = 0, 0.0
        orig = P.device.allocatedSize
        P.device.allocatedSize = lambda: 0            # no device on this machine
        P.setPeaks(8000.0, 2250.0, "nominal")
        P.recordKernel("matmul_q4", 0.01, P.algorithmicCost("matmul_q4", [1, 14336, 4096, 128]))   # 10 us
        P.recordKernel("matmul_q4", 0.01, P.algorithmicCost("matmul_q4", [1, 14336, 4096, 128]))
        P.recordKernel("other", 1.0)
        rep = P.report()
        mm = next(k for k in rep["kernels"] if k["kernel"] == "matmul_q4")
        assert abs(mm["gbs"] - 44113920 / 1e-5 / 1e9) < 1 and mm["bound"] == "hbm"
        assert abs(mm["pctRoofline"] - 100 * mm["gbs"] / 8000.0) < 0.01
        assert "gbs" not in next(k for k in rep["kernels"] if k["kernel"] == "other")
        assert rep["peaks"]["hbmGBs"] == 8000.0
    finally:
        P.device.allocatedSize = orig
        P._kernelStats.clear()
        P._kernelStats.update(saved[0])
        P._totalDispatches, P._totalGpuMs = saved[1], saved[2]


def test_dense_matmul_operator_messages_and_parameter_blocks():
    # src/ops/matmul.js:21-23, 91-93 -- raised before anything touches the device; src/dispatch.js:57-63, 92-94
    from smith_b200.ops import matmul as MM

    class _T(_FakeTensor):
        def __init__(self, shape):
            super().__init__(shape)
            self.strides = smith.tensor.computeStrides(shape)

    with pytest.raises(ValueError) as e:
        MM.matmul(_T([2, 3]), _T([4, 2]))
    assert str(e.value) == "matmul: inner dims don't match: 3 vs 4"
    with pytest.raises(ValueError) as e:
        MM.matmul(_T([3]), _T([3, 2]))
    assert str(e.value) == "matmul requires at least 2D tensors, got 1D and 2D"
    with pytest.raises(ValueError) as e:
        MM._broadcastShapes([2, 3], [4, 3])
    assert str(e.value) == "Cannot broadcast shapes [2,3] and [4,3]"
    assert MM._broadcastShapes([5, 1], [4]) == [5, 4]
    assert MM.matmulParams(3, 4, 5).tolist() == [3, 4, 5] and MM.matmulParams(3, 4, 5).dtype == np.uint32
    assert MM.batchMatmulParams(3, 4, 5, 6).tolist() == [3, 4, 5, 6]
    assert MM.k("matmul_simple", "f16") == "matmul_simple_f16" and MM.k("matmul_batched", "f32") == "matmul_batched"
    assert MM.TILE_THRESHOLD == 64
    from smith_b200 import profile as P
    assert P.algorithmicCost("matmul_f32", [64, 128, 256]) == (4 * (64 * 256 + 256 * 128 + 64 * 128), 2 * 64 * 128 * 256)
    assert P.algorithmicCost("matmul_batched_f16", [8, 16, 32, 5]) == (5 * 2 * (8 * 32 + 32 * 16 + 8 * 16), 5 * 2 * 8 * 16 * 32)
