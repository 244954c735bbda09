"""ctypes binding of libsmith_cuda.so -- the role src/device.js plays in the reference.

The reference binds 26 bridge functions with bun:ffi (src/device.js:10-50) and
wraps each in a thin function (src/device.js:93-215).  This module binds the
same functions of the CUDA bridge under the same (camelCase) names, plus the
additive entry points declared in include/smith_cuda_bridge.h.

The shared library is loaded when this module is imported and import fails
loudly if it is missing: there is no CPU fallback.  The device context is
created on first use (``ctx()``), so that importing on a machine without a GPU
(for symbol checks and host-logic tests) still works.
"""
import ctypes as C
import os

import numpy as np

SHARED = 0   # src/device.js:53
PRIVATE = 1  # src/device.js:54

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libsmith_cuda.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"smith: {LIB_PATH} is missing. Build it with `python smith_b200/build.py` "
        "(nvcc, sm_100a). There is no CPU fallback.")

lib = C.CDLL(LIB_PATH)

_p, _u64, _u32, _i64, _i32 = C.c_void_p, C.c_uint64, C.c_uint32, C.c_int64, C.c_int32


class SmithTiming(C.Structure):
    """native/gpu_bridge.h:113-117"""
    _fields_ = [("gpu_start", C.c_double), ("gpu_end", C.c_double), ("gpu_ms", C.c_double)]


class SmithListItem(C.Structure):
    """include/smith_cuda_bridge.h: one product of a list (smith_qmatmul_list_create)."""
    _fields_ = [("a", _p), ("a_offset", _u64), ("b", _p), ("b_offset", _u64), ("b2", _p), ("b2_offset", _u64),
                ("c", _p), ("c_offset", _u64), ("gamma", _p), ("residual", _p), ("residual_offset", _u64),
                ("N", _u64), ("K", _u64), ("eps", C.c_float), ("reserved", _u32)]


class SmithListGather(C.Structure):
    """include/smith_cuda_bridge.h: the fused all-gather of one item of a list."""
    _fields_ = [("world", _u32), ("reserved", _u32), ("n0", _u64), ("n_total", _u64), ("rows", _p * 8)]


# name -> (restype, argtypes).  Part 1 is the table of src/device.js:10-50.
SYMBOLS = {
    "smith_init": (_p, []),
    "smith_destroy": (None, [_p]),
    "smith_device_name": (_p, [_p]),
    "smith_max_threadgroup_memory": (_u64, [_p]),
    "smith_max_threads_per_threadgroup": (_u64, [_p]),
    "smith_alloc": (_p, [_p, _u64, _u32]),
    "smith_buffer_contents": (_p, [_p]),
    "smith_buffer_length": (_u64, [_p]),
    "smith_release_buffer": (None, [_p]),
    "smith_load_library": (_p, [_p, C.c_char_p]),
    "smith_compile_source": (_p, [_p, C.c_char_p, C.POINTER(C.c_char_p)]),
    "smith_create_pipeline": (_p, [_p, _p, C.c_char_p]),
    "smith_begin": (_p, [_p]),
    "smith_set_buffer": (None, [_p, _p, _u32]),
    "smith_set_bytes": (None, [_p, _p, _u32, _u32]),
    "smith_set_threadgroup_memory": (None, [_p, _u64, _u32]),
    "smith_set_pipeline": (None, [_p, _p]),
    "smith_dispatch": (None, [_p, _u64, _u64, _u64, _u64, _u64, _u64]),
    "smith_end_sync": (None, [_p]),
    "smith_end_async": (_p, [_p]),
    "smith_wait": (None, [_p]),
    "smith_end_timed": (C.POINTER(SmithTiming), [_p]),
    "smith_allocated_size": (_u64, [_p]),
    "smith_test_release": (_i64, [_p]),
    "smith_test_release_after_use": (_i64, [_p]),
    "smith_buffer_retain_count": (_i64, [_p]),
    "smith_dispatch_sync": (None, [_p, _p, C.POINTER(_p), C.POINTER(_u32), _u32, _p, _u32, _u32,
                                   _u64, _u64, _u64, _u64, _u64, _u64]),
    # Part 2: additions
    "smith_last_error": (C.c_char_p, []),
    "smith_clear_error": (None, []),
    "smith_device_count": (_i32, []),
    "smith_init_device": (_p, [_i32]),
    "smith_device_index": (_i32, [_p]),
    "smith_stream": (_p, [_p]),
    "smith_synchronize": (_i32, [_p]),
    "smith_buffer_device_ptr": (_p, [_p]),
    "smith_buffer_make_resident": (_i32, [_p]),
    "smith_buffer_evict": (_i32, [_p]),
    "smith_wrap_device_memory": (_p, [_p, _p, _u64]),
    "smith_upload": (_i32, [_p, _u64, _p, _u64]),
    "smith_download": (_i32, [_p, _u64, _p, _u64]),
    "smith_q4_pack": (_i32, [_p, _p, _p, _u64, _u64]),
    "smith_q8_pack": (_i32, [_p, _p, _p, _u64, _u64]),
    "smith_gguf_repack": (_i32, [_p, _u32, _p, _p, _u64, _u64]),
    "smith_qmatmul": (_i32, [_p, _u32, _p, _p, _p, _u64, _u64, _u64, _u64, _u32]),
    "smith_matmul": (_i32, [_p, _u32, _p, _p, _p, _u64, _u64, _u64, _u64, _u32]),
    "smith_qmatmul_path": (_i32, [_u32, _u64, _u64, _u64]),
    "smith_qmatmul_list_create": (_p, [_p, _u32, _u64, C.POINTER(SmithListItem), _u32]),
    "smith_qmatmul_list_create_gather": (_p, [_p, _u32, _u64, C.POINTER(SmithListItem), C.POINTER(SmithListGather), _u32, _u32,
                                              _u32]),
    "smith_qmatmul_list_next_tag": (_u32, [_p]),
    "smith_qmatmul_list_run": (_i32, [_p, _p]),
    "smith_qmatmul_list_destroy": (None, [_p]),
    "smith_qmatmul_list_supports": (_i32, [_u32, _u64, _u64, _u64]),
    "smith_qmatmul_static": (_i32, [_u32, _p, _p, _p, _u64, _u64, _u64, _u64, _p]),
    "smith_ipc_export": (_i32, [_p, _p]),
    "smith_ipc_import": (_p, [_p, _p, _u64]),
    "smith_qmatmul_allgather": (_i32, [_p, _u32, _p, _p, _u64, _u64, _u64, _u64, _u64, _u64, _u32, _u32,
                                        C.POINTER(_p), C.POINTER(_p), _u32]),
    "smith_qmatmul_allgather_ex": (_i32, [_p, _u32, _p, _p, _u64, _u64, _u64, _u64, _u64, _u64, _u32, _u32,
                                           C.POINTER(_p), C.POINTER(_p), _u32, _u32]),
    "smith_allgather_wait": (_i32, [_p, _p, _p, _u64, _u64]),
    "smith_qmatmul_multi": (_i32, [_p, _u32, _p, _u32, C.POINTER(_p), C.POINTER(_p), C.POINTER(_u64), _u64, _u64, _u64]),
    "smith_qmatmul_allreduce": (_i32, [_p, _u32, _p, _p, _p, _u64, _u64, _u64, _u64, _u32, _u32, C.POINTER(_p),
                                       C.POINTER(_p)]),
    "smith_qmatmul_allreduce_state_bytes": (_u64, [_u32, _u64, _u64, _u64]),
    "smith_qgemv_tiles": (_i32, [_u32, _u64, _u64, _u64]),
    "smith_kernel_status": (_i32, [_p]),
    "smith_launch_count": (_u64, [_p]),
    "smith_graph_begin": (_i32, [_p]),
    "smith_graph_end": (_p, [_p]),
    "smith_graph_launch": (_i32, [_p, _p]),
    "smith_graph_destroy": (None, [_p]),
    "smith_fill_normal": (_i32, [_p, _p, _u64, _u64, C.c_float]),
    "smith_flush_l2": (_i32, [_p]),
}

for _name, (_res, _args) in SYMBOLS.items():
    _f = getattr(lib, _name)  # AttributeError here = the library does not export a declared symbol
    _f.restype = _res
    _f.argtypes = _args

_libc = C.CDLL(None)
_libc.free.argtypes = [C.c_void_p]
_libc.free.restype = None

PATH_AUTO, PATH_GENERIC, PATH_DECODE, PATH_TENSOR, PATH_GEMV, PATH_SKINNY = 0, 1, 2, 3, 4, 5


class SmithError(RuntimeError):
    pass


def lastError():
    return (lib.smith_last_error() or b"").decode()


def _raise(prefix):
    raise SmithError(f"smith: {prefix}: {lastError()}")


def _check(status, what):
    if status != 0:
        _raise(what)


_ctx = None


def ctx():
    """The process-wide device context (src/device.js:57-58), created on first use."""
    global _ctx
    if _ctx is None:
        c = lib.smith_init()
        if not c:
            raise SmithError("smith: failed to initialize CUDA device. NVIDIA B200 (sm_100a) GPU required. "
                             + lastError())
        _ctx = c
    return _ctx


def destroy():
    global _ctx, _shaderLib
    if _ctx is not None:
        lib.smith_destroy(_ctx)
        _ctx = None
        _shaderLib = None
        _pipelines.clear()


def selfTest():
    """The import-time release self-test of src/device.js:61-65, on request."""
    return int(lib.smith_test_release(ctx())), int(lib.smith_test_release_after_use(ctx()))


_shaderLib = None
_pipelines = {}


def shaderLib():
    """src/device.js:71-78 -- here the handle of the built-in kernel registry."""
    global _shaderLib
    if not _shaderLib:
        _shaderLib = lib.smith_load_library(ctx(), b"builtin")
        if not _shaderLib:
            raise SmithError("smith: failed to load kernel library")
    return _shaderLib


def pipeline(kernelName):
    """src/device.js:83-91"""
    p = _pipelines.get(kernelName)
    if not p:
        p = lib.smith_create_pipeline(ctx(), shaderLib(), kernelName.encode())
        if not p:
            raise SmithError(f"smith: kernel '{kernelName}' not found in shader library")
        _pipelines[kernelName] = p
    return p


# --- device info (src/device.js:95-108) ---

def deviceName():
    ptr = lib.smith_device_name(ctx())
    s = C.string_at(ptr).decode()
    _libc.free(ptr)
    return s


def maxThreadgroupMemory():
    return int(lib.smith_max_threadgroup_memory(ctx()))


def maxThreadsPerThreadgroup():
    return int(lib.smith_max_threads_per_threadgroup(ctx()))


def deviceCount():
    return int(lib.smith_device_count())


def deviceIndex():
    return int(lib.smith_device_index(ctx()))


# --- buffers (src/device.js:112-140) ---

def alloc(nbytes, mode=SHARED):
    buf = lib.smith_alloc(ctx(), int(nbytes), mode)
    if not buf:
        raise SmithError(f"smith: failed to allocate {nbytes} bytes (mode={mode})")
    return buf


def bufferContents(buffer):
    return lib.smith_buffer_contents(buffer)


def bufferLength(buffer):
    return int(lib.smith_buffer_length(buffer))


def releaseBuffer(buffer):
    for key in [k for k in _viewCache if k[0] == buffer]:
        del _viewCache[key]
    lib.smith_release_buffer(buffer)


def bufferRetainCount(buffer):
    return int(lib.smith_buffer_retain_count(buffer))


_viewCache = {}   # (buffer, bytes, dtype) -> view; pooled buffers come back many times


def viewBuffer(buffer, byteLength, dtype=np.float32):
    """Zero-copy typed view of a SHARED buffer's host memory (src/device.js:136-140)."""
    dt = np.dtype(dtype)
    key = (buffer, int(byteLength), dt.str)
    hit = _viewCache.get(key)
    if hit is not None:
        return hit
    raw = lib.smith_buffer_contents(buffer)
    if not raw:
        raise SmithError("smith: buffer has no host-visible contents (PRIVATE buffer?)")
    n = int(byteLength) // dt.itemsize
    arr = np.frombuffer((C.c_uint8 * (n * dt.itemsize)).from_address(raw), dtype=dt, count=n)
    _viewCache[key] = arr
    return arr


def devicePtr(buffer):
    return lib.smith_buffer_device_ptr(buffer)


def makeResident(buffer):
    _check(lib.smith_buffer_make_resident(buffer), "make_resident")


def evict(buffer):
    _check(lib.smith_buffer_evict(buffer), "evict")


def wrapDeviceMemory(ptr, nbytes):
    buf = lib.smith_wrap_device_memory(ctx(), ptr, int(nbytes))
    if not buf:
        _raise("wrap_device_memory")
    return buf


def upload(buffer, array, offset=0):
    a = np.ascontiguousarray(array)
    _check(lib.smith_upload(buffer, offset, a.ctypes.data_as(C.c_void_p), a.nbytes), "upload")


def download(buffer, nbytes, dtype=np.uint8, offset=0):
    out = np.empty(int(nbytes) // np.dtype(dtype).itemsize, dtype=dtype)
    _check(lib.smith_download(buffer, offset, out.ctypes.data_as(C.c_void_p), out.nbytes), "download")
    return out


# --- compute dispatch (src/device.js:144-178) ---

def begin():
    return lib.smith_begin(ctx())


def setBuffer(enc, buffer, index):
    lib.smith_set_buffer(enc, buffer, index)


def setBytes(enc, data, length, index):
    a = np.ascontiguousarray(data)
    lib.smith_set_bytes(enc, a.ctypes.data_as(C.c_void_p), int(length), index)


def setThreadgroupMemory(enc, length, index):
    lib.smith_set_threadgroup_memory(enc, length, index)


def setPipeline(enc, pipelinePtr):
    lib.smith_set_pipeline(enc, pipelinePtr)


def dispatch(enc, gridX, gridY, gridZ, groupX, groupY, groupZ):
    lib.smith_dispatch(enc, gridX, gridY, gridZ, groupX, groupY, groupZ)


def dispatchSync(pipelinePtr, buffers, indices, paramBytes, paramIndex, grid, group):
    """native/gpu_bridge.h:104-108: bind, dispatch and wait in ONE call across the FFI (the reference's JS
    table does not list it; a call costs about a microsecond here, and the encoder path makes nine)."""
    n = len(buffers)
    lib.smith_clear_error()
    lib.smith_dispatch_sync(ctx(), pipelinePtr, (_p * n)(*buffers), (_u32 * n)(*indices), n,
                            paramBytes.ctypes.data_as(C.c_void_p) if paramBytes is not None else None,
                            paramBytes.nbytes if paramBytes is not None else 0, paramIndex,
                            grid[0], grid[1], grid[2], group[0], group[1], group[2])
    if lastError():
        _raise("dispatch failed")


def endSync(enc):
    lib.smith_clear_error()
    lib.smith_end_sync(enc)
    if lastError():
        _raise("dispatch failed")


def endAsync(enc):
    lib.smith_clear_error()
    tok = lib.smith_end_async(enc)
    if not tok:
        _raise("dispatch failed")
    return tok


def wait(token):
    lib.smith_clear_error()
    lib.smith_wait(token)
    if lastError():
        _raise("wait failed")


def endTimed(enc):
    """src/device.js:182-193 -- decodes (and here also frees) the SmithTiming struct."""
    lib.smith_clear_error()
    t = lib.smith_end_timed(enc)
    if not t:
        if lastError():
            _raise("dispatch failed")
        return {"gpuStart": 0.0, "gpuEnd": 0.0, "gpuMs": 0.0}
    out = {"gpuStart": t.contents.gpu_start, "gpuEnd": t.contents.gpu_end, "gpuMs": t.contents.gpu_ms}
    _libc.free(C.cast(t, C.c_void_p))
    return out


def allocatedSize():
    return int(lib.smith_allocated_size(ctx()))


def compileSource(source):
    err = C.c_char_p()
    library = lib.smith_compile_source(ctx(), source.encode(), C.byref(err))
    if not library:
        msg = err.value.decode() if err.value else "unknown error"
        raise SmithError(f"smith: shader compilation failed: {msg}")
    return library


def createPipeline(library, fnName):
    p = lib.smith_create_pipeline(ctx(), library, fnName.encode())
    if not p:
        raise SmithError(f"smith: kernel '{fnName}' not found")
    return p


# --- additions: direct entries, graphs, utilities ---

def stream():
    return lib.smith_stream(ctx())


def synchronize():
    _check(lib.smith_synchronize(ctx()), "synchronize")


def q4Pack(wBuffer, outBuffer, K, N):
    _check(lib.smith_q4_pack(ctx(), wBuffer, outBuffer, K, N), "q4_pack")


def q8Pack(wBuffer, outBuffer, K, N):
    _check(lib.smith_q8_pack(ctx(), wBuffer, outBuffer, K, N), "q8_pack")


GGML_Q4_0, GGML_Q8_0 = 2, 8


def ggufRepack(ggmlType, srcBuffer, dstBuffer, outDim, inDim):
    _check(lib.smith_gguf_repack(ctx(), ggmlType, srcBuffer, dstBuffer, outDim, inDim), "gguf_repack")


def qmatmul(kind, aBuffer, bBuffer, cBuffer, M, N, K, groups, path=PATH_AUTO):
    _check(lib.smith_qmatmul(ctx(), kind, aBuffer, bBuffer, cBuffer, M, N, K, groups, path), "qmatmul")


DTYPE_F32, DTYPE_F16 = 0, 1
DENSE_AUTO, DENSE_GENERIC, DENSE_TENSOR, DENSE_TENSOR_FAST = 0, 1, 2, 3


def matmul(dtype, aBuffer, bBuffer, cBuffer, M, N, K, batch=1, path=DENSE_AUTO):
    """smith_matmul: the dense matmul c[batch,M,N] = a[batch,M,K] @ b[batch,K,N] on device-side buffers."""
    _check(lib.smith_matmul(ctx(), dtype, aBuffer, bBuffer, cBuffer, M, N, K, batch, path), "matmul")


def qmatmulStatic(kind, aPtr, bPtr, cPtr, M, N, K, groups, streamPtr=None):
    """smith_qmatmul_static: raw device pointers, scratch inside the library, allocates nothing."""
    _check(lib.smith_qmatmul_static(kind, aPtr, bPtr, cPtr, M, N, K, groups, streamPtr), "qmatmul_static")


def qmatmulPath(kind, M, N, K):
    return int(lib.smith_qmatmul_path(kind, M, N, K))


def ipcExport(buffer):
    """64-byte handle another process on this box can import."""
    out = C.create_string_buffer(64)
    _check(lib.smith_ipc_export(buffer, out), "ipc_export")
    return out.raw


def ipcImport(handle, nbytes):
    buf = lib.smith_ipc_import(ctx(), handle, int(nbytes))
    if not buf:
        _raise("ipc_import")
    return buf


def qgemvTiles(kind, M, N, K):
    return int(lib.smith_qgemv_tiles(kind, M, N, K))


GATHER_DEFER = 1
GATHER_INPUT_IS_PREVIOUS_ROW = 2


def qmatmulAllGather(kind, aBuffer, bBuffer, M, nTotal, n0, nLocal, K, groups, world, rank, yBuffers, stateBuffers,
                     target, flags=0):
    ys = (_p * world)(*yBuffers)
    ss = (_p * world)(*stateBuffers)
    _check(lib.smith_qmatmul_allgather_ex(ctx(), kind, aBuffer, bBuffer, M, nTotal, n0, nLocal, K, groups, world,
                                          rank, ys, ss, target, flags), "qmatmul_allgather")


def allGatherWait(stateBuffer, yBuffer, M, nTotal):
    _check(lib.smith_allgather_wait(ctx(), stateBuffer, yBuffer, M, nTotal), "allgather_wait")


def qmatmulMulti(kind, aBuffer, bBuffers, cBuffers, Ns, M, K, groups):
    """One launch for several packed matrices that share the activations (M <= 4); see the header."""
    n = len(bBuffers)
    _check(lib.smith_qmatmul_multi(ctx(), kind, aBuffer, n, (_p * n)(*bBuffers), (_p * n)(*cBuffers),
                                   (_u64 * n)(*[int(x) for x in Ns]), M, K, groups), "qmatmul_multi")


def listItem(a, b, c, N, K, b2=None, gamma=None, residual=None, eps=1e-5, aOffset=0, bOffset=0, b2Offset=0,
             cOffset=0, residualOffset=0):
    """One product of a list: c = [residual +] (b2 ? silu(x b) * (x b2) : x b), x = gamma ? rmsnorm(a) * gamma : a."""
    return SmithListItem(a, aOffset, b, bOffset, b2, b2Offset, c, cOffset, gamma, residual, residualOffset, N, K,
                         eps, 0)


def qmatmulListCreate(kind, M, items):
    """A list of GEMV-shaped products that runs as one persistent launch (see the header)."""
    arr = (SmithListItem * len(items))(*items)
    h = lib.smith_qmatmul_list_create(ctx(), kind, M, arr, len(items))
    if not h:
        _raise("qmatmul_list_create")
    return h


LIST_NO_CLOSING_WAIT = 1


def listGather(world, n0, nTotal, rowBuffers):
    """The fused all-gather of one list item: its columns are [n0, n0 + N) of a row of nTotal."""
    g = SmithListGather()
    g.world, g.n0, g.n_total = world, n0, nTotal
    for r in range(world):
        g.rows[r] = rowBuffers[r]
    return g


def qmatmulListCreateGather(kind, M, items, gathers, rank, flags=0):
    """A list whose items may end in a fused all-gather over peer memory (see the header);
    gathers[i] is None for an item that is not gathered."""
    n = len(items)
    arr = (SmithListItem * n)(*items)
    garr = (SmithListGather * n)(*[g if g is not None else SmithListGather() for g in gathers])
    h = lib.smith_qmatmul_list_create_gather(ctx(), kind, M, arr, garr, n, rank, flags)
    if not h:
        _raise("qmatmul_list_create_gather")
    return h


def qmatmulListNextTag(handle):
    return int(lib.smith_qmatmul_list_next_tag(handle))


def qmatmulListRun(handle):
    _check(lib.smith_qmatmul_list_run(ctx(), handle), "qmatmul_list_run")


def qmatmulListDestroy(handle):
    lib.smith_qmatmul_list_destroy(handle)


def qmatmulListSupports(kind, M, N, K):
    return bool(lib.smith_qmatmul_list_supports(kind, M, N, K))


def qmatmulAllReduce(kind, aBuffer, bBuffer, outBuffer, M, N, kLocal, groupsLocal, world, rank, partialBuffers,
                     stateBuffers):
    ps = (_p * world)(*partialBuffers)
    ss = (_p * world)(*stateBuffers)
    _check(lib.smith_qmatmul_allreduce(ctx(), kind, aBuffer, bBuffer, outBuffer, M, N, kLocal, groupsLocal, world,
                                       rank, ps, ss), "qmatmul_allreduce")


def qmatmulAllReduceStateBytes(kind, M, N, kLocal):
    return int(lib.smith_qmatmul_allreduce_state_bytes(kind, M, N, kLocal))


def kernelStatus():
    """1 if a bounded device-side wait gave up since the last call, else 0."""
    return int(lib.smith_kernel_status(ctx()))


def launchCount():
    return int(lib.smith_launch_count(ctx()))


def graphBegin():
    _check(lib.smith_graph_begin(ctx()), "graph_begin")


def graphEnd():
    g = lib.smith_graph_end(ctx())
    if not g:
        _raise("graph_end")
    return g


def graphLaunch(graph):
    _check(lib.smith_graph_launch(ctx(), graph), "graph_launch")


def graphDestroy(graph):
    lib.smith_graph_destroy(graph)


def fillNormal(buffer, count, seed, std):
    _check(lib.smith_fill_normal(ctx(), buffer, count, seed, std), "fill_normal")


def flushL2():
    _check(lib.smith_flush_l2(ctx()), "flush_l2")
