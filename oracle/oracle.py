"""ctypes front-end of the CPU checkers.  TEST INFRASTRUCTURE ONLY.

Loads ``oracle/liboracle.so`` (this repository's C restatement of the
reference's quantizeQ4 / matmul_q4 / matmul_q8 arithmetic plus the build-defined
quantizeQ8) and, when it has been built, ``oracle/_ref/libsmith_ref.so`` (the
reference's own shader source compiled as C++).  Nothing in the shipped package
imports this module: it is the checker for the tests, the smoke check and the
benchmark's CPU-baseline leg.

Reference locations restated by the C side: src/ops/quantize.js:14-68,
src/dtype.js:29-79, shaders/matmul_q4.metal:24-65, shaders/matmul_q8.metal:20-57.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "liboracle.so")
_REF = os.path.join(_HERE, "_ref", "libsmith_ref.so")

Q4_GROUP, Q4_BYTES = 32, 24
Q8_GROUP, Q8_BYTES = 32, 34


def reference_dir():
    """Where a checkout of the reference lies: $SMITH_REFERENCE_DIR, else a directory named
    `reference` beside this repository; None when there is none (then only a prebuilt
    oracle/_ref is used)."""
    cands = [os.environ.get("SMITH_REFERENCE_DIR"),
             os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")]
    for c in cands:
        if c and os.path.isfile(os.path.join(c, "shaders", "matmul_q4.metal")):
            return c
    return None


def build(quiet=True):
    """Compile the checkers with the recipe in oracle/Makefile."""
    ref_dir = reference_dir()
    subprocess.run(["make", "-C", _HERE] + ([f"REF={ref_dir}"] if ref_dir else []), check=True,
                   stdout=subprocess.DEVNULL if quiet else None)


def _load(path):
    lib = C.CDLL(path)
    return lib


_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB):
            build()
        _lib = _load(_LIB)
        i64, p = C.c_int64, C.c_void_p
        _lib.oracle_quantize_q4.restype = i64
        _lib.oracle_quantize_q4.argtypes = [p, i64, i64, p]
        _lib.oracle_quantize_q8.restype = i64
        _lib.oracle_quantize_q8.argtypes = [p, i64, i64, p]
        _lib.oracle_to_float16.restype = C.c_uint16
        _lib.oracle_to_float16.argtypes = [C.c_double]
        _lib.oracle_from_float16.restype = C.c_double
        _lib.oracle_from_float16.argtypes = [C.c_uint16]
        for name in ("oracle_dequant_q4", "oracle_dequant_q8"):
            f = getattr(_lib, name)
            f.restype = None
            f.argtypes = [p, i64, i64, p]
        for name in ("oracle_matmul_q4", "oracle_matmul_q8"):
            f = getattr(_lib, name)
            f.restype = None
            f.argtypes = [p, p, p, i64, i64, i64, i64, i64, i64, C.c_int]
        _lib.oracle_max_threads.restype = C.c_int
        _lib.oracle_rmsnorm.restype = None
        _lib.oracle_rmsnorm.argtypes = [p, p, p, i64, i64, C.c_float]
        _lib.oracle_gguf_dequant.restype = C.c_int
        _lib.oracle_gguf_dequant.argtypes = [C.c_int, p, i64, p]
        _lib.oracle_swiglu.restype = None
        _lib.oracle_swiglu.argtypes = [p, p, p, i64]
        for name in ("oracle_dense_f32", "oracle_dense_f16"):
            f = getattr(_lib, name)
            f.restype = None
            f.argtypes = [p, p, p, i64, i64, i64, i64]
    return _lib


def have_ref():
    return os.path.exists(_REF)


def ref():
    """The reference's shader source compiled as C++ (None when not built)."""
    global _ref
    if _ref is None and have_ref():
        _ref = _load(_REF)
        i64, p = C.c_int64, C.c_void_p
        for name in ("ref_matmul_q4", "ref_matmul_q8"):
            f = getattr(_ref, name)
            f.restype = None
            f.argtypes = [p, p, p, i64, i64, i64, i64, i64, i64, C.c_int]
        _ref.ref_max_threads.restype = C.c_int
        if hasattr(_ref, "ref_rmsnorm"):
            _ref.ref_rmsnorm.restype = None
            _ref.ref_rmsnorm.argtypes = [p, p, p, i64, i64, C.c_float]
            _ref.ref_swiglu.restype = None
            _ref.ref_swiglu.argtypes = [p, p, p, i64]
        if hasattr(_ref, "ref_dense"):
            _ref.ref_dense.restype = C.c_int
            _ref.ref_dense.argtypes = [C.c_int, C.c_int, p, p, p, i64, i64, i64, i64]
    return _ref


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


def _f32_2d(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    assert a.ndim == 2
    return a


def groups_of(K):
    return (K + 31) // 32


def quantize_q4(w):
    """f32 [K,N] -> uint8 [groups*N*24], the reference's Q4 block layout."""
    w = _f32_2d(w)
    K, N = w.shape
    out = np.zeros(groups_of(K) * N * Q4_BYTES, dtype=np.uint8)
    lib().oracle_quantize_q4(_ptr(w), K, N, _ptr(out))
    return out


def quantize_q8(w):
    """f32 [K,N] -> uint8 [groups*N*34], the layout matmul_q8 consumes."""
    w = _f32_2d(w)
    K, N = w.shape
    out = np.zeros(groups_of(K) * N * Q8_BYTES, dtype=np.uint8)
    lib().oracle_quantize_q8(_ptr(w), K, N, _ptr(out))
    return out


def to_float16(v):
    return int(lib().oracle_to_float16(float(v)))


def from_float16(h):
    return float(lib().oracle_from_float16(int(h)))


def dequant(packed, K, N, kind):
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    w = np.zeros((K, N), dtype=np.float32)
    getattr(lib(), "oracle_dequant_" + kind)(_ptr(packed), K, N, _ptr(w))
    return w


def _matmul(fn, a, packed, K, N, groups, cols, threads):
    a = _f32_2d(a)
    M = a.shape[0]
    assert a.shape[1] == K
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    groups = groups_of(K) if groups is None else groups
    c0, c1 = (0, N) if cols is None else cols
    out = np.zeros((M, N), dtype=np.float32)
    fn(_ptr(a), _ptr(packed), _ptr(out), M, N, K, groups, c0, c1, int(threads))
    return out


def matmul(a, packed, K, N, kind, groups=None, cols=None, threads=1):
    """Sequential-f32 shader arithmetic on the CPU (this repository's restatement)."""
    return _matmul(getattr(lib(), "oracle_matmul_" + kind), a, packed, K, N, groups, cols, threads)


def ref_matmul(a, packed, K, N, kind, groups=None, cols=None, threads=1):
    """Same call served by the reference's compiled shader source."""
    r = ref()
    if r is None:
        raise RuntimeError("oracle/_ref/libsmith_ref.so has not been built")
    return _matmul(getattr(r, "ref_matmul_" + kind), a, packed, K, N, groups, cols, threads)


def _rmsnorm(fn, x, gamma, eps):
    x = _f32_2d(x)
    gamma = np.ascontiguousarray(gamma, dtype=np.float32)
    assert gamma.shape == (x.shape[1],)
    out = np.zeros_like(x)
    fn(_ptr(x), _ptr(gamma), _ptr(out), x.shape[0], x.shape[1], float(eps))
    return out


def rmsnorm(x, gamma, eps=1e-5):
    """shaders/rmsnorm.metal:15-49 restated: x [rows, cols] * rsqrt(mean(x^2) + eps) * gamma."""
    return _rmsnorm(lib().oracle_rmsnorm, x, gamma, eps)


def ref_rmsnorm(x, gamma, eps=1e-5):
    """Same call served by the reference's compiled shader source."""
    return _rmsnorm(ref().ref_rmsnorm, x, gamma, eps)


def _swiglu(fn, gate, up):
    gate = np.ascontiguousarray(gate, dtype=np.float32)
    up = np.ascontiguousarray(up, dtype=np.float32)
    assert gate.shape == up.shape
    out = np.zeros_like(gate)
    fn(_ptr(gate), _ptr(up), _ptr(out), gate.size)
    return out


def swiglu(gate, up):
    """shaders/swiglu.metal:12-22 restated: silu(gate) * up."""
    return _swiglu(lib().oracle_swiglu, gate, up)


def ref_swiglu(gate, up):
    return _swiglu(ref().ref_swiglu, gate, up)


def _dense_operands(a, b):
    f16 = a.dtype == np.float16
    dt = np.float16 if f16 else np.float32
    a = np.ascontiguousarray(a, dtype=dt)
    b = np.ascontiguousarray(b, dtype=dt)
    if a.ndim == 2:
        a, b = a[None], b[None]
    batch, M, K = a.shape
    assert b.shape[0] == batch and b.shape[1] == K
    return f16, a, b, batch, M, b.shape[2], K


def dense_matmul(a, b):
    """shaders/matmul.metal restated: c[b,M,N] = a[b,M,K] @ b[b,K,N], sequential f32 sums; f16 arrays
    give the half-storage variants.  2-D operands give a 2-D result."""
    two_d = np.asarray(a).ndim == 2
    f16, a3, b3, batch, M, N, K = _dense_operands(np.asarray(a), np.asarray(b))
    out = np.zeros((batch, M, N), np.float16 if f16 else np.float32)
    (lib().oracle_dense_f16 if f16 else lib().oracle_dense_f32)(_ptr(a3), _ptr(b3), _ptr(out), M, N, K, batch)
    return out[0] if two_d else out


def have_ref_dense():
    return have_ref() and hasattr(ref(), "ref_dense")


def ref_dense_matmul(a, b, which):
    """The same product from the reference's compiled shader source; which = "simple", "tiled" or
    "batched" names the shader function (matmul_simple, matmul_f32, matmul_batched and their _f16 forms)."""
    two_d = np.asarray(a).ndim == 2
    f16, a3, b3, batch, M, N, K = _dense_operands(np.asarray(a), np.asarray(b))
    out = np.zeros((batch, M, N), np.float16 if f16 else np.float32)
    code = {"simple": 0, "tiled": 1, "batched": 2}[which]
    if code != 2:
        assert batch == 1
    rc = ref().ref_dense(code, int(f16), _ptr(a3), _ptr(b3), _ptr(out), M, N, K, batch)
    if rc != 0:
        raise RuntimeError("a team of 64 threads could not be formed for the tiled shader")
    return out[0] if two_d else out


def gguf_dequant(ggml_type, blocks):
    """src/gguf.js:187-197 / 221-231 restated: raw Q4_0 (type 2) or Q8_0 (type 8) blocks -> f32, 32 per block."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    per = 18 if ggml_type == 2 else 34
    n = blocks.size // per
    out = np.zeros(n * 32, dtype=np.float32)
    if lib().oracle_gguf_dequant(int(ggml_type), _ptr(blocks), n, _ptr(out)) != 0:
        raise ValueError("gguf_dequant: only Q4_0 (2) and Q8_0 (8)")
    return out


def have_ref_glue():
    r = ref()
    return r is not None and hasattr(r, "ref_rmsnorm")


def host_threads():
    """Cores this process may run on (what OpenMP would use if nothing capped it)."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def max_threads():
    return int(lib().oracle_max_threads())


def tolerance_bound(a, w_deq, rel=1e-3):
    """Per-output bound rel * ||a_m||_2 * ||w_deq[:,n]||_2  ->  [M,N] float64."""
    an = np.linalg.norm(np.asarray(a, dtype=np.float64), axis=1)
    wn = np.linalg.norm(np.asarray(w_deq, dtype=np.float64), axis=0)
    return rel * an[:, None] * wn[None, :]
