"""-m gpu: the dense (unquantised) matmul family of shaders/matmul.metal behind smith_matmul and
behind the reference's kernel names, against the oracle (oracle_dense_f32 / oracle_dense_f16, which
the CPU tests pin bit for bit to the reference's shader source compiled as C++).

Bars, written where they are applied:
  * any-shape CUDA-core kernel (matmul_simple / matmul_batched and whatever the tensor-core kernel
    declines): bit-exact, f32 and f16;
  * tensor cores, f32 storage as three bf16 planes (six partial products):
        |c - oracle| <= 4e-6 * ||a_m||_2 * ||b_n||_2
    (the oracle's own sequential f32 sum is that far from the exact sum at these K);
  * tensor cores, f16 storage: |c - exact| <= 2^-10 * |exact| + 4e-6 * ||a_m|| * ||b_n||
    (exact products, f32 sums, one rounding of the result to half);
  * tensor cores, fast mode (f32 rounded to bf16 once): 1e-2 * ||a_m|| * ||b_n||.
"""
import numpy as np
import pytest

from gpu_util import DevBuf
from helpers import bits_equal
from oracle import oracle as O
import smith_b200 as smith
from smith_b200 import device

pytestmark = pytest.mark.gpu


def dense_on_device(a, b, path=device.DENSE_AUTO):
    f16 = a.dtype == np.float16
    a3, b3 = (a[None], b[None]) if a.ndim == 2 else (a, b)
    batch, M, K = a3.shape
    N = b3.shape[2]
    es = 2 if f16 else 4
    ab, bb, cb = DevBuf.of(a3), DevBuf.of(b3), DevBuf(batch * M * N * es)
    device.upload(cb.handle, np.full(batch * M * N, np.nan, a.dtype))
    device.matmul(device.DTYPE_F16 if f16 else device.DTYPE_F32, ab.handle, bb.handle, cb.handle, M, N, K, batch, path)
    device.synchronize()
    assert device.kernelStatus() == 0, "a bounded device-side wait gave up"
    out = cb.get(a.dtype).reshape(batch, M, N)
    for x in (ab, bb, cb):
        x.free()
    return out[0] if a.ndim == 2 else out


def _norm_bound(a, b, rel):
    an = np.linalg.norm(a.astype(np.float64), axis=-1)            # [.., M]
    bn = np.linalg.norm(b.astype(np.float64), axis=-2)            # [.., N]
    return rel * an[..., :, None] * bn[..., None, :]


def _data(seed, shape_a, shape_b, dtype=np.float32):
    rng = np.random.default_rng(seed)
    return rng.standard_normal(shape_a).astype(dtype), rng.standard_normal(shape_b).astype(dtype)


GENERIC_SHAPES = [(1, 1, 1), (2, 2, 2), (2, 3, 2), (16, 16, 16), (32, 64, 16), (63, 63, 63), (65, 17, 130),
                  (7, 1000, 77), (100, 33, 5), (128, 256, 64)]


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_any_shape_kernel_is_bit_exact(dtype):
    for i, (M, K, N) in enumerate(GENERIC_SHAPES):
        a, b = _data(i, (M, K), (K, N), dtype)
        got = dense_on_device(a, b, device.DENSE_GENERIC)
        want = O.dense_matmul(a, b)
        assert np.array_equal(got.view(np.uint16 if dtype == np.float16 else np.uint32),
                              want.view(np.uint16 if dtype == np.float16 else np.uint32)), (M, K, N)


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_batched_is_bit_exact(dtype):
    for i, (B, M, K, N) in enumerate([(1, 4, 4, 4), (3, 9, 17, 5), (12, 64, 64, 64), (8, 1, 128, 40), (2, 70, 30, 90)]):
        a, b = _data(50 + i, (B, M, K), (B, K, N), dtype)
        got = dense_on_device(a, b, device.DENSE_GENERIC)
        want = O.dense_matmul(a, b)
        assert np.array_equal(got.view(np.uint16 if dtype == np.float16 else np.uint32),
                              want.view(np.uint16 if dtype == np.float16 else np.uint32)), (B, M, K, N)


# one tile; ragged M, N and K (K not a multiple of 8 or 64; N not a multiple of 16); several row and
# column tiles; a K longer than the ring; a large square
TC_SHAPES = [(64, 64, 64), (128, 128, 128), (100, 200, 72), (130, 1001, 250), (257, 333, 129), (512, 4096, 1024),
             (64, 8192, 64), (1024, 1024, 1024),
             # more than one wave of 128 x 128 tiles: the three-plane mode then runs on CTA pairs
             # (256 x 256 tiles); the second shape has an odd number of row tiles and a ragged last column tile
             (2048, 256, 2048), (1300, 200, 1900)]


def test_tensor_core_f32_three_planes():
    worst_all = 0.0
    for i, (M, K, N) in enumerate(TC_SHAPES):
        a, b = _data(100 + i, (M, K), (K, N))
        got = dense_on_device(a, b, device.DENSE_TENSOR)
        want = O.dense_matmul(a, b)
        bound = _norm_bound(a, b, 4e-6)
        worst = float((np.abs(got.astype(np.float64) - want) / bound).max())
        assert np.all(np.isfinite(got)) and worst <= 1.0, f"M={M} K={K} N={N}: worst err/bound = {worst}"
        worst_all = max(worst_all, worst)
    assert worst_all > 0.0


def test_tensor_core_f32_is_closer_to_the_exact_product_than_the_sequential_sum_allows():
    # against the f64 product: the six partial products leave out terms below 2^-23 of each product
    M, K, N = 256, 2048, 256
    a, b = _data(7, (M, K), (K, N))
    got = dense_on_device(a, b, device.DENSE_TENSOR)
    exact = a.astype(np.float64) @ b.astype(np.float64)
    bound = _norm_bound(a, b, 1e-6)
    assert float((np.abs(got - exact) / bound).max()) <= 1.0


def test_tensor_core_f32_on_cta_pairs_with_non_finite_inputs():
    M, K, N = 2048, 128, 2048
    a, b = _data(9, (M, K), (K, N))
    a[1500, 3] = np.nan                                     # a row of the second CTA of a pair
    a[130, 5] = np.inf
    got = dense_on_device(a, b, device.DENSE_TENSOR)
    want = O.dense_matmul(a, b)
    assert np.all(np.isnan(got[1500])) and np.all(np.isinf(got[130]) | np.isnan(got[130]))
    rows = [r for r in range(M) if r not in (130, 1500)]
    assert np.all(np.isfinite(got[rows]))
    assert float((np.abs(got[rows].astype(np.float64) - want[rows]) / _norm_bound(a[rows], b, 4e-6)).max()) <= 1.0


def test_tensor_core_fast_mode():
    for i, (M, K, N) in enumerate([(128, 512, 128), (300, 1000, 200)]):
        a, b = _data(200 + i, (M, K), (K, N))
        got = dense_on_device(a, b, device.DENSE_TENSOR_FAST)
        want = O.dense_matmul(a, b)
        worst = float((np.abs(got.astype(np.float64) - want) / _norm_bound(a, b, 1e-2)).max())
        assert worst <= 1.0, f"M={M} K={K} N={N}: worst err/bound = {worst}"


def test_tensor_core_f16_storage():
    for i, (M, K, N) in enumerate([(64, 64, 64), (128, 256, 512), (200, 1000, 300), (257, 2048, 130), (512, 4096, 512)]):
        a, b = _data(300 + i, (M, K), (K, N), np.float16)
        got = dense_on_device(a, b, device.DENSE_TENSOR).astype(np.float64)
        exact = a.astype(np.float64) @ b.astype(np.float64)
        bound = 2.0 ** -10 * np.abs(exact) + _norm_bound(a, b, 4e-6)
        worst = float((np.abs(got - exact) / bound).max())
        assert worst <= 1.0, f"M={M} K={K} N={N}: worst err/bound = {worst}"


def test_tensor_core_declines_what_it_cannot_take():
    a, b = _data(1, (64, 100), (100, 64), np.float16)      # f16 rows of 200 bytes do not start on 16 bytes
    with pytest.raises(device.SmithError, match="does not take"):
        dense_on_device(a, b, device.DENSE_TENSOR)
    got = dense_on_device(a, b)                             # the automatic choice falls back, bit-exact
    assert np.array_equal(got.view(np.uint16), O.dense_matmul(a, b).view(np.uint16))


def test_non_finite_inputs_propagate():
    a, b = _data(5, (128, 128), (128, 128))
    a[3, 7] = np.inf
    a[100, 0] = np.nan
    b[5, 9] = 3.0e38                                        # rounds to infinity in bf16: must stay finite
    a[:, 5] *= 1e-4
    got = dense_on_device(a, b, device.DENSE_TENSOR)
    want = O.dense_matmul(a, b)
    assert np.all(np.isnan(got[100]))
    assert np.all(np.isinf(got[3]) | np.isnan(got[3]))
    rows = [r for r in range(128) if r not in (3, 100)]
    assert np.all(np.isfinite(got[rows]))
    bound = _norm_bound(a[rows], b, 4e-6)
    assert float((np.abs(got[rows].astype(np.float64) - want[rows]) / bound).max()) <= 1.0


# ---------------------------------------------------------------- the operators (src/ops/matmul.js)
def _close(actual, expected, tol=1e-4):
    assert np.all(np.abs(np.asarray(actual, np.float64) - np.asarray(expected, np.float64)) < tol), (actual, expected)


def test_operator_known_answers():
    # tests/matmul.test.js:15-48
    c = smith.matmul(smith.tensorFrom([1, 2, 3, 4], [2, 2]), smith.tensorFrom([5, 6, 7, 8], [2, 2]))
    _close(smith.toArray(c), [[19, 22], [43, 50]])
    c = smith.matmul(smith.tensorFrom([1, 2, 3, 4], [2, 2]), smith.tensorFrom([1, 0, 0, 1], [2, 2]))
    _close(smith.toArray(c), [[1, 2], [3, 4]])
    c = smith.matmul(smith.tensorFrom([1, 2, 3, 4, 5, 6], [2, 3]), smith.tensorFrom([7, 8, 9, 10, 11, 12], [3, 2]))
    assert c.shape == [2, 2]
    _close(smith.toArray(c), [[58, 64], [139, 154]])
    # tests/f16.test.js:88-98
    c = smith.matmul(smith.tensorFrom([1, 2, 3, 4], [2, 2], "f16"), smith.tensorFrom([5, 6, 7, 8], [2, 2], "f16"))
    assert c.dtype == "f16"
    _close(smith.toArray(c), [[19, 22], [43, 50]])


def test_operator_properties_of_the_reference_tests():
    rng = np.random.default_rng(11)
    # tests/matmul.test.js:74-86: A @ I = A
    N = 16
    av = (rng.random(N * N) * 2 - 1).astype(np.float32)
    r = smith.matmul(smith.tensorFrom(av, [N, N]), smith.tensorFrom(np.eye(N, dtype=np.float32).ravel(), [N, N]))
    assert np.all(np.abs(smith.toNumpy(r).ravel() - av) < 1e-3)
    # :88-103: [32x64] @ [64x16], one element against a scalar loop
    M, K, N = 32, 64, 16
    av, bv = (rng.random(M * K) - 0.5).astype(np.float32), (rng.random(K * N) - 0.5).astype(np.float32)
    c = smith.toNumpy(smith.matmul(smith.tensorFrom(av, [M, K]), smith.tensorFrom(bv, [K, N])))
    assert c.shape == (M, N)
    assert abs(c[7, 3] - sum(float(av[7 * K + k]) * float(bv[k * N + 3]) for k in range(K))) < 1e-3
    # :105-120: (A@B)@C ~ A@(B@C)
    N = 32
    A, B, C = (smith.tensorFrom((rng.random(N * N) - 0.5).astype(np.float32), [N, N]) for _ in range(3))
    left = smith.toNumpy(smith.matmul(smith.matmul(A, B), C))
    right = smith.toNumpy(smith.matmul(A, smith.matmul(B, C)))
    assert np.all(np.abs(left - right) < 1e-2)
    # tests/f16.test.js:100-123: f16 against f32 on the same values
    N = 16
    vals = (rng.random(N * N) * 2 - 1).astype(np.float32)
    c32 = smith.toNumpy(smith.matmul(smith.tensorFrom(vals, [N, N]), smith.tensorFrom(vals, [N, N]))).ravel()
    c16 = np.array(smith.toArray(smith.matmul(smith.tensorFrom(vals, [N, N], "f16"), smith.tensorFrom(vals, [N, N], "f16")))).ravel()
    assert np.max(np.abs(c32 - c16)) < 0.05


def test_operator_picks_the_tiled_name_from_64_and_handles_batches():
    a, b = _data(21, (96, 80), (80, 72))
    c = smith.toNumpy(smith.matmul(smith.tensorFrom(a.ravel(), [96, 80]), smith.tensorFrom(b.ravel(), [80, 72])))
    want = O.dense_matmul(a, b)
    assert float((np.abs(c.astype(np.float64) - want) / _norm_bound(a, b, 4e-6)).max()) <= 1.0
    a, b = _data(22, (4, 6, 10, 12), (4, 6, 12, 8))
    c = smith.matmul(smith.tensorFrom(a.ravel(), [4, 6, 10, 12]), smith.tensorFrom(b.ravel(), [4, 6, 12, 8]))
    assert c.shape == [4, 6, 10, 8]
    want = O.dense_matmul(a.reshape(24, 10, 12), b.reshape(24, 12, 8)).reshape(4, 6, 10, 8)
    assert bits_equal(smith.toNumpy(c), want)
    with pytest.raises(ValueError, match="inner dims don't match: 3 vs 4"):
        smith.matmul(smith.zeros([2, 3]), smith.zeros([4, 2]))
    with pytest.raises(ValueError, match="requires at least 2D"):
        smith.matmul(smith.zeros([3]), smith.zeros([3, 2]))
