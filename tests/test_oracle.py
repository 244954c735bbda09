"""CPU tests of the checker itself: the oracle against the reference's compiled
shader source, the golden vectors, hand-worked known answers and the
reference's own test assertions for this path."""
import numpy as np
import pytest

from helpers import bits_equal, golden_cases, load_golden, py_quantize_q4
from oracle import oracle as O
from smith_b200 import dtype as D


@pytest.mark.parametrize("name", golden_cases())
def test_oracle_reproduces_golden(name):
    g = load_golden(name)
    K, N = g["w"].shape
    assert np.array_equal(O.quantize_q4(g["w"]), g["packed_q4"])
    assert np.array_equal(O.quantize_q8(g["w"]), g["packed_q8"])
    with np.errstate(all="ignore"):
        for kind in ("q4", "q8"):
            c = O.matmul(g["a"], g["packed_" + kind], K, N, kind)
            assert bits_equal(c, g["c_" + kind]), f"{name} {kind}: oracle differs from the compiled reference shader"


@pytest.mark.skipif(not O.have_ref(), reason="oracle/_ref not built (reference checkout absent)")
@pytest.mark.parametrize("kind", ["q4", "q8"])
@pytest.mark.parametrize("M,K,N", [(1, 64, 32), (3, 100, 40), (17, 4096, 96), (2, 33, 5), (1, 4096, 512)])
def test_oracle_matches_compiled_reference_shader(kind, M, K, N):
    rng = np.random.default_rng(K * 31 + N)
    w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    a = rng.standard_normal((M, K)).astype(np.float32)
    packed = O.quantize_q4(w) if kind == "q4" else O.quantize_q8(w)
    c = O.matmul(a, packed, K, N, kind)
    assert bits_equal(c, O.ref_matmul(a, packed, K, N, kind))
    assert bits_equal(c, O.matmul(a, packed, K, N, kind, threads=4))
    # column windows address the same outputs
    part = O.matmul(a, packed, K, N, kind, cols=(1, min(N, 4)))
    assert bits_equal(part[:, 1:min(N, 4)], c[:, 1:min(N, 4)])


@pytest.mark.parametrize("name", ["quirks_k64_n16", "ragged_k100_n40", "tiny_k1_n1", "odd_n_k96_n7"])
def test_c_oracle_equals_python_reading_of_the_packer(name):
    w = load_golden(name)["w"]
    assert np.array_equal(O.quantize_q4(w), py_quantize_q4(w))


def test_packer_quirks_bytes():
    g = load_golden("quirks_k64_n16")
    p = g["packed_q4"].reshape(2, 16, 24)

    def sz(col):
        return p[0, col, 16:20].view(np.float32)[0], p[0, col, 20:24].view(np.float32)[0]

    # constant group: scale 1, zero 8, codes round(clamp(0.25 + 8)) = 8
    assert sz(0) == (1.0, 8.0) and np.all(p[0, 0, :16] == 0x88)
    assert sz(1) == (1.0, 8.0) and np.all(p[0, 1, :16] == 0x88)
    # min == +0: zero is stored as -0.0 (sign bit set)
    s, z = sz(2)
    assert z == 0.0 and np.signbit(z) and s > 0
    # all NaN: scale 1, zero 8, codes 0
    assert sz(5) == (1.0, 8.0) and np.all(p[0, 5, :16] == 0)
    # one NaN among numbers: its code is 0, others are normal codes
    assert (p[0, 4, 5 >> 1] >> 4) == 0
    # infinite range: scale inf
    assert np.isinf(sz(6)[0])
    # min == -0: -(-0)/scale = +0
    assert sz(8)[1] == 0.0 and not np.signbit(sz(8)[1])


def test_hand_worked_q4_block():
    # 32 values k/31*1.5: min 0, max 1.5 -> scale 0.1 (f64 1.5/15), zero -0.0, codes round(v/0.1)
    w = (np.arange(32, dtype=np.float64) / 31 * 1.5).astype(np.float32).reshape(32, 1)
    p = O.quantize_q4(w)
    assert p.size == 24
    assert p[16:20].view(np.float32)[0] == np.float32(1.5 / 15)
    codes = [(p[k >> 1] >> (4 * (k & 1))) & 0xF for k in range(32)]
    expect = []
    for k in range(32):
        t = float(w[k, 0]) / (1.5 / 15) + (-0.0)
        f = np.floor(t)
        expect.append(int(f + 1 if t - f >= 0.5 else f))
    assert codes == expect and codes[0] == 0 and codes[31] == 15


def test_hand_worked_matmul_answers():
    # Q4: every nibble byte 0x21 (codes 1,2), scale .5, zero 1, K=64, a=1 -> 2 groups * 16 * .5 = 16
    blk = np.zeros(24, np.uint8)
    blk[:16] = 0x21
    blk[16:20] = np.frombuffer(np.float32(0.5).tobytes(), np.uint8)
    blk[20:24] = np.frombuffer(np.float32(1.0).tobytes(), np.uint8)
    packed = np.tile(blk, 2)
    assert O.matmul(np.ones((1, 64), np.float32), packed, 64, 1, "q4")[0, 0] == 16.0
    # Q8: scale half 0x3800 (.5), codes 3,-1 alternating, K=64, a=1 -> 2 * 16 * .5 * 2 = 32
    blk8 = np.zeros(34, np.uint8)
    blk8[0], blk8[1] = 0x00, 0x38
    blk8[2::2] = 3
    blk8[3::2] = 0xFF
    assert O.matmul(np.ones((1, 64), np.float32), np.tile(blk8, 2), 64, 1, "q8")[0, 0] == 32.0


def test_q8_block_byte_order_like_reference_gguf_kat():
    # tests/gguf.test.js:228-243 pins [f16 scale LE][32 x int8]: scale 0x3C00, bytes 1 / 255 -> +1 / -1
    blk = np.zeros(34, np.uint8)
    blk[0], blk[1] = 0x00, 0x3C
    blk[2], blk[3] = 1, 255
    w = O.dequant(blk, 32, 1, "q8")
    assert w[0, 0] == 1.0 and w[1, 0] == -1.0 and np.all(w[2:, 0] == 0)


def test_reference_inference_test_assertions():
    # tests/inference.test.js:94-123: K=64, N=32, U[0,1) weights, ones activations, 15 % of the column sums
    g = load_golden("ref_test_k64_n32")
    K, N = g["w"].shape
    assert (K, N, O.groups_of(K)) == (64, 32, 2)
    c = O.matmul(g["a"], g["packed_q4"], K, N, "q4")
    assert c.shape == (1, N)
    expected = g["w"].astype(np.float32).sum(axis=0)
    rel = np.abs(c[0] - expected) / (np.abs(expected) + 1e-6)
    assert np.all(rel < 0.15)
    # tests/inference.test.js:125-135: packed size ratio vs f32 below 0.35 (it is 24/128)
    g = load_golden("ref_ratio_k256_n256")
    assert g["packed_q4"].size / (256 * 256 * 4) == 24 / 128 < 0.35


def test_f16_codec_known_answers_and_agreement():
    assert D.toFloat16(1.0) == 0x3C00 and D.toFloat16(0.5) == 0x3800 and D.toFloat16(-2.0) == 0xC000
    assert D.toFloat16(65504.0) == 0x7BFF and D.toFloat16(65520.0) == 0x7BFF  # truncation, not rounding
    assert D.toFloat16(1e5) == 0x7C00 and D.toFloat16(float("inf")) == 0x7C00
    assert D.toFloat16(float("nan")) & 0x7E00 == 0x7E00
    assert D.toFloat16(1e-5) == 0 and D.toFloat16(-1e-5) == 0x8000           # sub-normal range flushes
    assert D.toFloat16(1.0009765625 + 0.0009) == 0x3C01                       # mantissa truncated
    assert D.fromFloat16(0x3800) == 0.5 and D.fromFloat16(0x0001) == 2.0 ** -24
    rng = np.random.default_rng(7)
    vals = np.concatenate([rng.standard_normal(2000) * 10.0 ** rng.integers(-8, 6, 2000), [0.0, -0.0, 6.1e-5, 6.0e-5]])
    for v in vals:
        assert D.toFloat16(v) == O.to_float16(v)
    for h in list(range(0, 0x10000, 97)) + [0x7C00, 0xFC00, 0x0001, 0x8001]:
        a, b = D.fromFloat16(h), O.from_float16(h)
        assert (a == b) or (a != a and b != b)


def test_q8_rule_properties():
    rng = np.random.default_rng(11)
    w = (rng.standard_normal((64, 8)) * 0.02).astype(np.float32)
    w[:32, 0] = 0.0
    p = O.quantize_q8(w).reshape(2, 8, 34)
    assert np.all(p[0, 0] == 0)                       # zero block: scale 0, codes 0
    codes = p[..., 2:].view(np.int8)
    assert codes.min() >= -127 and codes.max() <= 127
    deq = O.dequant(p.reshape(-1), 64, 8, "q8")
    amax = np.abs(w.reshape(2, 32, 8)).max(axis=1)
    # scale is amax/127 truncated to half precision: error per element below one code step
    step = np.repeat(amax / 127, 32, axis=0).reshape(64, 8)
    assert np.all(np.abs(deq - w) <= step * 1.01 + 1e-12)


# ---- the pointwise glue of the decode step (folded into the list kernel)
@pytest.mark.skipif(not (O.have_ref() and O.have_ref_glue()), reason="oracle/_ref not built (no reference checkout on this machine)")
@pytest.mark.parametrize("rows,cols", [(1, 64), (3, 100), (2, 256), (1, 4096), (2, 14336), (1, 7)])
def test_rmsnorm_restatement_equals_the_compiled_shader(rows, cols):
    """oracle_rmsnorm against shaders/rmsnorm.metal compiled as C++ and run as a threadgroup (an OpenMP
    team): same partial sums, same halving tree, same bits."""
    rng = np.random.default_rng(rows * 1000 + cols)
    x = (rng.standard_normal((rows, cols)) * 3).astype(np.float32)
    g = (1.0 + 0.3 * rng.standard_normal(cols)).astype(np.float32)
    for eps in (1e-5, 1e-6):
        a, b = O.rmsnorm(x, g, eps), O.ref_rmsnorm(x, g, eps)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


@pytest.mark.skipif(not (O.have_ref() and O.have_ref_glue()), reason="oracle/_ref not built (no reference checkout on this machine)")
def test_swiglu_restatement_equals_the_compiled_shader():
    rng = np.random.default_rng(5)
    gate = (rng.standard_normal(5000) * 4).astype(np.float32)
    up = rng.standard_normal(5000).astype(np.float32)
    gate[:4] = [0.0, -0.0, 88.0, -88.0]
    assert np.array_equal(O.swiglu(gate, up).view(np.uint32), O.ref_swiglu(gate, up).view(np.uint32))


def test_rmsnorm_and_swiglu_known_answers():
    """Hand-checkable cases: a row of equal values normalises to gamma (up to eps); silu(0) = 0."""
    x = np.full((1, 64), 2.0, np.float32)
    g = np.arange(64, dtype=np.float32)
    out = O.rmsnorm(x, g, 0.0)
    assert np.allclose(out, g, rtol=1e-6)
    assert O.swiglu(np.zeros(3, np.float32), np.ones(3, np.float32)).tolist() == [0.0, 0.0, 0.0]
    big = O.swiglu(np.array([20.0], np.float32), np.array([2.0], np.float32))
    assert abs(float(big[0]) - 40.0) < 1e-5


# ---- GGUF block decoders (src/gguf.js:187-197, 221-231), the known answers of tests/gguf.test.js:208-243
def test_gguf_q4_0_block_known_answers():
    block = np.zeros(18, np.uint8)
    block[0], block[1] = 0x00, 0x38                 # scale 0.5 as f16
    block[2:] = 0x88                                # every nibble 8 -> 0.5 * (8 - 8) = 0
    assert np.all(O.gguf_dequant(2, block) == 0.0)
    block[2:] = 0xFF                                # every nibble 15 -> 0.5 * (15 - 8) = 3.5
    assert np.all(O.gguf_dequant(2, block) == 3.5)
    block[2] = 0x21                                 # element 0 = low nibble 1, element 1 = high nibble 2
    v = O.gguf_dequant(2, block)
    assert v[0] == 0.5 * (1 - 8) and v[1] == 0.5 * (2 - 8)


def test_gguf_q8_0_block_known_answers():
    block = np.zeros(34, np.uint8)
    block[0], block[1] = 0x00, 0x3C                 # scale 1.0 as f16
    block[2::2], block[3::2] = 1, 255               # +1, -1 alternating
    v = O.gguf_dequant(8, block)
    assert v[0] == 1.0 and v[1] == -1.0 and v[2] == 1.0


def test_gguf_q8_0_blocks_are_the_matmul_q8_blocks():
    """A Q8_0 tensor [outDim, inDim] re-tiled block by block is the packed [inDim/32][outDim][34] matrix:
    de-quantising either way gives the transposed weights bit for bit."""
    rng = np.random.default_rng(8)
    out_dim, in_dim = 24, 96
    G = in_dim // 32
    blocks = rng.integers(0, 256, (out_dim, G, 34), dtype=np.uint8)
    blocks[:, :, 1] = rng.integers(0x20, 0x3C, (out_dim, G))      # finite f16 scales
    w_file = O.gguf_dequant(8, blocks).reshape(out_dim, in_dim)   # the reference's f32 weights, [outDim, inDim]
    packed = np.ascontiguousarray(blocks.transpose(1, 0, 2)).reshape(-1)
    assert np.array_equal(O.dequant(packed, in_dim, out_dim, "q8").view(np.uint32), w_file.T.copy().view(np.uint32))


# ---------------------------------------------------------------- dense matmul (shaders/matmul.metal)
DENSE_SHAPES = [(1, 1, 1), (2, 3, 2), (16, 16, 16), (33, 70, 65), (64, 64, 64), (70, 100, 96)]


@pytest.mark.skipif(not (O.have_ref() and O.have_ref_dense()), reason="oracle/_ref not built (no reference checkout on this machine)")
@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_dense_restatement_equals_the_compiled_shaders(dtype):
    """oracle_dense_f32 / oracle_dense_f16 against matmul_simple, the tiled matmul_f32 (run as teams of
    64 threads with real barriers) and matmul_batched of shaders/matmul.metal compiled as C++: bit for bit."""
    rng = np.random.default_rng(17)
    bits = np.uint16 if dtype == np.float16 else np.uint32
    for M, K, N in DENSE_SHAPES:
        a, b = rng.standard_normal((M, K)).astype(dtype), rng.standard_normal((K, N)).astype(dtype)
        want = O.dense_matmul(a, b)
        assert np.array_equal(want.view(bits), O.ref_dense_matmul(a, b, "simple").view(bits)), (M, K, N)
        # the tiled kernel pads its last k-tile with zeros: +0 terms, which only a -0 sum could notice
        assert np.array_equal(want, O.ref_dense_matmul(a, b, "tiled")), (M, K, N)
    a, b = rng.standard_normal((3, 9, 17)).astype(dtype), rng.standard_normal((3, 17, 5)).astype(dtype)
    assert np.array_equal(O.dense_matmul(a, b).view(bits), O.ref_dense_matmul(a, b, "batched").view(bits))


def test_dense_known_answers_of_the_reference_tests():
    # tests/matmul.test.js:15-48 and tests/f16.test.js:88-98
    for dtype in (np.float32, np.float16):
        c = O.dense_matmul(np.array([[1, 2], [3, 4]], dtype), np.array([[5, 6], [7, 8]], dtype))
        assert c.dtype == dtype and c.tolist() == [[19, 22], [43, 50]]
        c = O.dense_matmul(np.array([[1, 2, 3], [4, 5, 6]], dtype), np.array([[7, 8], [9, 10], [11, 12]], dtype))
        assert c.tolist() == [[58, 64], [139, 154]]
    a = np.random.default_rng(2).standard_normal((16, 16)).astype(np.float32)
    assert np.array_equal(O.dense_matmul(a, np.eye(16, dtype=np.float32)), a)          # :74-86


def test_dense_restatement_is_a_sequential_f32_sum():
    rng = np.random.default_rng(4)
    a, b = rng.standard_normal((5, 300)).astype(np.float32), rng.standard_normal((300, 7)).astype(np.float32)
    want = np.zeros((5, 7), np.float32)
    for k in range(300):
        want = (want + (a[:, k:k + 1] * b[k:k + 1, :]).astype(np.float32)).astype(np.float32)
    assert np.array_equal(O.dense_matmul(a, b), want)
    ah, bh = a.astype(np.float16), b.astype(np.float16)
    want = np.zeros((5, 7), np.float32)
    for k in range(300):
        want = (want + (ah[:, k:k + 1].astype(np.float32) * bh[k:k + 1, :].astype(np.float32))).astype(np.float32)
    assert np.array_equal(O.dense_matmul(ah, bh), want.astype(np.float16))
