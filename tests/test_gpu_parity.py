"""-m gpu: the CUDA path against the oracle, through the C ABI.

Packed bytes must be bit-identical to the CPU restatement of the reference
packer; matmul outputs must satisfy max |delta_mn| <= 1e-3 * ||a_m|| * ||w_deq[:,n]||
against the sequential-f32 shader arithmetic (and be bit-identical on the
any-shape kernel, which keeps the shader's operation order)."""
import numpy as np
import pytest

import smith_b200 as smith
from gpu_util import DevBuf, matmul_on_device, pack_on_device
from helpers import bits_equal, golden_cases, load_golden, within_tolerance
from oracle import oracle as O
from smith_b200 import device

pytestmark = pytest.mark.gpu

REL = 1e-3  # tolerance factor stated by the north star for f32 accumulation


def _data(seed, M, K, N, std=0.02):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((K, N)) * std).astype(np.float32)
    a = rng.standard_normal((M, K)).astype(np.float32)
    return a, w


# ------------------------------------------------------------------ packers
@pytest.mark.parametrize("name", golden_cases())
def test_packers_reproduce_golden_bytes(name):
    g = load_golden(name)
    assert np.array_equal(pack_on_device(g["w"], "q4"), g["packed_q4"])
    assert np.array_equal(pack_on_device(g["w"], "q8"), g["packed_q8"])


@pytest.mark.parametrize("K,N", [(4096, 512), (4096, 1000), (1000, 257), (31, 3), (33, 300), (14336, 64)])
@pytest.mark.parametrize("kind", ["q4", "q8"])
def test_packers_bit_exact_random(kind, K, N):
    rng = np.random.default_rng(K + N)
    for w in ((rng.standard_normal((K, N)) * 0.02).astype(np.float32), rng.random((K, N), dtype=np.float32),
              (rng.standard_normal((K, N)) * 1e4).astype(np.float32)):
        want = O.quantize_q4(w) if kind == "q4" else O.quantize_q8(w)
        assert np.array_equal(pack_on_device(w, kind), want)


@pytest.mark.parametrize("kind", ["q4", "q8"])
def test_packers_bit_exact_where_the_f32_screen_is_weak_or_off(kind):
    """The packers screen every element in f32 and evaluate the f64 expression only next to a rounding
    boundary.  Data chosen to strain that: a large common offset (the f32 sum cancels, every element
    must take the f64 path), scales far outside the ordinary range (screen switched off), groups that
    are constant, denormal or infinite, and quotients that land on multiples of 1/8 and of 2^-20."""
    K, N = 96, 1536
    rng = np.random.default_rng(77)
    cases = [
        (1000.0 + rng.random((K, N)) * 1e-3).astype(np.float32),
        (-3.0e6 + rng.standard_normal((K, N))).astype(np.float32),
        (rng.standard_normal((K, N)) * 1e-36).astype(np.float32),
        (rng.standard_normal((K, N)) * 1e-41).astype(np.float32),            # denormals
        (rng.standard_normal((K, N)) * 1e36).astype(np.float32),
        np.full((K, N), 0.25, np.float32),
        (rng.integers(-120, 121, (K, N)) / 8.0).astype(np.float32),
        (rng.integers(0, 16, (K, N)) + rng.integers(-3, 4, (K, N)) * 2.0 ** -20 + 0.5).astype(np.float32),
    ]
    w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    w[5, ::7] = np.inf
    w[40, ::11] = -np.inf
    w[70, ::13] = np.nan
    cases.append(w)
    for i, w in enumerate(cases):
        with np.errstate(all="ignore"):
            want = O.quantize_q4(w) if kind == "q4" else O.quantize_q8(w)
        assert np.array_equal(pack_on_device(w, kind), want), f"case {i}"


def test_packer_rounding_boundaries():
    # values engineered to sit on and next to .5 code boundaries after v/scale + zero
    K, N = 32, 4096
    rng = np.random.default_rng(5)
    w = np.zeros((K, N), np.float32)
    w[0] = 0.0
    w[31] = 15.0                                     # scale exactly 1, zero -0.0
    half = rng.integers(0, 15, (30, N)) + 0.5
    w[1:31] = half + rng.choice([0.0, 1e-6, -1e-6, 2.0 ** -20, -2.0 ** -20], (30, N))
    assert np.array_equal(pack_on_device(w, "q4"), O.quantize_q4(w))
    assert np.array_equal(pack_on_device(w, "q8"), O.quantize_q8(w))


# ------------------------------------------------------------------ matmul: golden + every path
@pytest.mark.parametrize("name", golden_cases())
@pytest.mark.parametrize("kind", ["q4", "q8"])
def test_matmul_golden(name, kind):
    g = load_golden(name)
    K, N = g["w"].shape
    packed, a, want = g["packed_" + kind], g["a"], g["c_" + kind]
    got = matmul_on_device(a, packed, K, N, kind, device.PATH_GENERIC)
    if "quirks" not in name:
        assert bits_equal(got, want), "any-shape kernel must keep the shader's operation order"
    ok, worst = within_tolerance(got, want, a, packed, K, N, kind, REL)
    assert ok, worst
    got = matmul_on_device(a, packed, K, N, kind, device.PATH_AUTO)
    ok, worst = within_tolerance(got, want, a, packed, K, N, kind, REL)
    assert ok, worst


SHAPES = [
    # M, K, N
    (1, 4096, 4096),      # cfg1
    (1, 4096, 14336 // 8),
    (4, 4096, 1792),
    (16, 4096, 1792),
    (2, 512, 130),
    (7, 2048, 1000),
    (16, 14336, 512),     # down-projection-shaped K
    (64, 4096, 1024),
    (100, 1024, 768),
    (256, 4096, 512),
    (512, 1024, 1376),
    (33, 96, 66),
    (3, 100, 40),         # ragged K
    (130, 200, 56),       # ragged K, M > 128
]


@pytest.mark.parametrize("M,K,N", SHAPES)
@pytest.mark.parametrize("kind", ["q4", "q8"])
def test_matmul_auto_path_within_tolerance(kind, M, K, N):
    a, w = _data(M * 7 + K + N, M, K, N)
    packed = O.quantize_q4(w) if kind == "q4" else O.quantize_q8(w)
    want = O.matmul(a, packed, K, N, kind, threads=O.max_threads())
    got = matmul_on_device(a, packed, K, N, kind)
    ok, worst = within_tolerance(got, want, a, packed, K, N, kind, REL)
    assert ok, f"worst err/bound = {worst}"


@pytest.mark.parametrize("path", [device.PATH_GENERIC, device.PATH_DECODE, device.PATH_TENSOR, device.PATH_GEMV,
                                  device.PATH_SKINNY])
@pytest.mark.parametrize("kind", ["q4", "q8"])
def test_matmul_each_path_where_supported(kind, path):
    shapes = {device.PATH_GENERIC: [(1, 64, 32), (9, 1000, 77)],
              device.PATH_DECODE: [(1, 4096, 1024), (5, 1024, 256), (16, 2048, 640), (8, 4096, 104), (7, 4128, 136), (13, 96, 8),
                                   (9, 14336, 256), (24, 4096, 512), (32, 1024, 264), (20, 2048, 96), (17, 8192, 128)],
              device.PATH_GEMV: [(1, 4096, 1024), (2, 1024, 256), (4, 2048, 640), (3, 4096, 104), (1, 14336, 512),
                                 (1, 64, 8), (2, 28672, 64),
                                 # tensor-map boxes (narrow tiles, >= 192 group-rows) with ragged edges:
                                 # partial last stage, partial last tile, Q8's 8-column quantum
                                 (3, 6176, 1000), (1, 8192, 8200), (4, 6208, 2056)],
              # 1, 2 and 4 row tiles; ragged last column tile; one group; K-phases that do not divide the groups
              device.PATH_SKINNY: [(5, 256, 64), (16, 512, 1000), (17, 1024, 1192), (33, 2048, 4096), (64, 4096, 2048),
                                   (7, 32, 8), (1, 4096, 1024), (48, 4128, 136), (64, 14336, 512)],
              device.PATH_TENSOR: [(64, 1024, 256), (512, 4096, 512), (17, 256, 128), (200, 2048, 384), (300, 1056, 72),
                                   # two k-blocks per hand-off with a zero tail, narrow column tiles, ragged N
                                   (33, 1024, 48), (100, 4160, 1024), (130, 1056, 1000)]}[path]
    for M, K, N in shapes:
        a, w = _data(M + K + N + path, M, K, N)
        packed = O.quantize_q4(w) if kind == "q4" else O.quantize_q8(w)
        want = O.matmul(a, packed, K, N, kind, threads=O.max_threads())
        try:
            got = matmul_on_device(a, packed, K, N, kind, path)
        except device.SmithError as e:
            assert "does not take" in str(e), e
            continue
        if path == device.PATH_GENERIC:
            assert bits_equal(got, want)
        ok, worst = within_tolerance(got, want, a, packed, K, N, kind, REL)
        assert ok, f"path {path} M={M} K={K} N={N}: worst err/bound = {worst}"


def test_structured_inputs_ones_and_uniform():
    # the reference test's own shape of data: U[0,1) weights, all-ones activations (no cancellation)
    rng = np.random.default_rng(3)
    for M, K, N in [(1, 4096, 1024), (8, 4096, 512), (128, 1024, 256)]:
        w = rng.random((K, N), dtype=np.float32)
        a = np.ones((M, K), np.float32)
        for kind in ("q4", "q8"):
            packed = O.quantize_q4(w) if kind == "q4" else O.quantize_q8(w)
            want = O.matmul(a, packed, K, N, kind)
            got = matmul_on_device(a, packed, K, N, kind)
            ok, worst = within_tolerance(got, want, a, packed, K, N, kind, REL)
            assert ok, worst


def test_linearity_at_full_size():
    # size-independent property at the headline shape: f(a1 + a2) ~= f(a1) + f(a2), f(2a) == 2 f(a)
    K, N = 4096, 14336
    wb = DevBuf(K * N * 4)
    device.fillNormal(wb.handle, K * N, 1, 0.02)
    pb = DevBuf((K // 32) * N * 24)
    device.q4Pack(wb.handle, pb.handle, K, N)
    device.synchronize()
    wb.free()
    rng = np.random.default_rng(9)
    a1 = rng.standard_normal((1, K)).astype(np.float32)
    a2 = rng.standard_normal((1, K)).astype(np.float32)

    def f(a):
        ab, cb = DevBuf.of(a), DevBuf(a.shape[0] * N * 4)
        device.qmatmul(4, ab.handle, pb.handle, cb.handle, a.shape[0], N, K, K // 32, 0)
        device.synchronize()
        out = cb.get(np.float32).reshape(a.shape[0], N)
        ab.free()
        cb.free()
        return out

    y1, y2, y12, y2x = f(a1), f(a2), f(a1 + a2), f(2 * a1)
    assert np.array_equal(y2x, 2 * y1)
    scale = np.abs(y1).max() + np.abs(y2).max()
    assert np.abs(y12 - (y1 + y2)).max() <= 1e-4 * scale
    # sampled columns against the oracle
    packed = pb.get()
    cols = (5000, 5064)
    want = O.matmul(a1, packed, K, N, "q4", cols=cols)
    ok, worst = within_tolerance(y1[:, cols[0]:cols[1]], want[:, cols[0]:cols[1]], a1,
                                 packed.reshape(K // 32, N, 24)[:, cols[0]:cols[1]].reshape(-1), K, cols[1] - cols[0],
                                 "q4", REL)
    assert ok, worst
    pb.free()


def test_empty_and_degenerate_shapes():
    K, N = 64, 16
    a, w = _data(1, 2, K, N)
    packed = O.quantize_q4(w)
    assert matmul_on_device(a[:0], packed, K, N, "q4").shape == (0, N)
    # groups smaller than ceil(K/32): the shader simply stops early
    want = O.matmul(a, packed, K, N, "q4", groups=1)
    got = matmul_on_device(a, packed, K, N, "q4", device.PATH_GENERIC, groups=1)
    assert bits_equal(got, want)


# ------------------------------------------------------------------ operator API (reference test restated)
def test_operator_api_reference_test():
    # tests/inference.test.js:94-123
    K, N = 64, 32
    smith.tensor.seed(0)
    w = smith.rand([K, N])
    wq = smith.quantizeQ4(w)
    assert (wq.K, wq.N, wq.groups) == (K, N, 2) and wq["totalBytes"] == 2 * N * 24
    a = smith.ones([1, K])
    out = smith.matmulQ4(a, wq)
    assert out.shape == [1, N]
    expected = smith.toNumpy(w).sum(axis=0)
    actual = np.array(smith.toArray(out))
    assert np.all(np.abs(actual[0] - expected) / (np.abs(expected) + 1e-6) < 0.15)
    # tests/inference.test.js:125-135
    wq2 = smith.quantizeQ4(smith.rand([256, 256]))
    assert wq2.totalBytes < 256 * 256 * 4 and wq2.totalBytes / (256 * 256 * 4) < 0.35


def test_operator_api_q8_and_profile():
    K, N, M = 256, 128, 4
    smith.tensor.seed(1)
    w, a = smith.randn([K, N]), smith.randn([M, K])
    wq = smith.quantizeQ8(w)
    assert wq.totalBytes == (K // 32) * N * 34
    out = smith.toNumpy(smith.matmulQ8(a, wq))
    packed = O.quantize_q8(smith.toNumpy(w))
    assert np.array_equal(device.download(wq.buffer, wq.totalBytes), packed)
    want = O.matmul(smith.toNumpy(a), packed, K, N, "q8")
    ok, worst = within_tolerance(out, want, smith.toNumpy(a), packed, K, N, "q8", REL)
    assert ok, worst
    p = smith.profileFn(lambda: smith.matmulQ8(a, wq))
    assert p["dispatches"] == 1 and p["kernels"][0]["kernel"] == "matmul_q8" and p["gpuMs"] >= 0
    b = smith.benchmark("q8", lambda: smith.matmulQ8(a, wq), warmup=1, iterations=3)
    assert b["iterations"] == 3 and b["gpu"]["min"] >= 0
    with pytest.raises(ValueError, match="matmulQ8: inner dims don't match: 256 vs 512"):
        smith.matmulQ8(a, {"buffer": wq.buffer, "K": 512, "N": N, "groups": 16})


def test_shared_weights_and_residency():
    # a caller-supplied SHARED packed buffer (the reference's own storage mode) works, staged or resident
    K, N, M = 128, 64, 3
    a_np, w_np = _data(2, M, K, N)
    packed = O.quantize_q4(w_np)
    buf = device.alloc(packed.size, device.SHARED)
    device.viewBuffer(buf, packed.size, np.uint8)[:] = packed
    a = smith.tensorFrom(a_np, [M, K])
    want = O.matmul(a_np, packed, K, N, "q4")
    wq = {"buffer": buf, "K": K, "N": N, "groups": K // 32}
    out1 = smith.toNumpy(smith.matmulQ4(a, wq))
    device.makeResident(buf)
    out2 = smith.toNumpy(smith.matmulQ4(a, wq))
    assert np.array_equal(out1, out2)
    assert within_tolerance(out1, want, a_np, packed, K, N, "q4", REL)[0]
    device.evict(buf)
    device.releaseBuffer(buf)


# ------------------------------------------------------------------ bridge behaviour
def test_bridge_info_and_self_tests():
    info = smith.info()
    assert "B200" in info["device"] or "NVIDIA" in info["device"]
    assert info["maxThreadgroupMemory"] >= 200 * 1024 and info["maxThreadsPerThreadgroup"] == 1024
    assert device.selfTest() == (1048576, 1048576)          # src/device.js:61-65 expects ~1 MiB twice
    with pytest.raises(device.SmithError, match="not found"):
        device.pipeline("no_such_kernel")
    with pytest.raises(device.SmithError, match="compilation"):
        device.compileSource("kernel void f() {}")


def test_bridge_buffers_and_errors():
    before = device.allocatedSize()
    b = device.alloc(4096, device.SHARED)
    assert device.bufferLength(b) == 4096 and device.bufferContents(b) and device.bufferRetainCount(b) == 1
    assert device.allocatedSize() == before + 4096
    p = device.alloc(4096, device.PRIVATE)
    assert device.bufferContents(p) is None and device.devicePtr(p)
    device.releaseBuffer(b)
    device.releaseBuffer(p)
    assert device.allocatedSize() == before
    # a launch whose buffers are too small for its parameters is refused on the host
    small = DevBuf(64)
    with pytest.raises(device.SmithError, match="needs"):
        device.qmatmul(4, small.handle, small.handle, small.handle, 4, 64, 64, 2, 0)
    a = smith.ones([1, 64])
    with pytest.raises(device.SmithError, match="needs"):
        smith.matmulQ4(a, {"buffer": small.handle, "K": 64, "N": 4096, "groups": 2})
    small.free()


def test_async_submit_and_graph_replay():
    K, N, M = 1024, 512, 1
    a_np, w_np = _data(4, M, K, N)
    packed = O.quantize_q4(w_np)
    ab, bb, cb = DevBuf.of(a_np), DevBuf.of(packed), DevBuf(M * N * 4)
    device.qmatmul(4, ab.handle, bb.handle, cb.handle, M, N, K, K // 32, 0)   # sizes any scratch before capture
    device.synchronize()
    first = cb.get(np.float32)
    device.upload(cb.handle, np.zeros(M * N, np.float32))
    n0 = device.launchCount()
    device.graphBegin()
    for _ in range(3):
        device.qmatmul(4, ab.handle, bb.handle, cb.handle, M, N, K, K // 32, 0)
    g = device.graphEnd()
    assert device.launchCount() - n0 >= 3
    device.graphLaunch(g)
    device.synchronize()
    assert np.array_equal(cb.get(np.float32), first)
    device.graphDestroy(g)
    # encoder path, asynchronous submit
    enc = device.begin()
    device.setPipeline(enc, device.pipeline("matmul_q4"))
    for i, h in enumerate((ab.handle, bb.handle, cb.handle)):
        device.setBuffer(enc, h, i)
    prm = np.array([M, N, K, K // 32], np.uint32)
    device.setBytes(enc, prm, prm.nbytes, 3)
    device.dispatch(enc, N, M, 1, 16, 1, 1)
    device.wait(device.endAsync(enc))
    assert np.array_equal(cb.get(np.float32), first)


# ------------------------------------------------------------------ fused all-gather epilogue (one GPU)
def test_fused_gather_world_of_one_and_alternating_halves():
    from smith_b200.parallel import FusedGather
    K, N, M = 2048, 1024, 2
    rng = np.random.default_rng(21)
    w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    packed = O.quantize_q4(w)
    pb = DevBuf.of(packed)
    fg = FusedGather(M, N, 1, 0)
    for call in range(3):                                   # halves 0, 1, 0: the counters keep counting
        a = rng.standard_normal((M, K)).astype(np.float32)
        ab = DevBuf.of(a)
        half = fg.enqueue(4, ab.handle, pb.handle, K)
        device.synchronize()
        assert half == call % 2 and device.kernelStatus() == 0
        want = matmul_on_device(a, packed, K, N, "q4", device.PATH_GEMV)
        assert bits_equal(fg.read(half), want)
        ab.free()
    fg.close()
    pb.free()


def test_fused_gather_deferred_chain_world_of_one():
    # deferred mode: no launch waits at its end; each waits for its predecessor's arrivals at its
    # start, and finish() closes the chain
    from smith_b200.parallel import FusedGather
    K, N, M = 1024, 2048, 1
    rng = np.random.default_rng(23)
    w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    packed = O.quantize_q4(w)
    pb = DevBuf.of(packed)
    fg = FusedGather(M, N, 1, 0, deferred=True)
    acts = [rng.standard_normal((M, K)).astype(np.float32) for _ in range(3)]
    abs_ = [DevBuf.of(a) for a in acts]
    halves = [fg.enqueue(4, ab.handle, pb.handle, K) for ab in abs_]      # back to back, no host wait between
    fg.finish()
    device.synchronize()
    assert device.kernelStatus() == 0 and halves == [0, 1, 0]
    assert bits_equal(fg.read(0), matmul_on_device(acts[2], packed, K, N, "q4", device.PATH_GEMV))
    assert bits_equal(fg.read(1), matmul_on_device(acts[1], packed, K, N, "q4", device.PATH_GEMV))
    fg.close()
    for b in abs_ + [pb]:
        b.free()


def test_fused_gather_deferred_chain_reads_its_previous_row():
    # each launch takes the row gathered by the launch before it as its activations, on the device
    from smith_b200.parallel import FusedGather
    K = N = 1024
    rng = np.random.default_rng(24)
    packs = [O.quantize_q4((rng.standard_normal((K, N)) * 0.05).astype(np.float32)) for _ in range(2)]
    pbs = [DevBuf.of(p) for p in packs]
    x0 = rng.standard_normal((1, K)).astype(np.float32)
    xb = DevBuf.of(x0)
    fg = FusedGather(1, N, 1, 0, deferred=True)
    steps = 5
    for i in range(steps):
        fg.enqueue(4, xb.handle, pbs[i & 1].handle, K, from_previous=i > 0)
    fg.finish()
    device.synchronize()
    assert device.kernelStatus() == 0
    want = x0
    for i in range(steps):
        want = matmul_on_device(want, packs[i & 1], K, N, "q4", device.PATH_GEMV)
    assert bits_equal(fg.read((steps - 1) & 1), want)
    fg.close()
    for b in pbs + [xb]:
        b.free()


def test_fused_gather_two_shards_emulated_on_one_gpu():
    # Two ranks' launches run one after the other on this GPU, each storing its column slice into
    # both ranks' rows.  The first launch is told to expect only its own tiles (its peer has not run
    # yet and two kernels that wait on each other must never share a GPU); the second expects both.
    K, N, M, world = 1024, 512, 3, 2
    rng = np.random.default_rng(22)
    w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    a = rng.standard_normal((M, K)).astype(np.float32)
    packed = O.quantize_q8(w)
    from smith_b200 import parallel as P
    ys = [DevBuf.of(np.zeros(2 * M * N, np.float32)) for _ in range(world)]
    states = [DevBuf.of(np.zeros(64, np.uint32)) for _ in range(world)]
    ab = DevBuf.of(a)
    tiles = []
    for r in range(world):
        n0, n1 = P.column_shard(N, world, r)
        tiles.append(device.qgemvTiles(8, M, n1 - n0, K))
        shard = DevBuf.of(P.slice_packed_columns(packed, K // 32, N, 34, n0, n1))
        device.qmatmulAllGather(8, ab.handle, shard.handle, M, N, n0, n1 - n0, K, K // 32, world, r,
                                [y.handle for y in ys], [s.handle for s in states], sum(tiles))
        device.synchronize()
        assert device.kernelStatus() == 0
        shard.free()
    want = matmul_on_device(a, packed, K, N, "q8", device.PATH_GENERIC)
    for r in range(world):
        got = ys[r].get(np.float32)[:M * N].reshape(M, N)
        ok, worst = within_tolerance(got, want, a, packed, K, N, "q8", REL)
        assert ok, (r, worst)
        st = states[r].get(np.uint32)[:4]
        assert st[2] == sum(tiles) and st[3] == 0 and st[1] == 0      # all arrivals counted, ticket reset
    assert states[0].get(np.uint32)[0] == 1 and states[1].get(np.uint32)[0] == 1  # each rank advanced one step
    for b in ys + states + [ab]:
        b.free()


# ------------------------------------------------------------------ several matrices sharing one launch
@pytest.mark.parametrize("kind,M,K,Ns", [("q4", 1, 4096, [4096, 1024, 1024]), ("q8", 3, 1024, [512, 2048]),
                                         ("q4", 2, 2048, [1000 // 8 * 8, 24, 4096, 136]), ("q4", 8, 1024, [256, 512]),
                                         # decode-kernel shapes whose activation digits live in scratch memory:
                                         # made once for the call, read by every product
                                         ("q4", 16, 4096, [4096, 1024, 1024]), ("q8", 12, 4096, [2048, 512]),
                                         ("q4", 16, 14336, [4096, 256])])
def test_qmatmul_multi_matches_one_launch_per_matrix(kind, M, K, Ns):
    rng = np.random.default_rng(41 + M)
    a = rng.standard_normal((M, K)).astype(np.float32)
    ab = DevBuf.of(a)
    packs, pbs, cbs = [], [], []
    for n in Ns:
        w = (rng.standard_normal((K, n)) * 0.02).astype(np.float32)
        packs.append(O.quantize_q4(w) if kind == "q4" else O.quantize_q8(w))
        pbs.append(DevBuf.of(packs[-1]))
        cbs.append(DevBuf.of(np.full(M * n, np.nan, np.float32)))
    launches0 = device.launchCount()
    device.qmatmulMulti(4 if kind == "q4" else 8, ab.handle, [b.handle for b in pbs], [b.handle for b in cbs], Ns, M, K,
                        K // 32)
    device.synchronize()
    assert device.kernelStatus() == 0
    if M <= 4:
        assert device.launchCount() - launches0 == 1        # one launch for all of them
    elif K >= 4096:
        assert device.launchCount() - launches0 == len(Ns) + 1      # one digit launch, one product launch per matrix
    for n, packed, cb in zip(Ns, packs, cbs):
        got = cb.get(np.float32).reshape(M, n)
        want = O.matmul(a, packed, K, n, kind, threads=O.host_threads())
        ok, worst = within_tolerance(got, want, a, packed, K, n, kind, REL)
        assert ok, (n, worst)
        if M > 4:                                                    # the same bits as a call of its own
            assert bits_equal(got, matmul_on_device(a, packed, K, n, kind))
    for b in pbs + cbs + [ab]:
        b.free()


# ------------------------------------------------------------------ fused all-reduce epilogue (one GPU)
def test_fused_reduce_world_of_one_and_alternating_halves():
    from smith_b200.parallel import FusedReduce
    K, N, M = 2048, 1024, 2
    rng = np.random.default_rng(31)
    w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    packed = O.quantize_q4(w)
    pb = DevBuf.of(packed)
    out = DevBuf.of(np.zeros(M * N, np.float32))
    fr = FusedReduce(4, M, N, K, 1, 0)
    for call in range(3):                                   # halves 0, 1, 0; flags keep counting
        a = rng.standard_normal((M, K)).astype(np.float32)
        ab = DevBuf.of(a)
        fr.enqueue(ab.handle, pb.handle, out.handle)
        device.synchronize()
        assert device.kernelStatus() == 0
        want = matmul_on_device(a, packed, K, N, "q4", device.PATH_GEMV)
        got = out.get(np.float32).reshape(M, N)
        assert np.array_equal(got, want)                    # 0 + x: the one partial, unchanged
        ab.free()
    assert device.download(fr.state, 16, np.uint32)[0] == 3    # three steps completed
    fr.close()
    for b in (pb, out):
        b.free()


def test_fused_reduce_two_k_shards_with_a_preseeded_peer():
    # Rank 0 of a world of two runs alone on this GPU.  Its peer's slot (tagged partial sums for the
    # first two steps) is written by the host beforehand, so the launch never waits on another launch
    # (two kernels that wait on each other must never share a GPU); what is checked is rank 0's side
    # of the protocol: its partials pushed with the step's tag into its slot on both ranks, the
    # slots added in rank order.
    from smith_b200 import parallel as P
    K, N, M, world = 2048, 1536, 3, 2
    rng = np.random.default_rng(32)
    w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    a = rng.standard_normal((M, K)).astype(np.float32)
    packed = O.quantize_q8(w)
    G = K // 32
    g0, g1 = P.group_shard(G, world, 0)
    h0, h1 = P.group_shard(G, world, 1)
    kl = (g1 - g0) * 32
    peer_partial = O.matmul(a[:, h0 * 32:h1 * 32], P.slice_packed_groups(packed, G, N, 34, h0, h1), (h1 - h0) * 32, N, "q8")
    assert device.qmatmulAllReduceStateBytes(8, M, N, kl) == 16
    # slots [2][world][M][N] of (value bits, tag): the peer's slot of half h carries tag h + 1
    slots = np.zeros((2, world, M * N, 2), np.uint32)
    for h in range(2):
        slots[h, 1, :, 0] = peer_partial.reshape(-1).view(np.uint32)
        slots[h, 1, :, 1] = h + 1
    partials = [DevBuf.of(slots), DevBuf.of(np.zeros_like(slots))]
    states = [DevBuf.of(np.zeros(64, np.uint32)), DevBuf.of(np.zeros(64, np.uint32))]
    ab = DevBuf.of(np.ascontiguousarray(a[:, g0 * 32:g1 * 32]))
    shard = DevBuf.of(P.slice_packed_groups(packed, G, N, 34, g0, g1))
    out = DevBuf.of(np.zeros(M * N, np.float32))
    want = matmul_on_device(a, packed, K, N, "q8", device.PATH_GENERIC)
    for call in range(2):                                   # both halves
        device.qmatmulAllReduce(8, ab.handle, shard.handle, out.handle, M, N, kl, kl // 32, world, 0,
                                [b.handle for b in partials], [b.handle for b in states])
        device.synchronize()
        assert device.kernelStatus() == 0
        got = out.get(np.float32).reshape(M, N)
        ok, worst = within_tolerance(got, want, a, packed, K, N, "q8", REL)
        assert ok, (call, worst)
        mine = partials[0].get(np.uint32).reshape(2, world, M * N, 2)
        own = mine[call, 0, :, 0].copy().view(np.float32).reshape(M, N)
        assert (mine[call, 0, :, 1] == call + 1).all()      # own partials carry this step's tag
        assert np.array_equal(got, own + peer_partial)      # rank order: own partial first, then the peer's
        at_peer = partials[1].get(np.uint32).reshape(2, world, M * N, 2)
        assert np.array_equal(at_peer[call, 0], mine[call, 0])   # ... and went to the peer's memory too
    assert states[0].get(np.uint32)[0] == 2                 # two steps completed
    for b in partials + states + [ab, shard, out]:
        b.free()


# ------------------------------------------------------------------ full-size projection shapes, sampled columns
# Every Q4 linear projection of a Llama-3-8B-shaped and a 70B-shaped decode step.  Weights are generated and packed on the device at full size; a window of columns is
# downloaded and checked against the oracle (packed bytes bit-exact, outputs within tolerance).
LLAMA_8B = [("wq", 4096, 4096), ("wk", 4096, 1024), ("wo", 4096, 4096), ("gate", 4096, 14336), ("down", 14336, 4096),
            ("lm_head", 4096, 128256)]
LLAMA_70B = [("wq", 8192, 8192), ("wk", 8192, 1024), ("gate", 8192, 28672), ("down", 28672, 8192)]


def _check_projection(K, N, Ms, std, seed, kind="q4", windows=None):
    """Full-size weights generated and packed on the device; windows of 48 columns are brought back
    and checked: packed bytes bit-exact against the CPU packer on the same f32 columns, outputs within
    tolerance of the oracle for every M."""
    G = K // 32
    bb = 24 if kind == "q4" else 34
    k4 = 4 if kind == "q4" else 8
    wb = DevBuf(K * N * 4)
    device.fillNormal(wb.handle, K * N, seed, std)
    pb = DevBuf(G * N * bb)
    (device.q4Pack if kind == "q4" else device.q8Pack)(wb.handle, pb.handle, K, N)
    device.synchronize()
    starts = windows if windows is not None else [(N // 2) // 8 * 8]
    full_rows = wb.get(np.float32).reshape(K, N) if K * N <= (1 << 26) else None
    cols = []
    for c0 in starts:
        c1 = min(N, c0 + 48)
        w_cols = np.empty((K, c1 - c0), np.float32)
        if full_rows is not None:
            w_cols[:] = full_rows[:, c0:c1]
        else:                                               # too large to bring back whole: row by row
            for k in range(K):
                w_cols[k] = device.download(wb.handle, (c1 - c0) * 4, np.float32, offset=(k * N + c0) * 4)
        packed_cols = np.empty((G, (c1 - c0) * bb), np.uint8)
        for g in range(G):
            packed_cols[g] = device.download(pb.handle, (c1 - c0) * bb, np.uint8, offset=(g * N + c0) * bb)
        packed_cols = packed_cols.reshape(-1)
        want = O.quantize_q4(w_cols) if kind == "q4" else O.quantize_q8(w_cols)
        assert np.array_equal(packed_cols, want), f"packed bytes of columns [{c0}, {c1}) differ from the oracle"
        cols.append((c0, c1, packed_cols))
    wb.free()
    rng = np.random.default_rng(seed)
    for M in Ms:
        a = rng.standard_normal((M, K)).astype(np.float32)
        ab, cb = DevBuf.of(a), DevBuf(M * N * 4)
        device.qmatmul(k4, ab.handle, pb.handle, cb.handle, M, N, K, G, device.PATH_AUTO)
        device.synchronize()
        assert device.kernelStatus() == 0
        out = cb.get(np.float32).reshape(M, N)
        assert np.all(np.isfinite(out))
        for c0, c1, packed_cols in cols:
            want = O.matmul(a, packed_cols, K, c1 - c0, kind, threads=O.host_threads())
            ok, worst = within_tolerance(out[:, c0:c1], want, a, packed_cols, K, c1 - c0, kind, REL)
            assert ok, f"K={K} N={N} M={M} columns [{c0}, {c1}): worst err/bound = {worst}"
        ab.free()
        cb.free()
    pb.free()


# The two stated benchmark configurations at their full shapes.
@pytest.mark.parametrize("seed", [0, 1, 2, 3])
def test_q8_prefill_gemm_512x4096x11008_full_shape(seed):
    """Q8 prefill GEMM: activations [512, 4096] ~N(0,1), weight [4096, 11008] ~N(0,0.02) packed by
    quantizeQ8, seeds 0..3; three windows of columns (first, middle, last) against the oracle."""
    _check_projection(4096, 11008, (512,), 0.02, seed, kind="q8", windows=[0, 5496, 11008 - 48])


def test_q4_decode_and_skinny_sweep_4096x14336_full_shape():
    """Q4 weight [4096, 14336] ~N(0,0.02); activations [M, 4096] for M in {1, 4, 16, 64, 256}: every
    dispatch path (GEMV, decode, tensor) at the shape the decode target is quoted on."""
    _check_projection(4096, 14336, (1, 4, 16, 64, 256), 0.02, 0, kind="q4", windows=[0, 7168, 14336 - 48])


@pytest.mark.parametrize("name,K,N", LLAMA_8B)
def test_llama_8b_shaped_projections(name, K, N):
    _check_projection(K, N, (1, 16), 0.02, 40 + len(name))


@pytest.mark.parametrize("name,K,N", LLAMA_70B)
def test_llama_70b_shaped_projections(name, K, N):
    _check_projection(K, N, (1, 32, 256), 0.015, 70 + len(name))


def test_packed_weights_save_and_load_round_trip(tmp_path):
    """saveQuantized / loadQuantized: the packed bytes come back bit for bit and multiply the same."""
    rng = np.random.default_rng(77)
    K, N = 512, 264
    w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    a = rng.standard_normal((2, K)).astype(np.float32)
    wt, at = smith.tensorFrom(w, [K, N]), smith.tensorFrom(a, [2, K])
    q4, q8 = smith.quantizeQ4(wt), smith.quantizeQ8(wt)
    path = str(tmp_path / "packed")
    smith.saveQuantized({"layer0.wq": ("q4", q4), "layer0.wk": ("q8", q8)}, path)
    back = smith.loadQuantized(path)
    assert list(back) == ["layer0.wq", "layer0.wk"] and back["layer0.wq"][0] == "q4" and back["layer0.wk"][0] == "q8"
    for name, rec in (("layer0.wq", q4), ("layer0.wk", q8)):
        got = back[name][1]
        assert (got.K, got.N, got.groups, got.totalBytes) == (rec.K, rec.N, rec.groups, rec.totalBytes)
        assert np.array_equal(device.download(got.buffer, got.totalBytes), device.download(rec.buffer, rec.totalBytes))
    y0 = smith.toNumpy(smith.matmulQ4(at, q4))
    y1 = smith.toNumpy(smith.matmulQ4(at, back["layer0.wq"][1]))
    assert np.array_equal(y0.view(np.uint32), y1.view(np.uint32))
    import json
    manifest = json.load(open(path + ".json"))
    manifest["totalBytes"] += 1
    json.dump(manifest, open(path + ".json", "w"))
    with pytest.raises(ValueError):
        smith.loadQuantized(path)


def test_profile_report_carries_bandwidth_and_roofline():
    rng = np.random.default_rng(78)
    K, N = 4096, 1792
    wt = smith.tensorFrom((rng.standard_normal((K, N)) * 0.02).astype(np.float32), [K, N])
    at = smith.tensorFrom(rng.standard_normal((1, K)).astype(np.float32), [1, K])
    wq = smith.quantizeQ4(wt)
    prof = smith.profileFn(lambda: [smith.dispose(smith.matmulQ4(at, wq)) for _ in range(5)])
    mm = next(k for k in prof["kernels"] if k["kernel"] == "matmul_q4")
    assert mm["calls"] == 5 and mm["gbs"] > 10 and 0 < mm["pctRoofline"] <= 110 and mm["bound"] == "hbm"


@pytest.mark.parametrize("ggml_type,M", [(8, 1), (8, 64), (2, 1), (2, 3), (2, 96)])
def test_gguf_blocks_run_on_the_quantized_path(ggml_type, M):
    """Q8_0 / Q4_0 blocks as they lie in a GGUF file, re-tiled on the device (smith_gguf_repack), then
    matmulQ8 / matmulQ4: the result is held to the matmul tolerance against the reference's own route
    (de-quantise every block to f32, src/gguf.js:187-231; transpose, src/gguf_loader.js:236-252;
    sequential f32 product), and the re-tiled bytes de-quantise to exactly those f32 weights."""
    rng = np.random.default_rng(ggml_type * 10 + M)
    out_dim, in_dim = 1032, 2048                       # N (not a multiple of 256), K
    G = in_dim // 32
    per = 34 if ggml_type == 8 else 18
    blocks = rng.integers(0, 256, (out_dim, G, per), dtype=np.uint8)
    blocks[:, :, 0] = rng.integers(0, 256, (out_dim, G))
    blocks[:, :, 1] = rng.integers(0x1C, 0x24, (out_dim, G))      # f16 scales around 2^-8 .. 2^-6
    w_file = O.gguf_dequant(ggml_type, blocks).reshape(out_dim, in_dim)
    kind, rec = smith.quantizedFromGGUF(blocks, ggml_type, [out_dim, in_dim])
    knd = "q8" if ggml_type == 8 else "q4"
    assert kind == knd and (rec.K, rec.N, rec.groups) == (in_dim, out_dim, G)
    packed = device.download(rec.buffer, rec.totalBytes)
    assert np.array_equal(O.dequant(packed, in_dim, out_dim, knd).view(np.uint32), w_file.T.copy().view(np.uint32))
    a = rng.standard_normal((M, in_dim)).astype(np.float32)
    at = smith.tensorFrom(a, [M, in_dim])
    got = smith.toNumpy((smith.matmulQ8 if ggml_type == 8 else smith.matmulQ4)(at, rec))
    want = O.matmul(a, packed, in_dim, out_dim, knd, threads=O.host_threads())
    ok, worst = within_tolerance(got, want, a, packed, in_dim, out_dim, knd, REL)
    assert ok, worst
    with pytest.raises(ValueError):
        smith.quantizedFromGGUF(blocks, 3, [out_dim, in_dim])     # Q4_1: not the shaders' arithmetic
    device.releaseBuffer(rec.buffer)
