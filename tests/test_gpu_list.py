"""-m gpu: smith_qmatmul_list (a list of GEMV-shaped products as one persistent launch, with
RMSNorm / SwiGLU / residual folded in) against the oracle and against one launch per matrix.

The oracle side restates what the reference's decode step does between its matmuls
(src/gguf_cache.js:121-171): rmsnormForward -> linear; linear -> A.add; swigluForward(gate, up).
Matmul outputs are held to max |delta| <= 1e-3 * ||x_m|| * ||w_deq[:,n]||; a stage that applies a
pointwise function after the product is checked on inputs taken from the device's own previous
stage, so every stage is held to that bound by itself."""
import numpy as np
import pytest

from gpu_util import DevBuf
from helpers import within_tolerance
from oracle import oracle as O
from smith_b200 import device

pytestmark = pytest.mark.gpu

REL = 1e-3


def _pack(w, kind):
    return O.quantize_q4(w) if kind == "q4" else O.quantize_q8(w)


def _kind(kind):
    return 4 if kind == "q4" else 8


def _run(lst, times=1):
    for _ in range(times):
        device.qmatmulListRun(lst)
    device.synchronize()
    assert device.kernelStatus() == 0, "a bounded device-side wait gave up"


@pytest.mark.parametrize("kind", ["q4", "q8"])
@pytest.mark.parametrize("M", [1, 2, 3, 4])
def test_list_of_independent_matrices_matches_oracle_and_single_launches(kind, M):
    """Matrices of different shapes, no hazards: every output within tolerance of the oracle and
    within a few ulps-of-the-bound of the one-launch-per-matrix GEMV."""
    rng = np.random.default_rng(100 + M)
    shapes = [(256, 512), (512, 1024), (1024, 264), (4096, 1792), (2048, 4096), (32, 8), (4096, 1184)]
    bufs, items, want = [], [], []
    for K, N in shapes:
        w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
        a = rng.standard_normal((M, K)).astype(np.float32)
        packed = _pack(w, kind)
        ab, pb, cb = DevBuf.of(a), DevBuf.of(packed), DevBuf(M * N * 4)
        bufs.append((ab, pb, cb))
        items.append(device.listItem(ab.handle, pb.handle, cb.handle, N, K))
        want.append((a, packed, K, N))
    lst = device.qmatmulListCreate(_kind(kind), M, items)
    _run(lst)
    for (ab, pb, cb), (a, packed, K, N) in zip(bufs, want):
        got = cb.get(np.float32).reshape(M, N)
        ref = O.matmul(a, packed, K, N, kind, threads=O.host_threads())
        ok, worst = within_tolerance(got, ref, a, packed, K, N, kind, REL)
        assert ok, f"K={K} N={N}: worst err/bound = {worst}"
        one = DevBuf(M * N * 4)
        device.qmatmul(_kind(kind), ab.handle, pb.handle, one.handle, M, N, K, K // 32, device.PATH_GENERIC)
        device.synchronize()
        ok, worst = within_tolerance(got, one.get(np.float32).reshape(M, N), a, packed, K, N, kind, REL)
        assert ok, worst
        one.free()
    # a second and third run of the same list (the counters were restored) give the same bits
    first = [cb.get(np.float32).copy() for _, _, cb in bufs]
    for _, _, cb in bufs:
        device.upload(cb.handle, np.zeros(cb.nbytes // 4, np.float32))
    _run(lst, times=2)
    for f, (_, _, cb) in zip(first, bufs):
        assert np.array_equal(f.view(np.uint32), cb.get(np.uint32))
    device.qmatmulListDestroy(lst)
    for t in bufs:
        for b in t:
            b.free()


def test_list_same_matrix_many_times_and_graph_replay():
    """Twelve 4096 x 1792 matrices on one input (the benchmark's shape of list), replayed from a graph."""
    rng = np.random.default_rng(7)
    M, K, N, R = 1, 4096, 1792, 12
    a = rng.standard_normal((M, K)).astype(np.float32)
    ab = DevBuf.of(a)
    mats, outs, items = [], [], []
    for r in range(R):
        w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
        packed = O.quantize_q4(w)
        pb, cb = DevBuf.of(packed), DevBuf(M * N * 4)
        mats.append((packed, pb))
        outs.append(cb)
        items.append(device.listItem(ab.handle, pb.handle, cb.handle, N, K))
    lst = device.qmatmulListCreate(4, M, items)
    _run(lst)                                          # first run outside capture
    device.graphBegin()
    device.qmatmulListRun(lst)
    device.qmatmulListRun(lst)
    g = device.graphEnd()
    for cb in outs:
        device.upload(cb.handle, np.zeros(M * N, np.float32))
    for _ in range(3):
        device.graphLaunch(g)
    device.synchronize()
    assert device.kernelStatus() == 0
    for (packed, _), cb in zip(mats, outs):
        got = cb.get(np.float32).reshape(M, N)
        ref = O.matmul(a, packed, K, N, "q4", threads=O.host_threads())
        ok, worst = within_tolerance(got, ref, a, packed, K, N, "q4", REL)
        assert ok, worst
    device.graphDestroy(g)
    device.qmatmulListDestroy(lst)
    for _, pb in mats:
        pb.free()
    for cb in outs:
        cb.free()
    ab.free()


@pytest.mark.parametrize("M", [1, 4])
def test_list_chain_reads_what_earlier_items_wrote(M):
    """y1 = x W1; y2 = y1 W2; y3 = y2 W3 written over x's buffer (read-after-write twice, then a
    write-after-read): each stage against the oracle on the device's own input to that stage."""
    rng = np.random.default_rng(11)
    d0, d1, d2 = 1024, 2048, 512
    ws = [(rng.standard_normal((d0, d1)) * 0.05).astype(np.float32),
          (rng.standard_normal((d1, d2)) * 0.05).astype(np.float32),
          (rng.standard_normal((d2, d0)) * 0.05).astype(np.float32)]
    packed = [O.quantize_q4(w) for w in ws]
    x = rng.standard_normal((M, d0)).astype(np.float32)
    xb, y1, y2 = DevBuf.of(x), DevBuf(M * d1 * 4), DevBuf(M * d2 * 4)
    keep = DevBuf(M * d0 * 4)                          # a copy of y3's input chain end, to check the overwrite
    pbs = [DevBuf.of(p) for p in packed]
    items = [device.listItem(xb.handle, pbs[0].handle, y1.handle, d1, d0),
             device.listItem(y1.handle, pbs[1].handle, y2.handle, d2, d1),
             device.listItem(y2.handle, pbs[2].handle, xb.handle, d0, d2)]       # overwrites x
    lst = device.qmatmulListCreate(4, M, items)
    _run(lst)
    g1 = y1.get(np.float32).reshape(M, d1)
    g2 = y2.get(np.float32).reshape(M, d2)
    g3 = xb.get(np.float32).reshape(M, d0)
    for got, inp, p, K, N in ((g1, x, packed[0], d0, d1), (g2, g1, packed[1], d1, d2), (g3, g2, packed[2], d2, d0)):
        ref = O.matmul(inp, p, K, N, "q4", threads=O.host_threads())
        ok, worst = within_tolerance(got, ref, inp, p, K, N, "q4", REL)
        assert ok, f"K={K} N={N}: worst err/bound = {worst}"
    device.qmatmulListDestroy(lst)
    for b in [xb, y1, y2, keep] + pbs:
        b.free()


def _layer_weights(rng, dim, kv, ffn, std):
    names = [("wq", dim, dim), ("wk", dim, kv), ("wv", dim, kv), ("wo", dim, dim), ("gate", dim, ffn),
             ("up", dim, ffn), ("down", ffn, dim)]
    return {n: (rng.standard_normal((k, m)) * std).astype(np.float32) for n, k, m in names}


@pytest.mark.parametrize("kind,M,dim,kv,ffn,layers", [("q4", 1, 1024, 256, 2816, 3), ("q4", 2, 512, 128, 1408, 2),
                                                      ("q8", 1, 1024, 256, 2816, 2), ("q4", 4, 256, 64, 704, 2)])
def test_list_decode_layers_with_fused_glue(kind, M, dim, kv, ffn, layers):
    """The projections of `layers` Llama-shaped decode layers with the glue of
    src/gguf_cache.js:121-165 folded in (attention itself is outside the path: a fixed synthetic
    row stands in for its output).  Per layer:
        q,k,v = rmsnorm(x, ln1) W{q,k,v};  x2 = x + attn Wo;
        h = silu(rmsnorm(x2, ln2) Wgate) * (rmsnorm(x2, ln2) Wup);  x = x2 + h Wdown
    Every stage is checked against the oracle's rmsnorm / matmul / swiglu on the device's own inputs
    to that stage."""
    rng = np.random.default_rng(dim + M)
    eps = 1e-5
    x0 = rng.standard_normal((M, dim)).astype(np.float32)
    attn = rng.standard_normal((M, dim)).astype(np.float32)
    xs = [DevBuf.of(x0)] + [DevBuf(M * dim * 4) for _ in range(layers)]     # residual stream after each layer
    x2s = [DevBuf(M * dim * 4) for _ in range(layers)]
    attn_b = DevBuf.of(attn)
    items, per_layer, keep = [], [], []
    for l in range(layers):
        w = _layer_weights(rng, dim, kv, ffn, 0.04)
        p = {n: _pack(v, kind) for n, v in w.items()}
        pb = {n: DevBuf.of(v) for n, v in p.items()}
        ln1 = (1.0 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
        ln2 = (1.0 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
        g1, g2 = DevBuf.of(ln1), DevBuf.of(ln2)
        q, k, v, h = DevBuf(M * dim * 4), DevBuf(M * kv * 4), DevBuf(M * kv * 4), DevBuf(M * ffn * 4)
        x_in, x2, x_out = xs[l], x2s[l], xs[l + 1]
        items += [
            device.listItem(x_in.handle, pb["wq"].handle, q.handle, dim, dim, gamma=g1.handle, eps=eps),
            device.listItem(x_in.handle, pb["wk"].handle, k.handle, kv, dim, gamma=g1.handle, eps=eps),
            device.listItem(x_in.handle, pb["wv"].handle, v.handle, kv, dim, gamma=g1.handle, eps=eps),
            device.listItem(attn_b.handle, pb["wo"].handle, x2.handle, dim, dim, residual=x_in.handle),
            device.listItem(x2.handle, pb["gate"].handle, h.handle, ffn, dim, b2=pb["up"].handle, gamma=g2.handle, eps=eps),
            device.listItem(h.handle, pb["down"].handle, x_out.handle, dim, ffn, residual=x2.handle),
        ]
        per_layer.append((p, ln1, ln2, q, k, v, h))
        keep += list(pb.values()) + [g1, g2]
    lst = device.qmatmulListCreate(_kind(kind), M, items)
    _run(lst, times=2)                                 # the second run recomputes the same values
    T = O.host_threads()

    def check(got, inp, packed, K, N, what, post=None):
        ref = O.matmul(inp, packed, K, N, kind, threads=T)
        if post is not None:
            ref = post(ref)
        ok, worst = within_tolerance(got, ref, inp, packed, K, N, kind, REL)
        assert ok, f"{what}: worst err/bound = {worst}"

    for l, (p, ln1, ln2, q, k, v, h) in enumerate(per_layer):
        x_in = xs[l].get(np.float32).reshape(M, dim)
        x2 = x2s[l].get(np.float32).reshape(M, dim)
        x_out = xs[l + 1].get(np.float32).reshape(M, dim)
        n1 = O.rmsnorm(x_in, ln1, eps)
        check(q.get(np.float32).reshape(M, dim), n1, p["wq"], dim, dim, f"layer {l} wq")
        check(k.get(np.float32).reshape(M, kv), n1, p["wk"], dim, kv, f"layer {l} wk")
        check(v.get(np.float32).reshape(M, kv), n1, p["wv"], dim, kv, f"layer {l} wv")
        check(x2, attn, p["wo"], dim, dim, f"layer {l} wo + residual", post=lambda r: x_in + r)
        n2 = O.rmsnorm(x2, ln2, eps)
        # SwiGLU: |d(silu(g) u)| <= 1.1 |u| |dg| + |silu(g)| |du|; compare through the oracle's own gate / up
        gate = O.matmul(n2, p["gate"], dim, ffn, kind, threads=T)
        up = O.matmul(n2, p["up"], dim, ffn, kind, threads=T)
        want = O.swiglu(gate, up)
        got = h.get(np.float32).reshape(M, ffn)
        bg = O.tolerance_bound(n2, O.dequant(p["gate"], dim, ffn, kind), REL)
        bu = O.tolerance_bound(n2, O.dequant(p["up"], dim, ffn, kind), REL)
        silu = np.abs(gate / (1.0 + np.exp(-gate.astype(np.float64))))
        bound = 1.1 * np.abs(up) * bg + silu * bu + 1e-6 * np.abs(want) + 1e-30
        err = np.abs(got.astype(np.float64) - want)
        assert np.all(err <= bound), f"layer {l} swiglu(gate, up): worst err/bound = {(err / bound).max()}"
        check(x_out, got, p["down"], ffn, dim, f"layer {l} down + residual", post=lambda r: x2 + r)
    device.qmatmulListDestroy(lst)
    for b in xs + x2s + [attn_b] + keep:
        b.free()
    for _, _, _, q, k, v, h in per_layer:
        for b in (q, k, v, h):
            b.free()


def test_list_chain_through_channels(monkeypatch):
    """The same chain with SMITH_LIST_CHANNELS set: read-after-write hazards then travel as tagged
    {value, launch tag} pairs instead of through the counters (the mechanism the multi-GPU rows use)."""
    monkeypatch.setenv("SMITH_LIST_CHANNELS", "1")
    test_list_chain_reads_what_earlier_items_wrote(2)
    test_list_decode_layers_with_fused_glue("q4", 1, 1024, 256, 2816, 3)


def test_rmsnorm_prologue_alone_matches_oracle_to_rounding():
    """An identity-like check of the fused RMSNorm: with a one-hot-column weight the product is
    (code * scale) * normalised x[k], so the normalised row can be read back through the matmul."""
    rng = np.random.default_rng(3)
    M, K, N = 2, 2048, 64
    x = (rng.standard_normal((M, K)) * 3).astype(np.float32)
    gamma = (1.0 + 0.2 * rng.standard_normal(K)).astype(np.float32)
    w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    packed = O.quantize_q4(w)
    xb, gb, pb, cb = DevBuf.of(x), DevBuf.of(gamma), DevBuf.of(packed), DevBuf(M * N * 4)
    lst = device.qmatmulListCreate(4, M, [device.listItem(xb.handle, pb.handle, cb.handle, N, K, gamma=gb.handle, eps=1e-6)])
    _run(lst)
    n = O.rmsnorm(x, gamma, 1e-6)
    ref = O.matmul(n, packed, K, N, "q4")
    ok, worst = within_tolerance(cb.get(np.float32).reshape(M, N), ref, n, packed, K, N, "q4", REL)
    assert ok, worst
    device.qmatmulListDestroy(lst)
    for b in (xb, gb, pb, cb):
        b.free()


def test_list_refusals():
    rng = np.random.default_rng(1)
    K, N = 256, 64
    pb = DevBuf.of(O.quantize_q4((rng.standard_normal((K, N)) * 0.02).astype(np.float32)))
    ab, cb = DevBuf(4 * K * 4), DevBuf(4 * N * 4)
    with pytest.raises(device.SmithError):             # N not a multiple of 8
        device.qmatmulListCreate(4, 1, [device.listItem(ab.handle, pb.handle, cb.handle, 63, K)])
    with pytest.raises(device.SmithError):             # M too large for the GEMV arithmetic
        device.qmatmulListCreate(4, 5, [device.listItem(ab.handle, pb.handle, cb.handle, N, K)])
    with pytest.raises(device.SmithError):             # output buffer too small
        device.qmatmulListCreate(4, 4, [device.listItem(ab.handle, pb.handle, cb.handle, N, K, cOffset=64)])
    with pytest.raises(device.SmithError):             # output over the item's own input
        device.qmatmulListCreate(4, 1, [device.listItem(ab.handle, pb.handle, ab.handle, N, K)])
    with pytest.raises(device.SmithError):             # empty
        device.qmatmulListCreate(4, 1, [])
    assert device.qmatmulListSupports(4, 1, 14336, 4096)
    assert not device.qmatmulListSupports(4, 1, 14336, 4100)
    for b in (pb, ab, cb):
        b.free()


# ------------------------------------------------------------------ fused all-gather (weights sharded along N)
def _shard(packed, K, N, bb, n0, n1):
    from smith_b200 import parallel as P
    return P.slice_packed_columns(packed, K // 32, N, bb, n0, n1)


def test_list_gather_world_of_one_alternates_halves():
    """A list whose items end in the fused all-gather, with this GPU as the only rank: the rows hold
    {value, tag} pairs, launch t fills half t % 2 with tag t."""
    from smith_b200 import parallel as P
    rng = np.random.default_rng(21)
    M, K, N, R = 2, 1024, 2048, 5
    a = rng.standard_normal((M, K)).astype(np.float32)
    ab = DevBuf.of(a)
    packed = [O.quantize_q4((rng.standard_normal((K, N)) * 0.02).astype(np.float32)) for _ in range(R)]
    pbs = [DevBuf.of(p) for p in packed]
    sl = P.ShardedList(4, M, K, N, [b.handle for b in pbs], 1, 0, ab.handle)
    for launch in (1, 2, 3):
        sl.run()
        device.synchronize()
        assert device.kernelStatus() == 0
        for i in range(R):
            row, tags = sl.read(i)
            assert np.all(tags == launch)
            ref = O.matmul(a, packed[i], K, N, "q4", threads=O.host_threads())
            ok, worst = within_tolerance(row, ref, a, packed[i], K, N, "q4", REL)
            assert ok, worst
            # the plain local slice holds the same values
            local = device.download(sl.local[i], M * N * 4, np.uint32)
            assert np.array_equal(local, row.view(np.uint32).reshape(-1))
    sl.close()
    for b in pbs + [ab]:
        b.free()


def test_list_gather_two_shards_emulated_on_one_gpu():
    """Two ranks' lists, both on this GPU and sharing the two 'ranks' row buffers, launched one after
    the other (never two launches that wait on each other on one GPU: the closing wait is off)."""
    from smith_b200 import parallel as P
    rng = np.random.default_rng(22)
    M, K, N, R, world = 1, 2048, 4096, 3, 2
    a = rng.standard_normal((M, K)).astype(np.float32)
    ab = DevBuf.of(a)
    packed = [O.quantize_q4((rng.standard_normal((K, N)) * 0.02).astype(np.float32)) for _ in range(R)]
    row_bytes = 2 * M * N * 8
    rows = [DevBuf.of(np.zeros(R * row_bytes // 4, np.uint32)) for _ in range(world)]
    lists, keep = [], []
    for rank in range(world):
        n0, n1 = P.column_shard(N, world, rank)
        shards = [DevBuf.of(_shard(p, K, N, 24, n0, n1)) for p in packed]
        outs = [DevBuf((n1 - n0) * M * 4) for _ in range(R)]
        views = [[device.wrapDeviceMemory(device.devicePtr(rows[r].handle) + i * row_bytes, row_bytes) for r in range(world)]
                 for i in range(R)]
        items = [device.listItem(ab.handle, sh.handle, o.handle, n1 - n0, K) for sh, o in zip(shards, outs)]
        gathers = [device.listGather(world, n0, N, views[i]) for i in range(R)]
        lists.append(device.qmatmulListCreateGather(4, M, items, gathers, rank, device.LIST_NO_CLOSING_WAIT))
        keep += shards + outs
    for launch in (1, 2):
        for lst in lists:                              # rank 0's launch, then rank 1's
            device.qmatmulListRun(lst)
            device.synchronize()
        assert device.kernelStatus() == 0
        half = launch & 1
        for r in range(world):                         # both ranks' rows are whole and equal
            for i in range(R):
                pairs = device.download(rows[r].handle, M * N * 8, np.uint32, offset=i * row_bytes + half * M * N * 8).reshape(-1, 2)
                assert np.all(pairs[:, 1] == launch)
                row = np.ascontiguousarray(pairs[:, 0]).view(np.float32).reshape(M, N)
                ref = O.matmul(a, packed[i], K, N, "q4", threads=O.host_threads())
                ok, worst = within_tolerance(row, ref, a, packed[i], K, N, "q4", REL)
                assert ok, worst
    for lst in lists:
        device.qmatmulListDestroy(lst)
    for b in keep + rows + [ab]:
        b.free()


def test_bounded_wait_gives_up_when_a_peer_never_arrives():
    """Failure detection without any fault: a two-rank gather list whose peer never runs.  The closing
    wait of the launch runs out (~0.2 s), the kernel returns by itself, smith_kernel_status reports 1,
    and the context stays usable: an ordinary product afterwards is correct and the status is clear."""
    import time
    from smith_b200 import parallel as P
    rng = np.random.default_rng(23)
    M, K, N, world = 1, 1024, 2048, 2
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    packed = O.quantize_q4(w)
    ab = DevBuf.of(a)
    n0, n1 = P.column_shard(N, world, 0)
    shard, out = DevBuf.of(_shard(packed, K, N, 24, n0, n1)), DevBuf(M * (n1 - n0) * 4)
    rows = [DevBuf.of(np.zeros(2 * M * N * 2, np.uint32)) for _ in range(world)]    # the peer's slice stays empty
    lst = device.qmatmulListCreateGather(4, M, [device.listItem(ab.handle, shard.handle, out.handle, n1 - n0, K)],
                                         [device.listGather(world, n0, N, [r.handle for r in rows])], 0)
    t0 = time.perf_counter()
    device.qmatmulListRun(lst)
    device.synchronize()
    waited = time.perf_counter() - t0
    assert device.kernelStatus() == 1, "the closing wait should have given up"
    assert waited < 5.0
    assert device.kernelStatus() == 0                   # reading the status clears it
    # this rank's own slice did arrive (launch 1, half 1) and the plain output is right
    pairs = device.download(rows[0].handle, M * N * 8, np.uint32, offset=M * N * 8).reshape(-1, 2)
    assert np.all(pairs[n0:n1, 1] == 1) and np.all(pairs[n1:, 1] == 0)
    ref = O.matmul(a, packed, K, N, "q4")
    got = out.get(np.float32).reshape(M, n1 - n0)
    ok, worst = within_tolerance(got, ref[:, n0:n1], a, _shard(packed, K, N, 24, n0, n1), K, n1 - n0, "q4", REL)
    assert ok, worst
    # an ordinary product on the same context afterwards
    pb, cb = DevBuf.of(packed), DevBuf(M * N * 4)
    device.qmatmul(4, ab.handle, pb.handle, cb.handle, M, N, K, K // 32, device.PATH_AUTO)
    device.synchronize()
    assert device.kernelStatus() == 0
    ok, worst = within_tolerance(cb.get(np.float32).reshape(M, N), ref, a, packed, K, N, "q4", REL)
    assert ok, worst
    device.qmatmulListDestroy(lst)
    for b in [ab, shard, out, pb, cb] + rows:
        b.free()
