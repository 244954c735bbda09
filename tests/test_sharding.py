"""CPU tests of the multi-GPU host logic: shard arithmetic, byte-identity of a
column shard with packing the column slice on its own, and the gather / reduce
steps over a world-size-2 gloo process group (oracle arithmetic on each rank)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as O
from smith_b200 import parallel as P


def test_column_shard_covers_and_aligns():
    for N in (8, 64, 1000, 1024, 11008, 14336, 128256, 4096):
        for world in (1, 2, 4, 8):
            spans = [P.column_shard(N, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == N
            for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                assert a1 == b0
            assert all(s[0] % 8 == 0 for s in spans)
            widths = [b - a for a, b in spans]
            assert max(widths) - min(w for w in widths if w or N < 8 * world) <= 8 or N % 8
    # the configurations' shard widths at 8 GPUs
    assert P.column_shard(14336, 8, 3) == (5376, 7168) and P.column_shard(128256, 8, 7) == (112224, 128256)
    assert [P.group_shard(128, 8, r) for r in (0, 7)] == [(0, 16), (112, 128)]
    assert P.group_shard(10, 4, 0) == (0, 3) and P.group_shard(10, 4, 3) == (8, 10)


@pytest.mark.parametrize("kind,bb", [("q4", 24), ("q8", 34)])
def test_column_shard_of_packed_equals_packing_the_slice(kind, bb):
    rng = np.random.default_rng(0)
    K, N = 100, 48
    w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    quant = O.quantize_q4 if kind == "q4" else O.quantize_q8
    packed = quant(w)
    for world in (2, 4):
        for r in range(world):
            n0, n1 = P.column_shard(N, world, r)
            assert np.array_equal(P.slice_packed_columns(packed, O.groups_of(K), N, bb, n0, n1), quant(w[:, n0:n1]))
    g0, g1 = P.group_shard(O.groups_of(K), 2, 1)
    assert np.array_equal(P.slice_packed_groups(packed, O.groups_of(K), N, bb, g0, g1), quant(w[g0 * 32:, :]))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, M, K, N, kind, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(42)                      # same data on every rank
        w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
        a = rng.standard_normal((M, K)).astype(np.float32)
        quant = O.quantize_q4 if kind == "q4" else O.quantize_q8
        bb = 24 if kind == "q4" else 34
        full_packed = quant(w)
        want = O.matmul(a, full_packed, K, N, kind)
        # N-sharding: each rank multiplies its column shard, slices are all-gathered
        n0, n1 = P.column_shard(N, world, rank)
        shard = P.slice_packed_columns(full_packed, O.groups_of(K), N, bb, n0, n1)
        y_r = O.matmul(a, shard, K, n1 - n0, kind)
        y = P.gather_columns(torch.from_numpy(y_r), N, world, rank).numpy()
        ok_gather = np.array_equal(y.view(np.uint32), want.view(np.uint32))
        # K-sharding: each rank multiplies its group-rows, partial sums are all-reduced
        g0, g1 = P.group_shard(O.groups_of(K), world, rank)
        k0, k1 = g0 * 32, min(g1 * 32, K)
        part = O.matmul(a[:, k0:k1], P.slice_packed_groups(full_packed, O.groups_of(K), N, bb, g0, g1), k1 - k0, N, kind)
        tot = P.reduce_partials(torch.from_numpy(part.copy())).numpy()
        bound = O.tolerance_bound(a, O.dequant(full_packed, K, N, kind))
        ok_reduce = bool(np.all(np.abs(tot.astype(np.float64) - want) <= bound))
        if rank == 0:
            out_q.put((ok_gather, ok_reduce))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("kind", ["q4", "q8"])
@pytest.mark.parametrize("M,K,N", [(1, 256, 64), (3, 100, 40), (2, 128, 24)])
def test_world_size_2_gather_and_reduce(kind, M, K, N):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, M, K, N, kind, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert q.get(timeout=10) == (True, True)
