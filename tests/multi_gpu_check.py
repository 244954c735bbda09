"""Multi-GPU check of the sharded path, one process per GPU (not collected by pytest):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 tests/multi_gpu_check.py

Every rank multiplies its column shard; the output row is gathered either inside the GEMV
kernel (peer stores over NVLink, M <= 4) or by NCCL (wider M).  Then the same for weights
sharded along K, where the partial products are summed inside the GEMV kernel (peer loads,
M <= 4) or by an NCCL all-reduce.  Every rank compares its result with the CPU oracle.
Ranks only ever leave between steps."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    torch.cuda.set_device(local)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from helpers import within_tolerance
    from oracle import oracle as O
    from smith_b200 import device as D
    from smith_b200 import parallel as P
    D.ctx()
    failures = 0
    for kind, M, K, N in [(4, 1, 4096, 14336), (8, 2, 1024, 2048), (4, 4, 2048, 1000 // 8 * 8 * 4), (4, 8, 1024, 1024),
                          (8, 64, 1024, 1024)]:
        knd, bb = ("q4", 24) if kind == 4 else ("q8", 34)
        rng = np.random.default_rng(1234 + M + N)           # identical data on every rank
        w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
        packed = O.quantize_q4(w) if kind == 4 else O.quantize_q8(w)
        n0, n1 = P.column_shard(N, world, rank)
        shard = D.alloc((K // 32) * (n1 - n0) * bb, D.PRIVATE)
        D.upload(shard, P.slice_packed_columns(packed, K // 32, N, bb, n0, n1))
        sm = P.ShardedMatmul(kind, K, N, shard, M, world, rank)
        worst_all = 0.0
        for step in range(3):                                 # repeated calls exercise both halves / counters
            a = rng.standard_normal((M, K)).astype(np.float32)
            got = sm.forward(a)
            assert D.kernelStatus() == 0, "a bounded device-side wait gave up"
            want = O.matmul(a, packed, K, N, knd, threads=O.max_threads())
            ok, worst = within_tolerance(got, want, a, packed, K, N, knd, 1e-3)
            worst_all = max(worst_all, worst)
            if not ok:
                failures += 1
        flag = torch.tensor([failures], device="cuda")
        dist.all_reduce(flag)
        if rank == 0:
            print(f"world={world} kind={knd} M={M} K={K} N={N} fused={sm.fused}: worst err/bound {worst_all:.3f} "
                  f"failures(all ranks)={int(flag.item())}", flush=True)
        dist.barrier()
    # ---- the list form: R column-sharded products per launch, every item's epilogue gathering its row
    for kind, M, K, N, R in [(4, 1, 4096, 14336, 6), (8, 2, 1024, 2048, 4), (4, 4, 2048, 4096, 3)]:
        knd, bb = ("q4", 24) if kind == 4 else ("q8", 34)
        rng = np.random.default_rng(4321 + M + N)
        a = rng.standard_normal((M, K)).astype(np.float32)
        a_dev = D.alloc(M * K * 4, D.PRIVATE)
        D.upload(a_dev, a)
        packed, shards = [], []
        n0, n1 = P.column_shard(N, world, rank)
        for _ in range(R):
            w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
            pk = O.quantize_q4(w) if kind == 4 else O.quantize_q8(w)
            packed.append(pk)
            sh = D.alloc((K // 32) * (n1 - n0) * bb, D.PRIVATE)
            D.upload(sh, P.slice_packed_columns(pk, K // 32, N, bb, n0, n1))
            shards.append(sh)
        sl = P.ShardedList(kind, M, K, N, shards, world, rank, a_dev)
        worst_all = 0.0
        for launch in (1, 2, 3):                              # both halves of the row buffers, tags 1, 2, 3
            sl.run()
            D.synchronize()
            assert D.kernelStatus() == 0, "a bounded device-side wait gave up"
            dist.barrier()                                    # nobody starts the next launch while a row is read
            for i in range(R):
                row, tags = sl.read(i)
                if not np.all(tags == launch):
                    failures += 1
                want = O.matmul(a, packed[i], K, N, knd, threads=O.max_threads())
                ok, worst = within_tolerance(row, want, a, packed[i], K, N, knd, 1e-3)
                worst_all = max(worst_all, worst)
                if not ok:
                    failures += 1
            dist.barrier()
        flag = torch.tensor([failures], device="cuda")
        dist.all_reduce(flag)
        if rank == 0:
            print(f"world={world} list kind={knd} M={M} K={K} N={N} R={R}: worst err/bound {worst_all:.3f} "
                  f"failures(all ranks)={int(flag.item())}", flush=True)
        sl.close()
        for b in shards + [a_dev]:
            D.releaseBuffer(b)
        dist.barrier()
    # ---- a real chain: each launch reads the row the launch before it gathered (no host round trip)
    K = N = 4096
    steps = 24
    rng = np.random.default_rng(99)
    ws = [(rng.standard_normal((K, N)) * 0.02).astype(np.float32) for _ in range(2)]
    packs = [O.quantize_q4(w) for w in ws]
    n0, n1 = P.column_shard(N, world, rank)
    shards = []
    for pk in packs:
        sh = D.alloc((K // 32) * (n1 - n0) * 24, D.PRIVATE)
        D.upload(sh, P.slice_packed_columns(pk, K // 32, N, 24, n0, n1))
        shards.append(sh)
    fg = P.FusedGather(1, N, world, rank, deferred=True)
    x0 = rng.standard_normal((1, K)).astype(np.float32)
    x_dev = D.alloc(K * 4, D.PRIVATE)
    D.upload(x_dev, x0)
    for i in range(steps):                                   # enqueued back to back
        fg.enqueue(4, x_dev, shards[i & 1], K, from_previous=i > 0)
    fg.finish()
    D.synchronize()
    assert D.kernelStatus() == 0, "a bounded device-side wait gave up"
    got = fg.read((steps - 1) & 1)
    want = x0
    for i in range(steps):
        want = O.matmul(want, packs[i & 1], K, N, "q4", threads=O.max_threads())
    err = float(np.abs(got - want).max() / (np.abs(want).max() + 1e-30))
    bad = int(not (err < 5e-3))
    failures += bad
    flag = torch.tensor([failures], device="cuda")
    dist.all_reduce(flag)
    if rank == 0:
        print(f"world={world} chained gathers ({steps} launches, each reading its predecessor's gathered row): "
              f"max err / max |y| = {err:.2e} failures(all ranks)={int(flag.item())}", flush=True)
    dist.barrier()
    # ---- weights sharded along K, partial products summed over ranks
    for kind, M, K, N in [(4, 1, 4096, 4096), (8, 2, 2048, 1024), (4, 4, 14336, 4096), (4, 16, 2048, 1024)]:
        knd, bb = ("q4", 24) if kind == 4 else ("q8", 34)
        rng = np.random.default_rng(4321 + M + N)
        w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
        packed = O.quantize_q4(w) if kind == 4 else O.quantize_q8(w)
        g0, g1 = P.group_shard(K // 32, world, rank)
        shard = D.alloc((g1 - g0) * N * bb, D.PRIVATE)
        D.upload(shard, P.slice_packed_groups(packed, K // 32, N, bb, g0, g1))
        km = P.KShardedMatmul(kind, K, N, shard, M, world, rank)
        worst_all, same = 0.0, 1
        for step in range(3):
            a = rng.standard_normal((M, K)).astype(np.float32)
            got = km.forward(a)
            assert D.kernelStatus() == 0, "a bounded device-side wait gave up"
            want = O.matmul(a, packed, K, N, knd, threads=O.max_threads())
            ok, worst = within_tolerance(got, want, a, packed, K, N, knd, 1e-3)
            worst_all = max(worst_all, worst)
            if not ok:
                failures += 1
            if km.fused:                                      # rank-ordered sums: the same bits everywhere
                mine = torch.from_numpy(got.view(np.int32).astype(np.int64)).cuda()
                lo, hi = mine.clone(), mine.clone()
                dist.all_reduce(lo, op=dist.ReduceOp.MIN)
                dist.all_reduce(hi, op=dist.ReduceOp.MAX)
                same &= int(torch.equal(lo, hi))
        if not same:
            failures += 1
        flag = torch.tensor([failures], device="cuda")
        dist.all_reduce(flag)
        if rank == 0:
            print(f"world={world} K-sharded kind={knd} M={M} K={K} N={N} fused={km.fused}: worst err/bound "
                  f"{worst_all:.3f} identical on all ranks={bool(same)} failures(all ranks)={int(flag.item())}",
                  flush=True)
        dist.barrier()
    dist.destroy_process_group()
    sys.exit(1 if failures else 0)


if __name__ == "__main__":
    main()
