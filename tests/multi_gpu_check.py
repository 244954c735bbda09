"""Multi-GPU check of the sharded path, one process per GPU (not collected by pytest):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 tests/multi_gpu_check.py

Every rank multiplies its column shard; the output row is gathered either inside the GEMV
kernel (peer stores over NVLink, M <= 4) or by NCCL (wider M).  Rank 0 compares the gathered
rows of every rank-visible result with the CPU oracle.  Ranks only ever leave between steps."""
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
    dist.destroy_process_group()
    sys.exit(1 if failures else 0)


if __name__ == "__main__":
    main()
