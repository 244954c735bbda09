"""Sharding of the quantized matmul across the GPUs of one box (one process per GPU).

The reference is single-device; this module is new.  Packed weights are
sharded along the output dimension N: rank r owns the columns
``column_shard(N, P, r)`` of every group-row, i.e. a buffer ``[groups][N_r][block]``
that is byte-identical to packing the f32 column slice on its own (blocks are
independent per (group, column): src/ops/quantize.js:20-59).  Activations are
replicated, each rank computes its slice ``y_r [M, N_r]`` and the slices are
all-gathered into ``y [M, N]`` where the caller needs the full row.
K-sharding (for Wo / down projections) splits the group-rows instead and ends in
an all-reduce of partial ``[M, N]`` sums.

torch.distributed provides the process group (NCCL over NVLink on GPUs, gloo on
CPU for the host-logic tests); torch is imported only here.
"""
import numpy as np


def column_shard(N, world, rank, align=8):
    """[n0, n1) of rank's output columns; every boundary is a multiple of `align`
    (keeps each shard's group-rows 16-byte aligned for both block sizes)."""
    units = -(-N // align)
    base, extra = divmod(units, world)
    u0 = rank * base + min(rank, extra)
    u1 = u0 + base + (1 if rank < extra else 0)
    return min(u0 * align, N), min(u1 * align, N)


def group_shard(groups, world, rank):
    """[g0, g1) of rank's group-rows for K-sharding."""
    base, extra = divmod(groups, world)
    g0 = rank * base + min(rank, extra)
    return g0, g0 + base + (1 if rank < extra else 0)


def slice_packed_columns(packed, groups, N, block_bytes, n0, n1):
    """Columns [n0, n1) of a packed [groups][N][block] byte array, as the shard's own packed array."""
    p = np.asarray(packed, dtype=np.uint8).reshape(groups, N, block_bytes)
    return np.ascontiguousarray(p[:, n0:n1, :]).reshape(-1)


def slice_packed_groups(packed, groups, N, block_bytes, g0, g1):
    """Group-rows [g0, g1): a contiguous byte range of the packed array."""
    p = np.asarray(packed, dtype=np.uint8).reshape(groups, N * block_bytes)
    return np.ascontiguousarray(p[g0:g1]).reshape(-1)


def gather_columns(local, N, world, rank, group=None):
    """All-gather column slices ``local [M, N_r]`` (a torch tensor, any backend) into ``[M, N]``.

    Shards may differ in width (N not divisible by 8 * world), so slices are
    padded to the widest shard for the collective and trimmed afterwards."""
    import torch
    import torch.distributed as dist
    M = local.shape[0]
    widths = [column_shard(N, world, r)[1] - column_shard(N, world, r)[0] for r in range(world)]
    wmax = max(widths)
    send = local if local.shape[1] == wmax else torch.nn.functional.pad(local, (0, wmax - local.shape[1]))
    flat = torch.empty((world * M, wmax), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(flat, send.contiguous(), group=group)
    out = flat.view(world, M, wmax)
    if all(w == wmax for w in widths):
        return out.permute(1, 0, 2).reshape(M, N) if M > 1 else out.reshape(1, N)
    return torch.cat([out[r, :, :widths[r]] for r in range(world)], dim=1)


def reduce_partials(partial, group=None):
    """All-reduce (sum, f32) of K-sharded partial outputs ``[M, N]``, in place."""
    import torch.distributed as dist
    dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
    return partial


class OutputGather:
    """Device-side all-gather of a rank's output slice on the bridge's stream.

    Owns the slice buffer ``local`` (torch memory wrapped as a bridge buffer so
    the matmul writes straight into it) and the gathered ``full`` tensor."""
    capturable = False      # NCCL through torch is not recorded into the bridge's graph capture
    kernels_per_call = 1

    def __init__(self, M, N, world, rank):
        import torch
        from . import device as D
        self.M, self.N, self.world, self.rank = M, N, world, rank
        n0, n1 = column_shard(N, world, rank)
        self.local = torch.zeros((M, n1 - n0), dtype=torch.float32, device="cuda")
        self.local_buf = D.wrapDeviceMemory(self.local.data_ptr(), self.local.numel() * 4)
        self.stream = torch.cuda.ExternalStream(D.stream())
        self.full = None

    def enqueue(self):
        import torch
        with torch.cuda.stream(self.stream):
            self.full = gather_columns(self.local, self.N, self.world, self.rank)
        return self.full


class ShardedMatmul:
    """y = a @ dequant(W) with W N-sharded over the process group: the multi-GPU
    counterpart of matmulQ4 / matmulQ8 for one weight matrix."""

    def __init__(self, kind, K, N, packed_shard_buffer, M, world, rank):
        from . import device as D
        self.kind, self.K, self.N, self.M = kind, K, N, M
        self.world, self.rank = world, rank
        self.packed = packed_shard_buffer
        n0, n1 = column_shard(N, world, rank)
        self.Nl = n1 - n0
        self.gather = OutputGather(M, N, world, rank)
        self.a_dev = D.alloc(M * K * 4, D.PRIVATE)

    def enqueue(self, a_dev=None):
        """Asynchronous: matmul on this rank's shard, then the all-gather."""
        from . import device as D
        D.qmatmul(self.kind, a_dev or self.a_dev, self.packed, self.gather.local_buf, self.M, self.Nl, self.K,
                  self.K // 32, D.PATH_AUTO)
        return self.gather.enqueue()

    def forward(self, a_host):
        """End to end from host memory: upload activations, compute, gather, download the full rows."""
        from . import device as D
        D.upload(self.a_dev, np.ascontiguousarray(a_host, dtype=np.float32))
        full = self.enqueue()
        D.synchronize()
        return full.cpu().numpy()
