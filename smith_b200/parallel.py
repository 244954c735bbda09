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


class FusedGather:
    """Output row gathered by the GEMV kernel itself (M <= 4): every rank's kernel stores its
    column slice into every rank's row through peer-mapped memory and the launch completes
    when the local row is whole.  No NCCL call on the data path; capturable in a CUDA graph.

    Owns this rank's row buffer (two halves used alternately) and its 16-byte control block,
    and holds IPC mappings of the other ranks' buffers.

    ``deferred=True``: the low-latency form.  Outputs travel as 8-byte {value, step tag} stores (the
    row buffers hold such pairs), nothing is fenced, signalled or awaited at the end of a launch; the
    next ``enqueue`` polls the previous row's tags after its weights have begun to stream (the NVLink
    latency hides behind the stream), and ``finish()`` closes the chain -- call it before reading
    the last row."""
    capturable = True
    kernels_per_call = 0    # the gather is part of the matmul launch

    def __init__(self, M, N, world, rank, group=None, deferred=False):
        from . import device as D
        self.M, self.N, self.world, self.rank = M, N, world, rank
        self.deferred = deferred
        self._last = None
        self.spans = [column_shard(N, world, r) for r in range(world)]
        self.elem = 8 if deferred else 4
        self.y = D.alloc(2 * M * N * self.elem, D.PRIVATE)
        self.state = D.alloc(256, D.PRIVATE)
        D.upload(self.state, np.zeros(64, np.uint32))
        D.upload(self.y, np.zeros(2 * M * N * self.elem // 4, np.uint32))
        self.ys, self.states = [None] * world, [None] * world
        self.ys[rank], self.states[rank] = self.y, self.state
        if world > 1:
            import torch.distributed as dist
            mine = (D.ipcExport(self.y), D.ipcExport(self.state))
            handles = [None] * world
            dist.all_gather_object(handles, mine, group=group)
            for r in range(world):
                if r != rank:
                    self.ys[r] = D.ipcImport(handles[r][0], 2 * M * N * self.elem)
                    self.states[r] = D.ipcImport(handles[r][1], 256)
            dist.barrier(group=group)     # everyone has mapped everyone before the first store
        self.calls = 0
        self._targets = {}

    def target(self, kind, K):
        from . import device as D
        key = (kind, K)
        if key not in self._targets:
            tiles = [D.qgemvTiles(kind, self.M, b - a, K) for a, b in self.spans]
            if min(tiles) < 0:
                raise D.SmithError("smith: the GEMV kernel does not take this shard shape")
            self._targets[key] = sum(tiles)
        return self._targets[key]

    def enqueue(self, kind, a_buf, packed_shard_buf, K, from_previous=False):
        """Asynchronous fused matmul + all-gather; returns which half of the row buffer it fills, counted
        on the host (valid while no captured graph replays calls on this state: see ``last_half``).
        ``from_previous`` (deferred form, K == N): the activations are the row the previous call gathered."""
        from . import device as D
        n0, n1 = self.spans[self.rank]
        D.qmatmulAllGather(kind, a_buf, packed_shard_buf, self.M, self.N, n0, n1 - n0, K, K // 32, self.world,
                           self.rank, self.ys, self.states, self.target(kind, K),
                           (D.GATHER_DEFER | (D.GATHER_INPUT_IS_PREVIOUS_ROW if from_previous else 0))
                           if self.deferred else 0)
        self._last = (kind, K)
        half = self.calls & 1
        self.calls += 1
        return half

    def finish(self):
        """Deferred mode: enqueue the wait that makes the last step's row whole on this rank."""
        from . import device as D
        if self.deferred and self._last:
            D.allGatherWait(self.state, self.y, self.M, self.N)

    def last_half(self):
        """Which half of the row buffer the last finished call filled.  Taken from the step number the
        kernels keep in device memory: a host-side count of ``enqueue`` calls falls behind once calls
        are replayed from a captured graph.  Synchronises."""
        from . import device as D
        D.synchronize()
        step = int(D.download(self.state, 4, np.uint32)[0])
        return (step - 1) & 1

    def read(self, half=None):
        """The gathered rows [M, N] of one half (default: the half the last finished call filled), after
        ``finish()`` in deferred mode and a synchronize."""
        from . import device as D
        if half is None:
            half = self.last_half()
        n = self.M * self.N
        if self.deferred:                 # {value, tag} pairs
            pairs = D.download(self.y, n * 8, np.float32, offset=half * n * 8).reshape(n, 2)
            return np.ascontiguousarray(pairs[:, 0]).reshape(self.M, self.N)
        return D.download(self.y, n * 4, np.float32, offset=half * n * 4).reshape(self.M, self.N)

    def close(self):
        from . import device as D
        for r in range(self.world):
            if r != self.rank and self.ys[r]:
                D.releaseBuffer(self.ys[r])
                D.releaseBuffer(self.states[r])
        D.releaseBuffer(self.y)
        D.releaseBuffer(self.state)
        self.ys = self.states = []


class ShardedList:
    """R products y_i = a @ dequant(W_i), every W_i sharded along N over the ranks, as ONE persistent
    launch per rank (smith_qmatmul_list_create_gather): each rank walks its R column shards with its
    ring of weight stages never draining, and every item's epilogue stores its columns, as
    {value, launch tag} pairs, straight into every rank's gathered row over peer memory.  No NCCL call
    and no per-matrix hand-off between the GPUs: the ranks only meet at the end of a launch, when each
    waits (bounded) until its own rows are whole.

    Owns one device buffer with this rank's R row buffers (2 x M x N pairs each, the halves alternate
    with the launch number), exported to the other ranks through IPC, and the R local slices."""

    def __init__(self, kind, M, K, N, packed_shards, world, rank, a_buf, group=None, closing_wait=True):
        from . import device as D
        self.kind, self.M, self.K, self.N, self.world, self.rank = kind, M, K, N, world, rank
        self.R = len(packed_shards)
        self.n0, n1 = column_shard(N, world, rank)
        self.Nl = n1 - self.n0
        self.row_bytes = 2 * M * N * 8
        self.rows = D.alloc(self.R * self.row_bytes, D.PRIVATE)
        D.upload(self.rows, np.zeros(self.R * self.row_bytes // 4, np.uint32))
        self.local = [D.alloc(M * self.Nl * 4, D.PRIVATE) for _ in range(self.R)]
        self.all_rows = [None] * world
        self.all_rows[rank] = self.rows
        if world > 1:
            import torch.distributed as dist
            handles = [None] * world
            dist.all_gather_object(handles, D.ipcExport(self.rows), group=group)
            for r in range(world):
                if r != rank:
                    self.all_rows[r] = D.ipcImport(handles[r], self.R * self.row_bytes)
        # one view per (rank, item) of the ranks' row buffers
        self.views = [[D.wrapDeviceMemory(D.devicePtr(self.all_rows[r]) + i * self.row_bytes, self.row_bytes)
                       for r in range(world)] for i in range(self.R)]
        items = [D.listItem(a_buf, pk, c, self.Nl, K) for pk, c in zip(packed_shards, self.local)]
        gathers = [D.listGather(world, self.n0, N, self.views[i]) for i in range(self.R)]
        self.handle = D.qmatmulListCreateGather(kind, M, items, gathers, rank,
                                                0 if closing_wait else D.LIST_NO_CLOSING_WAIT)
        if world > 1:
            import torch.distributed as dist
            dist.barrier(group=group)     # everyone has mapped everyone before the first store

    def run(self):
        """Asynchronous: all R products on this rank's shards, gathered into every rank's rows."""
        from . import device as D
        D.qmatmulListRun(self.handle)

    def read(self, i):
        """Gathered row [M, N] of product i as the last finished launch left it (synchronises)."""
        from . import device as D
        half = (D.qmatmulListNextTag(self.handle) - 1) & 1
        n = self.M * self.N
        pairs = D.download(self.rows, n * 8, np.uint32, offset=i * self.row_bytes + half * n * 8).reshape(n, 2)
        return np.ascontiguousarray(pairs[:, 0]).view(np.float32).reshape(self.M, self.N), pairs[:, 1]

    def close(self):
        from . import device as D
        D.qmatmulListDestroy(self.handle)
        for vs in self.views:
            for v in vs:
                D.releaseBuffer(v)
        for r in range(self.world):
            if r != self.rank and self.all_rows[r]:
                D.releaseBuffer(self.all_rows[r])
        for b in self.local + [self.rows]:
            D.releaseBuffer(b)
        self.views, self.all_rows, self.local = [], [], []


class FusedReduce:
    """Sum over ranks of K-sharded partial products, formed by the GEMV kernel itself (M <= 4): every
    rank's kernel pushes its partial sums as {value, step tag} pairs into its slot on every rank
    (8-byte stores through peer-mapped memory, no fences), polls all ranks' slots in its own memory
    and adds them in rank order.  No NCCL call on the data path; capturable in a CUDA graph; every
    rank ends with the same bits.

    Owns this rank's slot array (2 x world x M x N pairs) and its state block, and holds IPC mappings
    of the other ranks'."""
    capturable = True
    kernels_per_call = 0    # the reduction is part of the matmul launch

    def __init__(self, kind, M, N, k_local, world, rank, group=None):
        from . import device as D
        self.kind, self.M, self.N, self.k_local, self.world, self.rank = kind, M, N, k_local, world, rank
        sbytes = D.qmatmulAllReduceStateBytes(kind, M, N, k_local)
        if sbytes == 0:
            raise D.SmithError("smith: the GEMV kernel does not take this shard shape")
        self.pbytes = 2 * world * M * N * 8
        self.partial = D.alloc(self.pbytes, D.PRIVATE)
        self.state = D.alloc(max(sbytes, 256), D.PRIVATE)
        D.upload(self.state, np.zeros(max(sbytes, 256) // 4, np.uint32))
        D.upload(self.partial, np.zeros(self.pbytes // 4, np.uint32))
        self.partials, self.states = [None] * world, [None] * world
        self.partials[rank], self.states[rank] = self.partial, self.state
        if world > 1:
            import torch.distributed as dist
            mine = (D.ipcExport(self.partial), D.ipcExport(self.state))
            handles = [None] * world
            dist.all_gather_object(handles, mine, group=group)
            for r in range(world):
                if r != rank:
                    self.partials[r] = D.ipcImport(handles[r][0], self.pbytes)
                    self.states[r] = D.ipcImport(handles[r][1], max(sbytes, 256))
            dist.barrier(group=group)     # everyone has mapped everyone before the first flag is written

    def enqueue(self, a_buf, packed_shard_buf, out_buf):
        from . import device as D
        D.qmatmulAllReduce(self.kind, a_buf, packed_shard_buf, out_buf, self.M, self.N, self.k_local,
                           self.k_local // 32, self.world, self.rank, self.partials, self.states)

    def close(self):
        from . import device as D
        for r in range(self.world):
            if r != self.rank and self.partials[r]:
                D.releaseBuffer(self.partials[r])
                D.releaseBuffer(self.states[r])
        D.releaseBuffer(self.partial)
        D.releaseBuffer(self.state)
        self.partials = self.states = []


class KShardedMatmul:
    """y = a @ dequant(W) with W sharded along K over the process group (the Wo / down projections
    of a tensor-parallel layer): rank r holds group-rows ``group_shard(K / 32, P, r)`` of all N
    columns and multiplies the matching K-slice of the activations; the partial [M, N] products are
    summed over ranks -- inside the GEMV kernel for M <= 4, by an NCCL all-reduce otherwise.
    The summation order differs from the single-device sequential one, so results agree with it to
    the stated tolerance, not bitwise."""

    def __init__(self, kind, K, N, packed_shard_buffer, M, world, rank):
        import torch
        from . import device as D
        self.kind, self.K, self.N, self.M, self.world, self.rank = kind, K, N, M, world, rank
        g0, g1 = group_shard(K // 32, world, rank)
        self.k0, self.k1 = g0 * 32, g1 * 32
        self.kl = self.k1 - self.k0
        self.packed = packed_shard_buffer
        shapes = [(b - a) * 32 for a, b in (group_shard(K // 32, world, r) for r in range(world))]
        # the fused form needs the same tiling of N on every rank: equal K-slices and a GEMV-shaped M
        self.fused = M <= 4 and len(set(shapes)) == 1 and D.qgemvTiles(kind, M, N, self.kl) > 0
        self.a_dev = D.alloc(M * self.kl * 4, D.PRIVATE)
        if self.fused:
            self.reduce = FusedReduce(kind, M, N, self.kl, world, rank)
            self.out = D.alloc(M * N * 4, D.PRIVATE)
        else:
            self.reduce = None
            self.out_t = torch.zeros((M, N), dtype=torch.float32, device="cuda")
            self.out = D.wrapDeviceMemory(self.out_t.data_ptr(), M * N * 4)
            self.stream = torch.cuda.ExternalStream(D.stream())

    def enqueue(self, a_dev=None):
        """Asynchronous: this rank's partial product and the sum over ranks into ``self.out``."""
        import torch
        from . import device as D
        if self.fused:
            self.reduce.enqueue(a_dev or self.a_dev, self.packed, self.out)
            return
        D.qmatmul(self.kind, a_dev or self.a_dev, self.packed, self.out, self.M, self.N, self.kl, self.kl // 32,
                  D.PATH_AUTO)
        with torch.cuda.stream(self.stream):
            reduce_partials(self.out_t)

    def forward(self, a_host):
        """End to end from host memory: ``a_host`` is the full [M, K] activation matrix; this rank
        uploads its K-slice, computes, reduces, and downloads the full [M, N] result."""
        from . import device as D
        a = np.ascontiguousarray(np.asarray(a_host, dtype=np.float32)[:, self.k0:self.k1])
        D.upload(self.a_dev, a)
        self.enqueue()
        D.synchronize()
        return D.download(self.out, self.M * self.N * 4, np.float32).reshape(self.M, self.N)


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
        self.fused = M <= 4 and all(D.qgemvTiles(kind, M, b - a, K) > 0
                                    for a, b in (column_shard(N, world, r) for r in range(world)))
        self.gather = FusedGather(M, N, world, rank, deferred=True) if self.fused else OutputGather(M, N, world, rank)
        self.a_dev = D.alloc(M * K * 4, D.PRIVATE)

    def enqueue(self, a_dev=None):
        """Asynchronous: matmul on this rank's shard and the all-gather (fused into the kernel for
        M <= 4, NCCL otherwise).  Returns the half index (fused) or the gathered torch tensor."""
        from . import device as D
        if self.fused:
            return self.gather.enqueue(self.kind, a_dev or self.a_dev, self.packed, self.K)
        D.qmatmul(self.kind, a_dev or self.a_dev, self.packed, self.gather.local_buf, self.M, self.Nl, self.K,
                  self.K // 32, D.PATH_AUTO)
        return self.gather.enqueue()

    def forward(self, a_host):
        """End to end from host memory: upload activations, compute, gather, download the full rows."""
        from . import device as D
        D.upload(self.a_dev, np.ascontiguousarray(a_host, dtype=np.float32))
        out = self.enqueue()
        if self.fused:
            self.gather.finish()
        D.synchronize()
        if self.fused:
            return self.gather.read(out)
        return out.cpu().numpy()
