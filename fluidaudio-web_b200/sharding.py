"""Multi-GPU host logic: the path shards by independent units (audio windows, decode streams), so each
rank (one process per GPU) takes a contiguous block of units, runs them with no data-path collective,
and rank 0 concatenates the per-rank results on the host in unit order.  The reference already treats
windows as independent (src/engines/asr-parakeet/raw-encoder.js:230-242, pipeline.js:35-41)."""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np


def shard_range(n_units: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous block [lo, hi) of `n_units` for `rank`; the first n_units % world ranks get one extra."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(n_units, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard(units: Sequence, world: int, rank: int) -> list:
    lo, hi = shard_range(len(units), world, rank)
    return list(units[lo:hi])


def gather_rows(local: np.ndarray, world: int, rank: int, group=None) -> Optional[np.ndarray]:
    """Host gather of per-rank row blocks to rank 0 in rank (= unit) order.  Ranks may hold different row
    counts (ragged shards, empty included).  Returns the concatenation on rank 0, None elsewhere."""
    local = np.ascontiguousarray(local, dtype=np.float32)
    if world == 1:
        return local
    import torch
    import torch.distributed as dist

    parts: List[Optional[np.ndarray]] = [None] * world if rank == 0 else None
    dist.gather_object(local, parts, dst=0, group=group)
    if rank != 0:
        return None
    cols = next((p.shape[1] for p in parts if p.size), local.shape[1] if local.ndim == 2 else 0)
    return np.concatenate([p.reshape(-1, cols) for p in parts], axis=0)


def column_shard(w: np.ndarray, world: int, rank: int) -> np.ndarray:
    """This rank's block of output columns of a [K, N] weight matrix (N divisible by world)."""
    N = w.shape[1]
    if N % world:
        raise ValueError(f"N={N} does not split evenly over {world} ranks")
    ns = N // world
    return np.ascontiguousarray(w[:, rank * ns:(rank + 1) * ns])


def unshard_cols_host(gathered: np.ndarray, world: int) -> np.ndarray:
    """Host statement of the device unshardCols: [world*M, Ns] -> [M, world*Ns]."""
    M = gathered.shape[0] // world
    return np.ascontiguousarray(gathered.reshape(world, M, -1).transpose(1, 0, 2).reshape(M, -1))


class _DeviceArray:
    """A device buffer of the context seen through __cuda_array_interface__, so torch.distributed can
    send and receive it in place (no staging copy)."""

    def __init__(self, ptr: int, shape):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<f4", "data": (int(ptr), False), "version": 2}


def as_torch(ctx, t):
    import torch

    return torch.as_tensor(_DeviceArray(ctx.devicePtr(t), (t.rows, t.cols)), device=f"cuda:{ctx.device}")


def matmul_n_sharded(ctx, a, w_shard, opts=None, group=None):
    """The one exchange step of the path: every rank multiplies the same activations [M, K] by its block of
    output columns [K, N/world] on its own GPU, then an NCCL all-gather over NVLink brings all blocks to
    every rank and unshardCols lays them out as the row-major [M, N] product.  The collective runs on the
    context's stream (ordered after the product, before the unshard)."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    c_local = ctx.matmul(a, w_shard, opts)
    if world == 1:
        return c_local
    gathered = ctx.alloc(world * c_local.rows, c_local.cols)
    stream = torch.cuda.ExternalStream(ctx.stream(), device=ctx.device)
    with torch.cuda.stream(stream):
        dist.all_gather_into_tensor(as_torch(ctx, gathered), as_torch(ctx, c_local), group=group)
    out = ctx.unshardCols(gathered, world)
    ctx.freeTensor(gathered)
    ctx.freeTensor(c_local)
    return out


def matmul_n_sharded_many(ctx, pairs, group=None):
    """Several N-sharded products back to back, pipelined: the all-gather of product i runs on a side
    stream while product i+1 is computed; the unshard of each result waits only for its own gather.
    `pairs` = [(a, w_shard), ...]; returns the row-major [M, N] products in order."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    if world == 1:
        return [ctx.matmul(a, w) for a, w in pairs]
    ext = torch.cuda.ExternalStream(ctx.stream(), device=ctx.device)
    comm = getattr(ctx, "_comm_stream", None)
    if comm is None:
        comm = ctx._comm_stream = torch.cuda.Stream(device=ctx.device)
    pending = []
    for a, w in pairs:
        c = ctx.matmul(a, w)
        g = ctx.alloc(world * c.rows, c.cols)
        ready = torch.cuda.Event()
        ready.record(ext)
        comm.wait_event(ready)
        with torch.cuda.stream(comm):
            dist.all_gather_into_tensor(as_torch(ctx, g), as_torch(ctx, c), group=group)
            done = torch.cuda.Event()
            done.record(comm)
        pending.append((c, g, done))
    outs = []
    for c, g, done in pending:
        ext.wait_event(done)
        outs.append(ctx.unshardCols(g, world))
        ctx.freeTensor(g)
        ctx.freeTensor(c)
    return outs


class ScatterResult:
    """A full [M, N] f32 result buffer on every rank, each mapped into every other rank (CUDA IPC), for
    products whose epilogue stores its tiles straight into all of them (matmul_n_sharded_scatter)."""

    def __init__(self, ctx, M: int, N: int, group=None):
        import torch.distributed as dist

        self.ctx, self.M, self.N, self.group = ctx, M, N, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.local = ctx.pin(ctx.alloc(M, N))
        handles = [None] * self.world
        dist.all_gather_object(handles, ctx.ipcExport(self.local), group=group)
        own = ctx.devicePtr(self.local)
        self._peers = {r: ctx.ipcOpen(h) for r, h in enumerate(handles) if r != self.rank}
        self.ptrs = [own] + [self._peers[r] for r in sorted(self._peers)]  # own buffer first

    def close(self):
        import torch.distributed as dist

        self.ctx.sync()
        dist.barrier(group=self.group)  # nobody unmaps while a peer may still be writing
        for p in self._peers.values():
            self.ctx.ipcClose(p)
        self._peers = {}
        dist.barrier(group=self.group)
        self.ctx.freeTensor(self.local)


def stream_barrier(ctx, group=None):
    """Orders the ranks on the context's stream: work enqueued after it starts only when every rank's work
    enqueued before it has finished (a one-element NCCL all-reduce on that stream)."""
    import torch
    import torch.distributed as dist

    flag = getattr(ctx, "_barrier_flag", None)
    if flag is None:
        flag = ctx._barrier_flag = torch.zeros(1, device=f"cuda:{ctx.device}")
    with torch.cuda.stream(torch.cuda.ExternalStream(ctx.stream(), device=ctx.device)):
        dist.all_reduce(flag, group=group)


def matmul_n_sharded_scatter(ctx, a, w_shard, res: ScatterResult, opts=None):
    """N-sharded product with the all-gather inside the GEMM: the epilogue of this rank's column block stores
    each finished tile into every rank's result buffer over NVLink (plain peer stores).  Call stream_barrier
    afterwards, before any rank reads `res.local`, and again before the next product reuses `res`."""
    o = opts or {}
    ns = w_shard.cols
    ctx.matmulScatter(a, w_shard, res.ptrs, res.N, res.rank * ns, bias=o.get("bias"), act=o.get("act", "none"))
    return res.local


def encode_windows_sharded(ctx, enc, mels: Sequence[np.ndarray], world: int, rank: int, batch: int = 32, group=None):
    """Encode this rank's block of windows in batches of `batch` and gather the frames on rank 0.
    Returns ([n_windows * Tsub, D] on rank 0 else None, Tsub)."""
    from .engines import fastconformer

    mine = shard(mels, world, rank)
    outs, Tsub, D = [], 0, enc["cfg"]["D"]
    for i in range(0, len(mine), batch):
        h = ctx.pushArena()
        x, Tsub = fastconformer.encode_batch(ctx, enc, mine[i:i + batch])
        outs.append(np.asarray(ctx.download(x), np.float32).reshape(-1, D))
        ctx.popArena(h)
    local = np.concatenate(outs, axis=0) if outs else np.zeros((0, D), np.float32)
    return gather_rows(local, world, rank, group), Tsub
