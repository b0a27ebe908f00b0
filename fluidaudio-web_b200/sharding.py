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
