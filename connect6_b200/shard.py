"""Multi-GPU plumbing: one process per GPU, boards sharded by global index, no collective on
the forward path.  The only exchange is the sum of the small integer statistics vector the
self-play collector forms once per step (connect6/train.py:888-911: segment lengths, wins per
colour, draws, game lengths, historical games/wins/losses/draws) -- 9 x int64 = 72 bytes,
all-reduced over NCCL (NVLink) on GPUs or gloo on CPU.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from .boards import shard_range  # re-exported: the partitioning rule

ROLLOUT_STATS_FIELDS = (
    "segment_lengths", "black_wins", "white_wins", "draws", "game_lengths",
    "historical_games", "historical_wins", "historical_losses", "historical_draws",
)


def init_from_env(backend: str | None = None) -> tuple[int, int, int]:
    """(rank, world, local_rank) from torchrun's environment; initialises the default process
    group when WORLD_SIZE > 1."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29531")
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(local_rank)
        dist.init_process_group(backend=backend, rank=rank, world_size=world)
    return rank, world, local_rank


def reduce_rollout_stats(stats: torch.Tensor) -> torch.Tensor:
    """Sum an int64 statistics vector over all ranks in place (no-op for one process)."""
    if stats.dtype != torch.int64:
        raise TypeError("rollout statistics must be int64")
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.SUM)
    return stats


class RolloutStatsReducer:
    """Per-step sum of the statistics vector over all ranks WITHOUT putting the collective on the compute
    stream's critical path: `submit()` fills one buffer of a small ring and starts its all-reduce
    asynchronously (NCCL runs it on its own stream, ordered after the work that produced the buffer), the
    compute stream carries on; `drain()` waits for everything outstanding and returns the last reduced
    vector.  A buffer is waited for before it is reused, so at most `depth` reductions are in flight.
    With one process it degenerates to plain copies."""

    def __init__(self, device: torch.device | str, fields: int = len(ROLLOUT_STATS_FIELDS), depth: int = 4) -> None:
        self._bufs = [torch.zeros(fields, dtype=torch.int64, device=device) for _ in range(depth)]
        self._work: list = [None] * depth
        self._next = 0
        self._last = 0
        self._multi = dist.is_initialized() and dist.get_world_size() > 1

    def buffer(self) -> torch.Tensor:
        """The buffer the next submit() will reduce (write this step's statistics into it first)."""
        k = self._next
        if self._work[k] is not None:
            self._work[k].wait()
            self._work[k] = None
        return self._bufs[k]

    def submit(self) -> None:
        k = self._next
        if self._multi:
            self._work[k] = dist.all_reduce(self._bufs[k], op=dist.ReduceOp.SUM, async_op=True)
        self._last = k
        self._next = (k + 1) % len(self._bufs)

    def drain(self) -> torch.Tensor:
        for k, w in enumerate(self._work):
            if w is not None:
                w.wait()
                self._work[k] = None
        return self._bufs[self._last]


def max_over_ranks(value: float, device: torch.device | str = "cpu") -> float:
    """Maximum of a scalar over ranks (timing: the slowest rank defines the step)."""
    if not (dist.is_initialized() and dist.get_world_size() > 1):
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier() -> None:
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


__all__ = ["ROLLOUT_STATS_FIELDS", "RolloutStatsReducer", "init_from_env", "reduce_rollout_stats", "max_over_ranks",
           "barrier", "shard_range"]
