"""Seeded synthetic Connect6 positions, keyed by GLOBAL board index.

Stand-in for live self-play positions (no dataset is involved): per board a stone count
n ~ U{0..max_stones}, n distinct cells chosen uniformly, split into own/opponent stones with
|own - opp| <= 2, and a constant third plane that is all 0 or all 1 with probability 1/2.
Every random number is a hash of (seed, board index, lane), so a board's content does not
depend on batch size, sharding or GPU count.  Output format is the reference's network input
(connect6/vector_env.py:196-218): float32 [B, 3, n, n].
"""
from __future__ import annotations

import numpy as np

DEFAULT_SEED = 0xC6


def _mix64(x: np.ndarray) -> np.ndarray:
    """splitmix64 finaliser on uint64 arrays."""
    with np.errstate(over="ignore"):
        x = (x + np.uint64(0x9E3779B97F4A7C15)).astype(np.uint64)
        x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return x ^ (x >> np.uint64(31))


def _stream(seed: int, index: np.ndarray, lane: np.ndarray | int) -> np.ndarray:
    with np.errstate(over="ignore"):
        base = _mix64(np.uint64(seed) ^ _mix64(index.astype(np.uint64)))
        return _mix64(base + np.uint64(0xD1B54A32D192ED03) * np.asarray(lane, dtype=np.uint64))


def generate_planes(first_index: int, count: int, board_size: int = 19, max_stones: int = 120,
                    seed: int = DEFAULT_SEED) -> np.ndarray:
    """Boards [first_index, first_index + count) as float32 [count, 3, n, n]."""
    n = int(board_size)
    cells = n * n
    idx = np.arange(first_index, first_index + count, dtype=np.uint64)
    stones = (_stream(seed, idx, 0) % np.uint64(min(max_stones, cells) + 1)).astype(np.int64)
    # own - opponent in {-2, 0, 2} for an even stone count, {-1, 1} for an odd one
    h = _stream(seed, idx, 1)
    delta = np.where(stones % 2 == 0, 2 * (h % np.uint64(3)).astype(np.int64) - 2,
                     2 * (h % np.uint64(2)).astype(np.int64) - 1)
    mine = np.clip((stones + delta) // 2, 0, stones)
    last = (_stream(seed, idx, 2) & np.uint64(1)).astype(np.float32)
    # a uniformly random permutation of the cells per board: rank of per-cell hashes
    keys = _stream(seed, idx[:, None], np.arange(3, 3 + cells, dtype=np.uint64)[None, :])
    rank = np.argsort(np.argsort(keys, axis=1, kind="stable"), axis=1, kind="stable")
    planes = np.zeros((count, 3, cells), dtype=np.float32)
    planes[:, 0] = rank < mine[:, None]
    planes[:, 1] = (rank >= mine[:, None]) & (rank < stones[:, None])
    planes[:, 2] = last[:, None]
    return planes.reshape(count, 3, n, n)


def shard_range(total: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous, balanced range [lo, hi) of global board indices owned by `rank`."""
    lo = total * rank // world
    hi = total * (rank + 1) // world
    return lo, hi
