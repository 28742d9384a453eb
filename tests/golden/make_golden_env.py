"""Generate the environment fixtures (env_*.npz) in this directory from the UNMODIFIED reference.

Run where the reference checkout is importable:
    python tests/golden/make_golden_env.py [/path/to/reference]
It imports `connect6.vector_env.VectorConnect6` from that path (default: $C6_REFERENCE or
/root/reference), plays seeded games with it on CPU and stores the actions, every step's outputs
and state snapshots.  The tests only read the .npz files; they never need the reference.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REF = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("C6_REFERENCE", "/root/reference"))
sys.path.insert(0, str(REF))

from connect6.vector_env import VectorConnect6  # noqa: E402


def pick_actions(rng: np.random.Generator, env: VectorConnect6, mode: str) -> np.ndarray:
    """uniform: any empty cell.  cluster: mostly a free neighbour of one of the mover's own stones
    (lines form, games end by a win).  sloppy: any cell at all, occupied ones included."""
    E, n = env.num_envs, env.board_size
    boards = env.boards.numpy()
    out = np.zeros(E, np.int64)
    for e in range(E):
        b = boards[e]
        empty = np.flatnonzero(b.reshape(-1) == 0)
        if mode == "sloppy" or empty.size == 0:
            out[e] = rng.integers(0, n * n)
            continue
        choice = int(rng.choice(empty))
        if mode == "cluster" and rng.random() < 0.75:
            own = np.argwhere(b == int(env.current_player[e]))
            if len(own):
                r, c = own[rng.integers(0, len(own))]
                nb = [(r + dr, c + dc) for dr in (-1, 0, 1) for dc in (-1, 0, 1) if (dr or dc)]
                nb = [(rr, cc) for rr, cc in nb if 0 <= rr < n and 0 <= cc < n and b[rr, cc] == 0]
                if nb:
                    rr, cc = nb[rng.integers(0, len(nb))]
                    choice = int(rr * n + cc)
        out[e] = choice
    return out


def play(name: str, seed: int, E: int, n: int, win: int, steps: int, mode: str, partial_reset_every: int = 0) -> None:
    rng = np.random.default_rng(seed)
    env = VectorConnect6(E, n, win, device="cpu")
    rec = {k: [] for k in ("actions", "reward", "done", "winner", "transition_sign", "game_lengths", "reset_idx")}
    snaps = {}
    for t in range(steps):
        a = pick_actions(rng, env, mode)
        step = env.step(torch.from_numpy(a))
        rec["actions"].append(a)
        rec["reward"].append(step.reward.numpy().copy())
        rec["done"].append(step.done.numpy().copy())
        rec["winner"].append(step.winner.numpy().copy())
        rec["transition_sign"].append(step.transition_sign.numpy().copy())
        rec["game_lengths"].append(step.game_lengths.numpy().copy())
        idx = torch.nonzero(step.done, as_tuple=False).flatten()
        if partial_reset_every and t % partial_reset_every == partial_reset_every - 1:
            extra = torch.from_numpy(rng.choice(E, size=max(1, E // 8), replace=False).astype(np.int64))
            idx = torch.unique(torch.cat((idx, extra)))
        pad = np.full(E, -1, np.int64)
        pad[: idx.numel()] = idx.numpy()
        rec["reset_idx"].append(pad)
        env.reset(idx)
        if t in (steps // 3, steps - 1):
            snaps[f"boards_{t}"] = env.boards.numpy().copy()
            snaps[f"player_{t}"] = env.current_player.numpy().copy()
            snaps[f"stones_{t}"] = env.stones_left.numpy().copy()
            snaps[f"empty_{t}"] = env.empty_count.numpy().copy()
            snaps[f"moves_{t}"] = env.move_count.numpy().copy()
            snaps[f"legal_{t}"] = env.legal_mask().numpy().copy()
    out = {k: np.stack(v) for k, v in rec.items()}
    done = out["done"]
    print(f"{name}: {steps} steps x {E} envs, finished games {int(done.sum())}, wins {int((out['winner'] != 0).sum())}, "
          f"draws {int((done & (out['winner'] == 0)).sum())}")
    np.savez_compressed(HERE / f"{name}.npz", board_size=n, win_length=win, num_envs=E, snapshot_steps=np.array(
        [steps // 3, steps - 1]), **out, **snaps)


def main() -> None:
    play("env_19x19_win6_cluster", seed=61, E=24, n=19, win=6, steps=260, mode="cluster")
    play("env_7x7_win4_uniform", seed=62, E=16, n=7, win=4, steps=160, mode="uniform", partial_reset_every=17)
    play("env_5x5_win5_sloppy", seed=63, E=8, n=5, win=5, steps=150, mode="sloppy")
    play("env_5x5_win5_uniform", seed=64, E=8, n=5, win=5, steps=130, mode="uniform")


if __name__ == "__main__":
    main()
