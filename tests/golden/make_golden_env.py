"""Generate the environment fixtures (env_*.npz) in this directory from the UNMODIFIED reference.

Run where the reference checkout is importable:
    python tests/golden/make_golden_env.py [/path/to/reference]
It imports `connect6.vector_env.VectorConnect6` from that path (or from $C6_REFERENCE), plays seeded games with it on CPU and stores the actions, every step's outputs
and state snapshots.  The tests only read the .npz files; they never need the reference.

The collector fixtures (collector_*.npz) pin the finished-game bookkeeping of the reference's
rollout loop.  Those statements sit in the middle of `connect6.train.train()` and cannot be called,
so the generator cuts them out of the reference's syntax tree at run time -- the assignments that
set the collector state up (connect6/train.py:702-721) and the `done_idx = ...` / `if
done_idx.numel():` block (connect6/train.py:871-943) -- compiles those nodes unchanged and executes
them on the reference's own environment and `_historical_layout`.  No reference text is stored here.
"""
from __future__ import annotations

import ast
import os
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
if len(sys.argv) < 2 and "C6_REFERENCE" not in os.environ:
    raise SystemExit("usage: python " + sys.argv[0] + " /path/to/the/reference/checkout   (or set C6_REFERENCE)")
REF = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ["C6_REFERENCE"])
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


COLLECTOR_STATE = ("current_segment_lengths", "current_episode_ids", "next_episode_id", "episode_results",
                   "episode_terminal_moves")
COLLECTOR_COUNTERS = ("completed_positions", "update_games", "update_black", "update_white", "update_draws",
                      "game_length_sum", "update_hist_games", "update_hist_wins", "update_hist_losses",
                      "update_hist_draws")


def reference_collector_code():
    """(setup, block): code objects compiled from the reference's own statements inside train()."""
    tree = ast.parse((REF / "connect6" / "train.py").read_text())
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "train")
    first_assign, done_assign, done_if = {}, None, None
    for node in ast.walk(fn):
        if isinstance(node, ast.Assign) and len(node.targets) == 1 and isinstance(node.targets[0], ast.Name):
            name = node.targets[0].id
            if name in COLLECTOR_STATE and (name not in first_assign or node.lineno < first_assign[name].lineno):
                first_assign[name] = node
            if name == "done_idx":
                done_assign = node
        if isinstance(node, ast.If) and ast.unparse(node.test) == "done_idx.numel()":
            done_if = node
    assert set(first_assign) == set(COLLECTOR_STATE) and done_assign is not None and done_if is not None
    setup_nodes = sorted(first_assign.values(), key=lambda n: n.lineno)
    print(f"collector statements: setup lines {setup_nodes[0].lineno}-{setup_nodes[-1].end_lineno}, "
          f"block lines {done_assign.lineno}-{done_if.end_lineno} of connect6/train.py")

    def code(nodes, tag):
        mod = ast.Module(body=list(nodes), type_ignores=[])
        return compile(ast.fix_missing_locations(mod), f"<reference train.py: {tag}>", "exec")

    return code(setup_nodes, "collector state"), code([done_assign, done_if], "finished games")


def play_collector(name: str, seed: int, E: int, n: int, win: int, steps: int, mode: str, fraction: float,
                   models: int) -> None:
    """Play with the reference environment and run the reference's own bookkeeping statements after
    every step; store what they did to every piece of collector state."""
    import connect6.train as RT
    setup_code, block_code = reference_collector_code()
    rng = np.random.default_rng(seed)
    torch.manual_seed(seed)                       # _historical_layout shuffles colours with torch.randperm
    device = torch.device("cpu")
    env = VectorConnect6(E, n, win, device="cpu")
    hist_mask, _, hist_colors = RT._historical_layout(E, fraction, models, device)
    capacity = E * steps
    ns = {"torch": torch, "device": device, "num_envs": E, "env": env, "buffer": types.SimpleNamespace(capacity=capacity),
          "UNKNOWN_EPISODE_RESULT": RT.UNKNOWN_EPISODE_RESULT, "UNKNOWN_TERMINAL_MOVE": RT.UNKNOWN_TERMINAL_MOVE,
          "historical_mask": hist_mask, "historical_current_colors": hist_colors}
    ns.update({k: 0 for k in COLLECTOR_COUNTERS})
    exec(setup_code, ns)
    rec = {k: [] for k in ("actions", "seg_inc", "done", "winner", "game_lengths", "done_idx", "stats", "episode_ids",
                           "segment_lengths", "colors", "next_episode_id", "counters")}
    init_colors = hist_colors.numpy().copy()
    for t in range(steps):
        a = pick_actions(rng, env, mode)
        # the tables on which the current policy moves collect one more position (connect6/train.py:760-765, 811)
        actor = ~hist_mask | (hist_mask & env.current_player.eq(ns["historical_current_colors"]))
        ns["current_segment_lengths"][actor] += 1
        ns["step"] = env.step(torch.from_numpy(a))
        ns.pop("batch_stats", None)
        exec(block_code, ns)
        idx = ns["done_idx"]
        pad = np.full(E, -1, np.int64)
        pad[: idx.numel()] = idx.numpy()
        stats = np.zeros(10, np.int64)
        if idx.numel():
            stats[:9] = ns["batch_stats"].numpy()
            stats[9] = idx.numel()
        rec["actions"].append(a)
        rec["seg_inc"].append(actor.numpy().copy())
        rec["done"].append(ns["step"].done.numpy().copy())
        rec["winner"].append(ns["step"].winner.numpy().copy())
        rec["game_lengths"].append(ns["step"].game_lengths.numpy().copy())
        rec["done_idx"].append(pad)
        rec["stats"].append(stats)
        rec["episode_ids"].append(ns["current_episode_ids"].numpy().copy())
        rec["segment_lengths"].append(ns["current_segment_lengths"].numpy().copy())
        rec["colors"].append(ns["historical_current_colors"].numpy().copy())
        rec["next_episode_id"].append(np.int64(ns["next_episode_id"]))
        rec["counters"].append(np.array([ns[k] for k in COLLECTOR_COUNTERS], np.int64))
    out = {k: np.stack(v) for k, v in rec.items()}
    total = out["stats"].sum(0)
    print(f"{name}: {steps} steps x {E} envs, finished {int(total[9])}, historical finished {int(total[5])} "
          f"(won {int(total[6])}, lost {int(total[7])}, drawn {int(total[8])})")
    np.savez_compressed(HERE / f"{name}.npz", board_size=n, win_length=win, num_envs=E, episode_capacity=capacity + E + 1,
                        historical_mask=hist_mask.numpy(), initial_colors=init_colors,
                        episode_results=ns["episode_results"].numpy(),
                        episode_terminal_moves=ns["episode_terminal_moves"].numpy(),
                        final_boards=env.boards.numpy().copy(), final_moves=env.move_count.numpy().copy(), **out)


def main() -> None:
    play("env_19x19_win6_cluster", seed=61, E=24, n=19, win=6, steps=260, mode="cluster")
    play("env_7x7_win4_uniform", seed=62, E=16, n=7, win=4, steps=160, mode="uniform", partial_reset_every=17)
    play("env_5x5_win5_sloppy", seed=63, E=8, n=5, win=5, steps=150, mode="sloppy")
    play("env_5x5_win5_uniform", seed=64, E=8, n=5, win=5, steps=130, mode="uniform")
    play_collector("collector_7x7_win4_history", seed=71, E=24, n=7, win=4, steps=220, mode="cluster", fraction=0.5, models=3)
    play_collector("collector_5x5_win5_draws", seed=72, E=12, n=5, win=5, steps=160, mode="uniform", fraction=0.34, models=2)
    play_collector("collector_19x19_win6_plain", seed=73, E=16, n=19, win=6, steps=200, mode="cluster", fraction=0.0, models=0)


if __name__ == "__main__":
    main()
