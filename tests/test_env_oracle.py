"""The environment oracle against games played by the unmodified reference (CPU only)."""
from __future__ import annotations

import numpy as np
import pytest

import c6_env_oracle as EO
from conftest import GOLDEN

ENV_FIXTURES = ["env_19x19_win6_cluster", "env_7x7_win4_uniform", "env_5x5_win5_sloppy", "env_5x5_win5_uniform"]


def replay(fx, make_env, step_fn, reset_fn, snapshot_fn):
    """Drive an environment through a recorded game and compare every output of every step."""
    E = int(fx["num_envs"])
    env = make_env(E, int(fx["board_size"]), int(fx["win_length"]))
    snaps = set(int(t) for t in fx["snapshot_steps"])
    for t in range(fx["actions"].shape[0]):
        out = step_fn(env, fx["actions"][t])
        for k in ("reward", "done", "winner", "transition_sign", "game_lengths"):
            got = np.asarray(out[k])
            assert got.dtype == fx[k].dtype, (k, got.dtype)
            assert np.array_equal(got, fx[k][t]), (k, t)
        idx = fx["reset_idx"][t]
        reset_fn(env, idx[idx >= 0])
        if t in snaps:
            state = snapshot_fn(env)
            for k in ("boards", "player", "stones", "empty", "moves", "legal"):
                assert np.array_equal(state[k], fx[f"{k}_{t}"]), (k, t)


@pytest.mark.parametrize("name", ENV_FIXTURES)
def test_env_oracle_replays_reference_games(name):
    fx = np.load(GOLDEN / f"{name}.npz")
    replay(fx, EO.EnvOracle, lambda env, a: env.step(a), lambda env, idx: env.reset(idx),
           lambda env: {"boards": env.boards, "player": env.current_player, "stones": env.stones_left,
                        "empty": env.empty_count, "moves": env.move_count, "legal": env.legal_mask()})


def test_fixtures_cover_wins_draws_and_overwrites():
    wins = draws = 0
    for name in ENV_FIXTURES:
        fx = np.load(GOLDEN / f"{name}.npz")
        wins += int((fx["winner"] != 0).sum())
        draws += int((fx["done"] & (fx["winner"] == 0)).sum())
    assert wins > 100 and draws > 20


def test_collector_oracle_invariants():
    rng = np.random.default_rng(5)
    E = 40
    env = EO.EnvOracle(E, 5, 4)
    hist = rng.random(E) < 0.5
    colours = np.where(rng.random(E) < 0.5, 1, -1).astype(np.int8)
    col = EO.CollectorOracle(env, 4000, hist, colours)
    total = np.zeros(10, np.int64)
    for t in range(200):
        legal = env.legal_mask()
        a = np.array([rng.choice(np.flatnonzero(legal[e])) for e in range(E)])
        col.current_segment_lengths += 1
        step = env.step(a)
        done_idx, stats = col.collect_done(step)
        assert np.array_equal(done_idx, np.flatnonzero(step["done"]))
        assert stats[9] == done_idx.size == stats[1] + stats[2] + stats[3]
        assert stats[5] == stats[6] + stats[7] + stats[8]
        assert (env.move_count[done_idx] == 0).all() and (env.boards[done_idx] == 0).all()
        total += stats
    finished = col.episode_results != EO.UNKNOWN_EPISODE_RESULT
    assert finished.sum() == total[9] and col.next_episode_id == E + total[9]
    assert col.episode_terminal_moves[finished].astype(np.int64).sum() == total[4]
    assert len(set(col.current_episode_ids.tolist())) == E


@pytest.mark.parametrize("impl", ["oracle_port", "bench_bar"])
@pytest.mark.parametrize("name", ENV_FIXTURES)
def test_torch_env_port_replays_reference_games(name, impl):
    """Both torch restatements -- the checker under oracle/ and the library timing bar inside
    bench.py -- reproduce the reference's games (win_length >= 2)."""
    import torch
    import torch_port as TP
    import bench
    fx = np.load(GOLDEN / f"{name}.npz")
    win = int(fx["win_length"])

    class State:
        def __init__(self, E, n, _win):
            self.boards = torch.zeros(E, n, n, dtype=torch.int8)
            self.player = torch.ones(E, dtype=torch.int8)
            self.stones = torch.ones(E, dtype=torch.int8)
            self.empty = torch.full((E,), n * n, dtype=torch.int16)
            self.moves = torch.zeros(E, dtype=torch.int16)

    def step(s, a):
        if impl == "oracle_port":
            out = TP.env_step_torch(s.boards, s.player, s.stones, s.empty, s.moves, torch.from_numpy(a), win)
        else:
            out = bench.stock_torch_env_step([s.boards, s.player, s.stones, s.empty, s.moves], torch.from_numpy(a), win)
        return dict(zip(("reward", "done", "winner", "transition_sign", "game_lengths"), (o.numpy() for o in out)))

    def reset(s, idx):
        idx = torch.from_numpy(idx)
        s.boards[idx] = 0
        s.player[idx] = 1
        s.stones[idx] = 1
        s.empty[idx] = s.boards.shape[-1] ** 2
        s.moves[idx] = 0

    replay(fx, State, step, reset,
           lambda s: {"boards": s.boards.numpy(), "player": s.player.numpy(), "stones": s.stones.numpy(),
                      "empty": s.empty.numpy(), "moves": s.moves.numpy(),
                      "legal": (s.boards.reshape(s.boards.shape[0], -1) == 0).numpy()})
