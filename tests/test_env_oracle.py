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


COLLECTOR_FIXTURES = ["collector_7x7_win4_history", "collector_5x5_win5_draws", "collector_19x19_win6_plain"]


def replay_collector(fx, make, bump_segments, step_fn, collect_fn, state_fn):
    """Drive an environment + collector through a game recorded while the reference's own
    bookkeeping statements (connect6/train.py:871-943) ran, and compare what they did after every
    step: finished indices, the nine sums, episode ids, segment lengths, colours, the id counter."""
    E = int(fx["num_envs"])
    obj = make(E, int(fx["board_size"]), int(fx["win_length"]), int(fx["episode_capacity"]), fx["historical_mask"],
               fx["initial_colors"])
    for t in range(fx["actions"].shape[0]):
        bump_segments(obj, fx["seg_inc"][t])
        out = step_fn(obj, fx["actions"][t])
        for k in ("done", "winner", "game_lengths"):
            assert np.array_equal(np.asarray(out[k]), fx[k][t]), (k, t)
        done_idx, stats = collect_fn(obj, out)
        want_idx = fx["done_idx"][t]
        want_idx = want_idx[want_idx >= 0]
        assert np.array_equal(np.asarray(stats), fx["stats"][t]), (t, stats, fx["stats"][t])
        assert np.array_equal(np.asarray(done_idx)[: want_idx.size], want_idx), t
        st = state_fn(obj)
        assert np.array_equal(st["episode_ids"], fx["episode_ids"][t]), t
        assert np.array_equal(st["segment_lengths"], fx["segment_lengths"][t]), t
        assert np.array_equal(st["colors"], fx["colors"][t]), t
        assert int(st["next_episode_id"]) == int(fx["next_episode_id"][t]), t
    st = state_fn(obj)
    assert np.array_equal(st["episode_results"], fx["episode_results"])
    assert np.array_equal(st["episode_terminal_moves"], fx["episode_terminal_moves"])
    assert np.array_equal(st["boards"], fx["final_boards"]) and np.array_equal(st["moves"], fx["final_moves"])
    # the reference's host-side running totals are the column sums of the per-step statistics
    totals = fx["stats"].sum(0)
    assert np.array_equal(fx["counters"][-1], totals[[0, 9, 1, 2, 3, 4, 5, 6, 7, 8]])


@pytest.mark.parametrize("name", COLLECTOR_FIXTURES)
def test_collector_oracle_replays_reference_bookkeeping(name):
    fx = np.load(GOLDEN / f"{name}.npz")

    def make(E, n, win, capacity, hist, colours):
        env = EO.EnvOracle(E, n, win)
        return env, EO.CollectorOracle(env, capacity, hist, colours)

    def bump(obj, mask):
        obj[1].current_segment_lengths[mask] += 1

    replay_collector(fx, make, bump, lambda obj, a: obj[0].step(a), lambda obj, out: obj[1].collect_done(out),
                     lambda obj: {"episode_ids": obj[1].current_episode_ids, "segment_lengths": obj[1].current_segment_lengths,
                                  "colors": obj[1].historical_current_colors, "next_episode_id": obj[1].next_episode_id,
                                  "episode_results": obj[1].episode_results,
                                  "episode_terminal_moves": obj[1].episode_terminal_moves,
                                  "boards": obj[0].boards, "moves": obj[0].move_count})


def test_collector_fixtures_cover_history_outcomes():
    tot = sum(np.load(GOLDEN / f"{n}.npz")["stats"].sum(0) for n in COLLECTOR_FIXTURES)
    assert tot[9] > 300 and tot[6] > 20 and tot[7] > 20 and tot[8] > 5 and tot[3] > 20


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
