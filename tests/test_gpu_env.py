"""The environment kernels through the C ABI (connect6_b200.vector_env) against recorded reference
games, the numpy oracle and the torch restatement.  Integer work: everything is bit-exact."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import c6_env_oracle as EO
import c6_oracle as O
import torch_port as TP
from conftest import GOLDEN
from test_env_oracle import COLLECTOR_FIXTURES, ENV_FIXTURES, replay, replay_collector

pytestmark = pytest.mark.gpu


def _snapshot(env):
    return {"boards": env.boards.cpu().numpy(), "player": env.current_player.cpu().numpy(),
            "stones": env.stones_left.cpu().numpy(), "empty": env.empty_count.cpu().numpy(),
            "moves": env.move_count.cpu().numpy(), "legal": env.legal_mask().cpu().numpy()}


def _step_np(env, a, phase=0):
    s = env.step(torch.from_numpy(np.asarray(a, np.int64)), view_phase=phase)
    return {"reward": s.reward.cpu().numpy(), "done": s.done.cpu().numpy(), "winner": s.winner.cpu().numpy(),
            "transition_sign": s.transition_sign.cpu().numpy(), "game_lengths": s.game_lengths.cpu().numpy()}


@pytest.mark.parametrize("name", ENV_FIXTURES)
def test_env_kernels_replay_reference_games(cuda_device, name):
    from connect6_b200.vector_env import VectorConnect6
    fx = np.load(GOLDEN / f"{name}.npz")
    replay(fx, lambda E, n, w: VectorConnect6(E, n, w, device=cuda_device), _step_np,
           lambda env, idx: env.reset(torch.from_numpy(idx).to(cuda_device)), _snapshot)


def _random_legal(env, gen, corner: int = 0):
    """One uniformly drawn empty cell per environment; with corner = k only cells of the top-left
    k x k square are drawn while that square has room (stones crowd together, lines form early)."""
    legal = env.legal_mask().float()
    if corner:
        n = env.board_size
        inside = torch.zeros(n, n, device=legal.device)
        inside[:corner, :corner] = 1.0
        crowded = legal * inside.reshape(1, -1)
        legal = torch.where(crowded.sum(1, keepdim=True) > 0, crowded, legal)
    legal[legal.sum(1) == 0] = 1.0
    return torch.multinomial(legal, 1, generator=gen).squeeze(1)


@pytest.mark.parametrize("E,n,win", [(1, 19, 6), (257, 9, 5), (3000, 19, 6), (513, 3, 3), (130, 40, 7), (64, 6, 1)])
def test_env_step_matches_torch_port_on_large_batches(cuda_device, E, n, win):
    """Random legal play with view-phase actions; the CPU torch restatement steps the same games."""
    from connect6_b200.vector_env import VectorConnect6
    env = VectorConnect6(E, n, win, device=cuda_device)
    ref = [torch.zeros(E, n, n, dtype=torch.int8), torch.ones(E, dtype=torch.int8), torch.ones(E, dtype=torch.int8),
           torch.full((E,), n * n, dtype=torch.int16), torch.zeros(E, dtype=torch.int16)]
    gen = torch.Generator(device=cuda_device).manual_seed(11)
    finished = 0
    for t in range(150 if E < 3000 else 120):
        phase = t % 8
        a = _random_legal(env, gen)
        k, flip = O.symmetry_for_phase(phase)
        a_view = torch.from_numpy(O.transform_actions(a.cpu().numpy(), n, k, flip)).to(cuda_device)
        step = env.step(a_view, view_phase=phase)
        want = TP.env_step_torch(*ref, a.cpu(), win)
        got = (step.reward, step.done, step.winner, step.transition_sign, step.game_lengths)
        for g, w in zip(got, want):
            assert g.dtype == w.dtype and torch.equal(g.cpu(), w)
        idx = torch.nonzero(step.done).flatten()
        finished += idx.numel()
        env.reset(idx)
        ci = idx.cpu()
        ref[0][ci] = 0; ref[1][ci] = 1; ref[2][ci] = 1; ref[3][ci] = n * n; ref[4][ci] = 0
    for mine, theirs in zip((env.boards, env.current_player, env.stones_left, env.empty_count, env.move_count), ref):
        assert torch.equal(mine.cpu(), theirs)
    assert int(env.faults.sum()) == 0
    if E >= 257:
        assert finished > 0


def test_env_edge_cases_and_faults(cuda_device):
    from connect6_b200.vector_env import VectorConnect6
    empty = VectorConnect6(0, 19, 6, device=cuda_device)
    s = empty.step(torch.zeros(0, dtype=torch.long, device=cuda_device))
    assert s.done.shape == (0,) and empty.legal_mask().shape == (0, 361)
    empty.reset()
    with pytest.raises(RuntimeError):
        VectorConnect6(4, device="cpu")
    env = VectorConnect6(4, 5, 3, device=cuda_device)
    with pytest.raises(ValueError):
        env.step(torch.zeros(3, dtype=torch.long, device=cuda_device))
    env.step(torch.tensor([0, 1, 2, 3], device=cuda_device))
    before = _snapshot(env)
    # env 0 replays an occupied cell (silently overwritten, counted); env 1 gets an action off the board
    s = env.step(torch.tensor([0, 25, 7, -1], device=cuda_device))
    after = _snapshot(env)
    assert env.faults.tolist() == [1, 2, 0, 0]
    for k in ("boards", "player", "stones", "empty", "moves"):
        assert np.array_equal(before[k][[1, 3]], after[k][[1, 3]]), k
    assert after["empty"][0] == 23 and after["moves"][0] == 2 and after["boards"][0, 0, 0] == -1
    assert s.done.tolist() == [False] * 4
    checked = VectorConnect6(2, 5, 3, device=cuda_device, debug_checks=True)
    checked.step(torch.tensor([3, 4], device=cuda_device))
    held = _snapshot(checked)
    for bad_actions, phase in (([3, 5], 0), ([6, 25], 0), ([1, 0], 4)):   # occupied; off the board; occupied through view 4
        with pytest.raises(RuntimeError, match="no environment was changed"):
            checked.step(torch.tensor(bad_actions, device=cuda_device), view_phase=phase)
        now = _snapshot(checked)
        assert all(np.array_equal(held[k], now[k]) for k in held)          # raised before touching any state
    assert checked.faults.tolist() == [0, 0, 0, 0]
    # partial reset with duplicates, a boolean mask, and out-of-range entries that are skipped
    env.reset(torch.tensor([2, 2, 99, -5], device=cuda_device))
    st = _snapshot(env)
    assert (st["boards"][2] == 0).all() and st["moves"][2] == 0 and st["moves"][0] == 2
    env.reset(torch.tensor([True, False, False, False], device=cuda_device))
    assert _snapshot(env)["moves"].tolist()[0] == 0


@pytest.mark.parametrize("E,n,win,with_history", [(1000, 5, 4, True), (300, 7, 4, False), (8192, 19, 6, True)])
def test_collect_done_matches_collector_oracle(cuda_device, E, n, win, with_history):
    """Finished-game bookkeeping: indices, per-episode records, statistics, resets, new episode ids
    and colour swaps equal the CPU restatement after every step."""
    from connect6_b200.vector_env import RolloutBookkeeper, VectorConnect6
    rng = np.random.default_rng(3)
    hist = (rng.random(E) < 0.4) if with_history else None
    colours = np.where(rng.random(E) < 0.5, 1, -1).astype(np.int8) if with_history else None
    env = VectorConnect6(E, n, win, device=cuda_device)
    steps = 120 if E < 8192 else 40
    capacity = E + E * steps
    book = RolloutBookkeeper(env, capacity, None if hist is None else torch.from_numpy(hist),
                             None if colours is None else torch.from_numpy(colours))
    o_env = EO.EnvOracle(E, n, win)
    o_col = EO.CollectorOracle(o_env, capacity, hist, colours)
    gen = torch.Generator(device=cuda_device).manual_seed(5)
    use_oracle_step = E <= 1000
    total_done = 0
    for t in range(steps):
        a = _random_legal(env, gen, corner=7 if E == 8192 else 0)
        book.current_segment_lengths += 1
        o_col.current_segment_lengths += 1
        step = env.step(a)
        if use_oracle_step:
            o_step = o_env.step(a.cpu().numpy())
        else:
            ref = [torch.from_numpy(x) for x in (o_env.boards, o_env.current_player, o_env.stones_left,
                                                  o_env.empty_count, o_env.move_count)]
            out = TP.env_step_torch(*ref, a.cpu(), win)
            o_step = dict(zip(("reward", "done", "winner", "transition_sign", "game_lengths"), (x.numpy() for x in out)))
        assert np.array_equal(step.done.cpu().numpy(), o_step["done"])
        done_idx, stats = book.collect(step)
        want_idx, want_stats = o_col.collect_done(o_step)
        stats = stats.cpu().numpy()
        assert np.array_equal(stats, want_stats), (t, stats, want_stats)
        assert np.array_equal(done_idx[: want_idx.size].cpu().numpy(), want_idx)
        total_done += int(stats[9])
        if t % 10 == 9 or t == steps - 1:
            assert np.array_equal(book.current_episode_ids.cpu().numpy(), o_col.current_episode_ids)
            assert np.array_equal(book.current_segment_lengths.cpu().numpy(), o_col.current_segment_lengths)
            assert int(book.next_episode_id) == o_col.next_episode_id
            assert np.array_equal(env.boards.cpu().numpy(), o_env.boards)
            assert np.array_equal(env.move_count.cpu().numpy(), o_env.move_count)
            assert np.array_equal(env.current_player.cpu().numpy(), o_env.current_player)
            if with_history:
                assert np.array_equal(book.historical_current_colors.cpu().numpy(), o_col.historical_current_colors)
    assert np.array_equal(book.episode_results.cpu().numpy(), o_col.episode_results)
    assert np.array_equal(book.episode_terminal_moves.cpu().numpy(), o_col.episode_terminal_moves)
    assert total_done > 0 and int(env.faults.sum()) == 0


@pytest.mark.parametrize("name", COLLECTOR_FIXTURES)
def test_collect_done_replays_reference_bookkeeping(cuda_device, name):
    """c6_env_collect_done against fixtures recorded while the reference's own collector statements
    (connect6/train.py:871-943) ran on the reference environment."""
    from connect6_b200.vector_env import RolloutBookkeeper, VectorConnect6
    fx = np.load(GOLDEN / f"{name}.npz")

    def make(E, n, win, capacity, hist, colours):
        env = VectorConnect6(E, n, win, device=cuda_device)
        return env, RolloutBookkeeper(env, capacity, torch.from_numpy(hist), torch.from_numpy(colours))

    def bump(obj, mask):
        obj[1].current_segment_lengths[torch.from_numpy(mask).to(cuda_device)] += 1

    def step(obj, a):
        s = obj[0].step(torch.from_numpy(np.asarray(a, np.int64)))
        return {"done": s.done.cpu().numpy(), "winner": s.winner.cpu().numpy(),
                "game_lengths": s.game_lengths.cpu().numpy(), "_step": s}

    def collect(obj, out):
        idx, stats = obj[1].collect(out["_step"])
        return idx.cpu().numpy(), stats.cpu().numpy()

    replay_collector(fx, lambda *a: list(make(*a)), bump, step, collect,
                     lambda obj: {"episode_ids": obj[1].current_episode_ids.cpu().numpy(),
                                  "segment_lengths": obj[1].current_segment_lengths.cpu().numpy(),
                                  "colors": obj[1].historical_current_colors.cpu().numpy(),
                                  "next_episode_id": int(obj[1].next_episode_id),
                                  "episode_results": obj[1].episode_results.cpu().numpy(),
                                  "episode_terminal_moves": obj[1].episode_terminal_moves.cpu().numpy(),
                                  "boards": obj[0].boards.cpu().numpy(), "moves": obj[0].move_count.cpu().numpy()})


def test_collect_done_flags_episode_ids_beyond_capacity(cuda_device):
    from connect6_b200.vector_env import RolloutBookkeeper, VectorConnect6
    env = VectorConnect6(4, 3, 1, device=cuda_device)        # win_length 1: every first stone wins
    book = RolloutBookkeeper(env, 6)
    step = env.step(torch.tensor([0, 1, 2, 3], device=cuda_device))
    assert step.done.all() and step.winner.tolist() == [1, 1, 1, 1]
    _, stats = book.collect(step)
    assert stats.tolist() == [0, 4, 0, 0, 4, 0, 0, 0, 0, 4]
    assert book.current_episode_ids.tolist() == [4, 5, 6, 7]
    _, stats = book.collect(env.step(torch.tensor([0, 1, 2, 3], device=cuda_device)))
    assert env.faults.tolist() == [0, 0, 2, 0]               # ids 6 and 7 do not fit 6 slots
    assert book.episode_results.tolist() == [1, 1, 1, 1, 1, 1]
