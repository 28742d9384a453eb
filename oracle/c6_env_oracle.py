"""CPU oracle for the vectorised Connect6 environment step (TEST INFRASTRUCTURE ONLY).

Plain numpy / Python-loop restatement of the integer work the reference project
mgxmateusz/connect6 does per self-play step outside the network: placing a stone, the local
win test, turn hand-over, reset, and the rollout collector's finished-game bookkeeping.
Nothing in the shipped package imports it.

Pinning: EnvOracle.step / reset / legal_mask are checked move by move against games played by
the unmodified reference environment on CPU (tests/golden/env_*.npz, made by
tests/golden/make_golden_env.py).  CollectorOracle.collect_done restates a block of statements
inside the reference's training loop that is not callable on its own; it is pinned by
tests/golden/collector_*.npz, recorded while those very statements -- cut out of the reference's
syntax tree by the fixture generator and executed unchanged -- ran on the reference environment
with the reference's historical-table layout (finished indices, the nine sums, episode ids and
records, segment lengths, colour swaps, resets after every step).

Reference citations (paths inside the reference project):
  connect6/vector_env.py:34-53    state tensors and dtypes          -> EnvOracle.__init__
  connect6/vector_env.py:77-92    reset                             -> EnvOracle.reset
  connect6/vector_env.py:94-95    legal_mask                        -> EnvOracle.legal_mask
  connect6/vector_env.py:106-164  step                              -> EnvOracle.step
  connect6/vector_env.py:166-193  _check_win_local                  -> EnvOracle._wins
  connect6/train.py:702-721       collector state                   -> CollectorOracle.__init__
  connect6/train.py:866-941       finished-game bookkeeping         -> CollectorOracle.collect_done
"""
from __future__ import annotations

import numpy as np

DIRECTIONS = ((1, 0), (0, 1), (1, 1), (1, -1))
UNKNOWN_EPISODE_RESULT = 2   # connect6/train.py:26
UNKNOWN_TERMINAL_MOVE = -1   # connect6/train.py:27


class EnvOracle:
    def __init__(self, num_envs: int, board_size: int = 19, win_length: int = 6) -> None:
        self.num_envs, self.board_size, self.win_length = int(num_envs), int(board_size), int(win_length)
        n = self.board_size
        self.boards = np.zeros((num_envs, n, n), np.int8)
        self.current_player = np.ones(num_envs, np.int8)
        self.stones_left = np.ones(num_envs, np.int8)
        self.empty_count = np.full(num_envs, n * n, np.int16)
        self.move_count = np.zeros(num_envs, np.int16)

    def reset(self, indices=None) -> None:
        idx = np.arange(self.num_envs) if indices is None else np.asarray(indices, np.int64).reshape(-1)
        self.boards[idx] = 0
        self.current_player[idx] = 1
        self.stones_left[idx] = 1
        self.empty_count[idx] = self.board_size * self.board_size
        self.move_count[idx] = 0

    def legal_mask(self) -> np.ndarray:
        return self.boards.reshape(self.num_envs, -1) == 0

    def _wins(self, e: int, r: int, c: int, who: int) -> bool:
        """True if the stone just placed at (r, c) lies in a line of >= win_length stones of `who`:
        1 + (contiguous stones on one side) + (contiguous stones on the other), each side looking at
        most win_length - 1 cells away, over the four line directions."""
        n, b = self.board_size, self.boards[e]
        for dr, dc in DIRECTIONS:
            total = 1
            for sgn in (1, -1):
                for s in range(1, self.win_length):
                    rr, cc = r + sgn * dr * s, c + sgn * dc * s
                    if not (0 <= rr < n and 0 <= cc < n) or b[rr, cc] != who:
                        break
                    total += 1
            if total >= self.win_length:
                return True
        return False

    def step(self, actions) -> dict:
        actions = np.asarray(actions, np.int64)
        assert actions.shape == (self.num_envs,)
        E, n = self.num_envs, self.board_size
        reward = np.zeros(E, np.float32)
        done = np.zeros(E, bool)
        winner = np.zeros(E, np.int8)
        sign = np.zeros(E, np.int8)
        with np.errstate(over="ignore"):
            for e in range(E):
                r, c = divmod(int(actions[e]), n)
                actor = int(self.current_player[e])
                self.boards[e, r, c] = actor                      # an occupied cell is overwritten silently
                self.empty_count[e] = np.int16(self.empty_count[e] - np.int16(1))
                self.move_count[e] = np.int16(self.move_count[e] + np.int16(1))
                won = self._wins(e, r, c, actor)
                over = won or self.empty_count[e] == 0
                done[e], reward[e], winner[e] = over, float(won), actor if won else 0
                if over:
                    continue                                      # turn state of a finished game is left as it is
                remaining = int(self.stones_left[e]) - 1
                if remaining > 0:
                    self.stones_left[e], sign[e] = remaining, 1
                else:
                    self.current_player[e], self.stones_left[e], sign[e] = -actor, 2, -1
        return {"reward": reward, "done": done, "winner": winner, "transition_sign": sign,
                "game_lengths": self.move_count.copy()}


class CollectorOracle:
    """Per-environment bookkeeping of the rollout collector and its finished-game update."""

    def __init__(self, env: EnvOracle, episode_capacity: int, historical_mask=None, historical_current_colors=None):
        E = env.num_envs
        self.env = env
        self.current_segment_lengths = np.zeros(E, np.int32)
        self.current_episode_ids = np.arange(E, dtype=np.int32)
        self.next_episode_id = E
        self.episode_results = np.full(episode_capacity, UNKNOWN_EPISODE_RESULT, np.int8)
        self.episode_terminal_moves = np.full(episode_capacity, UNKNOWN_TERMINAL_MOVE, np.int16)
        self.historical_mask = np.zeros(E, bool) if historical_mask is None else np.asarray(historical_mask, bool).copy()
        self.historical_current_colors = (np.ones(E, np.int8) if historical_current_colors is None
                                          else np.asarray(historical_current_colors, np.int8).copy())

    def collect_done(self, step: dict):
        """Returns (done_idx ascending, stats int64[10]): the nine sums the reference sends to the
        host per step, then the number of finished games."""
        done_idx = np.flatnonzero(step["done"]).astype(np.int64)
        stats = np.zeros(10, np.int64)
        if done_idx.size == 0:
            return done_idx, stats
        ids = self.current_episode_ids[done_idx].astype(np.int64)
        winners = step["winner"][done_idx]
        lengths = step["game_lengths"][done_idx].astype(np.int64)
        self.episode_results[ids] = winners
        self.episode_terminal_moves[ids] = lengths.astype(np.int16)
        hist = self.historical_mask[done_idx]
        colours = self.historical_current_colors[done_idx]
        stats[:] = (self.current_segment_lengths[done_idx].astype(np.int64).sum(), (winners == 1).sum(),
                    (winners == -1).sum(), (winners == 0).sum(), lengths.sum(), hist.sum(),
                    (hist & (winners == colours)).sum(), (hist & (winners == -colours)).sum(),
                    (hist & (winners == 0)).sum(), done_idx.size)
        self.env.reset(done_idx)
        self.current_segment_lengths[done_idx] = 0
        self.current_episode_ids[done_idx] = np.arange(self.next_episode_id, self.next_episode_id + done_idx.size,
                                                       dtype=np.int64).astype(np.int32)
        self.next_episode_id += int(done_idx.size)
        self.historical_current_colors[done_idx] = np.where(hist, -colours, colours)
        return done_idx, stats
