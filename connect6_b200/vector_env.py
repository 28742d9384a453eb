"""Drop-in for the reference's vectorised environment (`connect6/vector_env.py`): same class,
attributes, methods and result types, with the per-step integer work done by the library's own
kernels (one launch per `step`, in place on the state tensors) instead of some thirty small
PyTorch kernels.  CUDA only: there is no CPU implementation in this package.

Additions beyond the reference's surface: `step(actions, view_phase=p)` folds the
`_inverse_transform_actions` call of `connect6/train.py:846-853` into the step, and
`RolloutBookkeeper` does the finished-game bookkeeping of `connect6/train.py:866-941` on the
device without a host synchronisation.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib as L
from .selfplay import canonical_network_input

UNKNOWN_EPISODE_RESULT = 2      # connect6/train.py:26
UNKNOWN_TERMINAL_MOVE = -1      # connect6/train.py:27


@dataclass(slots=True)
class StepBatch:
    """connect6/vector_env.py:8-14."""
    reward: torch.Tensor
    done: torch.Tensor
    winner: torch.Tensor
    transition_sign: torch.Tensor
    game_lengths: torch.Tensor


def canonical_observation(boards: torch.Tensor, current_player: torch.Tensor, stones_left: torch.Tensor) -> torch.Tensor:
    """connect6/vector_env.py:221-226."""
    return canonical_network_input(boards, current_player, stones_left)


class VectorConnect6:
    """connect6/vector_env.py:17-193: num_envs independent Connect6 games stepped together."""

    def __init__(self, num_envs: int, board_size: int = 19, win_length: int = 6,
                 device: str | torch.device = "cuda", debug_checks: bool = False) -> None:
        self.num_envs = int(num_envs)
        self.board_size = int(board_size)
        self.win_length = int(win_length)
        self.device = torch.device(device)
        self.debug_checks = bool(debug_checks)
        if self.device.type != "cuda":
            raise RuntimeError(f"VectorConnect6: expected a CUDA device, got {self.device} (no CPU path in this package)")
        if not (1 <= self.win_length <= self.board_size <= 127):
            raise ValueError(f"need 1 <= win_length <= board_size <= 127, got {self.win_length}, {self.board_size}")
        L.load()
        dev = self.device
        self.boards = torch.zeros((self.num_envs, self.board_size, self.board_size), dtype=torch.int8, device=dev)
        self.current_player = torch.ones(self.num_envs, dtype=torch.int8, device=dev)
        self.stones_left = torch.ones(self.num_envs, dtype=torch.int8, device=dev)
        self.empty_count = torch.full((self.num_envs,), self.board_size * self.board_size, dtype=torch.int16, device=dev)
        self.move_count = torch.zeros(self.num_envs, dtype=torch.int16, device=dev)
        # Device counters the step and bookkeeping kernels only ever increment (slots C6_ENV_FAULT_* of
        # include/c6_env.h: stones on occupied cells, actions outside the board, episode ids beyond the
        # record arrays).  With debug_checks off nothing raises: poll this tensor when convenient.
        self.faults = torch.zeros(L.C6_ENV_FAULT_COUNT, dtype=torch.int32, device=dev)

    # ---- reference surface -------------------------------------------------------------------
    @property
    def action_size(self) -> int:
        return self.board_size * self.board_size

    @property
    def input_channels(self) -> int:
        return 3

    def _state(self) -> L.C6EnvState:
        for t in (self.boards, self.current_player, self.stones_left, self.empty_count, self.move_count):
            if not (t.is_cuda and t.is_contiguous()):
                raise RuntimeError("VectorConnect6: state tensors must stay contiguous CUDA tensors")
        return L.C6EnvState(self.boards.data_ptr(), self.current_player.data_ptr(), self.stones_left.data_ptr(),
                            self.empty_count.data_ptr(), self.move_count.data_ptr(), self.num_envs,
                            self.board_size, self.win_length)

    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def reset(self, indices: torch.Tensor | None = None) -> None:
        """connect6/vector_env.py:77-92."""
        st = self._state()
        with torch.cuda.device(self.device):
            if indices is None:
                L.check(L.load().c6_env_reset(C.byref(st), None, 0, self._stream()), None, "c6_env_reset")
                return
            if indices.numel() == 0:
                return
            if indices.dtype == torch.bool:
                indices = torch.nonzero(indices, as_tuple=False).flatten()
            idx = indices.to(device=self.device, dtype=torch.int64).contiguous().flatten()
            L.check(L.load().c6_env_reset(C.byref(st), idx.data_ptr(), idx.numel(), self._stream()), None, "c6_env_reset")

    def legal_mask(self) -> torch.Tensor:
        """connect6/vector_env.py:94-95."""
        out = torch.empty((self.num_envs, self.action_size), dtype=torch.bool, device=self.device)
        st = self._state()
        with torch.cuda.device(self.device):
            L.check(L.load().c6_env_legal_mask(C.byref(st), out.data_ptr(), self._stream()), None, "c6_env_legal_mask")
        return out

    def network_input(self) -> torch.Tensor:
        """connect6/vector_env.py:97-100."""
        return canonical_network_input(self.boards, self.current_player, self.stones_left)

    def observation(self) -> torch.Tensor:
        return self.network_input()

    @torch.no_grad()
    def step(self, actions: torch.Tensor, view_phase: int = 0) -> StepBatch:
        """connect6/vector_env.py:106-164.  With view_phase = p in 1..7 the actions are cell indices
        inside D4 view p (connect6/train.py:216-219) and are mapped back to board cells first."""
        actions = actions.to(device=self.device, dtype=torch.long, non_blocking=True)
        if actions.shape != (self.num_envs,):
            raise ValueError(f"expected actions of shape {(self.num_envs,)}, got {tuple(actions.shape)}")
        actions = actions.contiguous()
        dev = self.device
        if self.debug_checks and self.num_envs:
            # as the reference (connect6/vector_env.py:121-127): look first, raise before any state changes.
            # A debugging aid: it reads the result on the host.
            cells = self.board_size * self.board_size
            board_actions = actions
            if int(view_phase) % 8:
                from .selfplay import _inverse_transform_actions, _symmetry_for_phase
                board_actions = _inverse_transform_actions(actions, self.board_size, *_symmetry_for_phase(view_phase))
            outside = (actions < 0) | (actions >= cells)
            target = self.boards.reshape(self.num_envs, cells).gather(1, board_actions.clamp(0, cells - 1).unsqueeze(1))
            occupied = (target.squeeze(1) != 0) & ~outside
            n_out, n_occ = int(outside.sum()), int(occupied.sum())
            if n_out or n_occ:
                raise RuntimeError(f"step: {n_occ} stone(s) aimed at an occupied cell, {n_out} action(s) outside the "
                                   "board; no environment was changed")
        out = StepBatch(
            reward=torch.empty(self.num_envs, dtype=torch.float32, device=dev),
            done=torch.empty(self.num_envs, dtype=torch.bool, device=dev),
            winner=torch.empty(self.num_envs, dtype=torch.int8, device=dev),
            transition_sign=torch.empty(self.num_envs, dtype=torch.int8, device=dev),
            game_lengths=torch.empty(self.num_envs, dtype=torch.int16, device=dev),
        )
        st = self._state()
        with torch.cuda.device(dev):
            L.check(L.load().c6_env_step(C.byref(st), actions.data_ptr(), int(view_phase) % 8, out.reward.data_ptr(),
                                         out.done.data_ptr(), out.winner.data_ptr(), out.transition_sign.data_ptr(),
                                         out.game_lengths.data_ptr(), self.faults.data_ptr(), self._stream()),
                    None, "c6_env_step")
        return out


class RolloutBookkeeper:
    """The finished-game bookkeeping of the rollout collector (connect6/train.py:702-721, 866-941)
    kept on the device: episode ids, segment lengths, per-episode results, historical-table colours,
    and the per-step statistics vector.  `collect(step)` never synchronises; `stats` holds the nine
    sums of the reference's batch_stats followed by the number of finished games of the last call."""

    def __init__(self, env: VectorConnect6, episode_capacity: int, historical_mask: torch.Tensor | None = None,
                 historical_current_colors: torch.Tensor | None = None) -> None:
        self.env = env
        dev, E = env.device, env.num_envs
        self.current_segment_lengths = torch.zeros(E, dtype=torch.int32, device=dev)
        self.current_episode_ids = torch.arange(E, dtype=torch.int32, device=dev)
        self.next_episode_id = torch.full((1,), E, dtype=torch.int64, device=dev)
        self.episode_capacity = int(episode_capacity)
        self.episode_results = torch.full((self.episode_capacity,), UNKNOWN_EPISODE_RESULT, dtype=torch.int8, device=dev)
        self.episode_terminal_moves = torch.full((self.episode_capacity,), UNKNOWN_TERMINAL_MOVE, dtype=torch.int16,
                                                 device=dev)
        if (historical_mask is None) != (historical_current_colors is None):
            raise ValueError("historical_mask and historical_current_colors come together")
        self.historical_mask = None if historical_mask is None else historical_mask.to(dev, torch.bool).contiguous()
        self.historical_current_colors = (None if historical_current_colors is None
                                          else historical_current_colors.to(dev, torch.int8).contiguous())
        self.done_idx = torch.empty(E, dtype=torch.int64, device=dev)
        self.stats = torch.zeros(L.C6_STAT_COUNT, dtype=torch.int64, device=dev)
        ws = int(L.load().c6_env_collect_workspace_bytes(E))
        self._workspace = torch.empty((ws + 7) // 8, dtype=torch.int64, device=dev)

    def collect(self, step: StepBatch) -> tuple[torch.Tensor, torch.Tensor]:
        """Process the environments that `step` finished; returns (done_idx buffer, stats): the first
        stats[9] entries of done_idx are the finished environments in ascending order."""
        env = self.env
        st = env._state()
        col = L.C6CollectorState(self.current_episode_ids.data_ptr(), self.current_segment_lengths.data_ptr(),
                                 L.ptr(self.historical_mask), L.ptr(self.historical_current_colors),
                                 self.episode_results.data_ptr(), self.episode_terminal_moves.data_ptr(),
                                 self.episode_capacity, self.next_episode_id.data_ptr())
        with torch.cuda.device(env.device):
            L.check(L.load().c6_env_collect_done(C.byref(st), C.byref(col), step.done.data_ptr(), step.winner.data_ptr(),
                                                 step.game_lengths.data_ptr(), self.done_idx.data_ptr(),
                                                 self.stats.data_ptr(), env.faults.data_ptr(),
                                                 self._workspace.data_ptr(), env._stream()),
                    None, "c6_env_collect_done")
        return self.done_idx, self.stats
