"""Drop-in for the forward half of the reference's `connect6/history.py`: the ensemble of frozen
historical opponents evaluated as ONE grouped launch sequence.

The reference folds M checkpoints into channel groups and calls F.conv2d(groups=M) per layer
(connect6/history.py:251-303).  Here the M weight sets are packed once into an engine with
`groups = M`; every kernel of the pass takes the group as a scheduling dimension, so the
permute/reshape copies of the reference disappear.  Checkpoint discovery and caching
(connect6/history.py:35-183) are host bookkeeping and stay with the caller.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any

import torch

from .engine import Engine
from .model import DEFAULT_CHANNELS, DEFAULT_KERNELS


@dataclass(slots=True)
class HistoricalCheckpoint:
    """Lean checkpoint record, field-compatible with connect6/history.py:26-32."""
    path: Path
    update: int
    model_state: dict[str, torch.Tensor]
    model_config: dict[str, Any]
    game_config: dict[str, Any]


def _arch_of(cfg: dict[str, Any]) -> dict[str, Any]:
    return {k: v for k, v in dict(cfg).items() if k not in ("compile", "compile_mode")}


class HistoricalPolicyEnsemble:
    """M frozen policy CNNs evaluated together; input [M, T, 3, H, W] -> logits [M, T, H*W].

    Same constructor and attributes as connect6/history.py:186-232.  `dtype` picks the
    arithmetic like the reference's ensemble dtype: torch.bfloat16 / torch.float16 -> tensor-core
    modes, torch.float32 (or None) -> fp32 mode.  Outputs are returned in that dtype.
    """

    def __init__(self, checkpoints: list[HistoricalCheckpoint], device: torch.device, *,
                 dtype: torch.dtype | None = None) -> None:
        if not checkpoints:
            raise ValueError("HistoricalPolicyEnsemble needs at least 1 checkpoint")
        self.device = torch.device(device)
        self.dtype = dtype or torch.float32
        if self.dtype not in (torch.float32, torch.bfloat16, torch.float16):
            raise ValueError("ensemble dtype must be torch.float32, torch.bfloat16 or torch.float16")
        self.num_models = len(checkpoints)
        self.updates = [cp.update for cp in checkpoints]
        self.paths = [cp.path for cp in checkpoints]

        arch = _arch_of(checkpoints[0].model_config)
        self.board_size = int(checkpoints[0].game_config["board_size"])
        self.kernels = tuple(int(v) for v in arch.get("kernels", DEFAULT_KERNELS))
        self.channels = tuple(int(v) for v in arch.get("channels", DEFAULT_CHANNELS))
        self.input_channels = 3
        self.action_size = self.board_size * self.board_size
        for cp in checkpoints[1:]:
            if int(cp.game_config["board_size"]) != self.board_size:
                raise ValueError("historical checkpoints use different board sizes")
            if _arch_of(cp.model_config) != arch:
                raise ValueError("historical checkpoints have different CNN architectures")

        self.has_value = all("value_output.weight" in cp.model_state for cp in checkpoints)
        self._engine = Engine(self.device, self.board_size, self.kernels, self.channels, self.num_models,
                              {torch.bfloat16: "bf16", torch.float16: "f16"}.get(self.dtype, "fp32"))
        for g, cp in enumerate(checkpoints):
            try:
                self._engine.load_state_dict(cp.model_state, group=g, need_value=False)
            except KeyError as exc:
                raise KeyError(f"{exc.args[0]} in historical checkpoints") from exc

    def _check(self, x: torch.Tensor) -> None:
        if x.ndim != 5:
            raise ValueError("history ensemble expects input [MODELS, TABLES, 3, H, W]")
        tail = (self.input_channels, self.board_size, self.board_size)
        if x.shape[0] != self.num_models or tuple(x.shape[2:]) != tail:
            raise ValueError(
                f"bad history batch {tuple(x.shape)}; expected [{self.num_models}, T, {tail[0]}, {tail[1]}, {tail[2]}]"
            )

    @torch.no_grad()
    def forward_grouped(self, x: torch.Tensor) -> torch.Tensor:
        """connect6/history.py:276-303."""
        self._check(x)
        if x.device != self._engine.device:
            x = x.to(self._engine.device, non_blocking=True)
        if x.dtype not in (torch.float32, torch.bfloat16):
            x = x.float()
        logits, _ = self._engine.forward_grouped(x, want_value=False)
        return logits if self.dtype == torch.float32 else logits.to(self.dtype)

    @torch.no_grad()
    def forward_grouped_with_value(self, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """Per-group logits [M,T,A] and values [M,T] (each model's own PolicyValueNet.forward,
        connect6/model.py:96-111); needs value heads in every checkpoint."""
        self._check(x)
        if not self.has_value:
            raise KeyError("missing parameter value_output.weight in historical checkpoints")
        if x.device != self._engine.device:
            x = x.to(self._engine.device, non_blocking=True)
        if x.dtype not in (torch.float32, torch.bfloat16):
            x = x.float()
        return self._engine.forward_grouped(x, want_value=True)
