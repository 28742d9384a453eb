"""Drop-in for the reference's `connect6/model.py`: PolicyValueNet, build_model, mask_logits.

The module keeps the reference's constructor, attributes, parameter names and shapes
(connect6/model.py:26-94), so checkpoints, optimisers and `load_state_dict` work unchanged.
What changes is who executes the inference forward: without autograd the call goes to the
CUDA engine (hand-written sm_100a kernels behind a C ABI); with autograd enabled -- the PPO
update of connect6/train.py:1032-1056, which is outside this library's scope -- the PyTorch
modules that own the parameters run as before.  There is no CPU inference path: a CPU input
in inference mode raises.
"""
from __future__ import annotations

from typing import Any, Sequence

import torch
from torch import nn

from . import _lib as L
from .engine import Engine

DEFAULT_KERNELS = (23, 3, 3, 3, 3, 3, 3, 3)
DEFAULT_CHANNELS = (32, 32, 64, 64, 64, 96, 96, 96)


class PolicyValueNet(nn.Module):
    """Fully convolutional policy + value network for an n x n Connect6 board.

    Input [B, 3, n, n]: plane 0 = own stones, plane 1 = opponent stones, plane 2 = "this is
    the last stone of the turn".  Output: (logits [B, n*n] unmasked, value [B] in [-1, 1]).
    Mirrors connect6/model.py:9-111.

    `engine_backward=True` routes the backward of the 3x3 backbone layers in the grad-enabled forward (the PPO
    update, connect6/train.py:1047-1119) through the library's tensor-core kernels; parameters, optimizer and
    `loss.backward()` stay PyTorch's.

    `engine_precision` selects the engine's arithmetic: "bf16" (tcgen05 tensor cores, the
    default), "f16" (the same kernels with fp16 weights and activations: 11-bit significands,
    for callers that need the fp32 network's moves) or "fp32" (CUDA cores, reference-exact to
    1e-3).  It is an engine property and does not follow torch.autocast.
    """

    DEFAULT_KERNELS = DEFAULT_KERNELS
    DEFAULT_CHANNELS = DEFAULT_CHANNELS
    INPUT_CHANNELS = 3

    def __init__(self, board_size: int = 19, kernels: Sequence[int] | None = None,
                 channels: Sequence[int] | None = None, engine_precision: str = "bf16",
                 engine_backward: bool = False) -> None:
        super().__init__()
        self.board_size = int(board_size)
        self.action_size = self.board_size ** 2
        self.input_channels = self.INPUT_CHANNELS
        ks = tuple(DEFAULT_KERNELS if kernels is None else kernels)
        cs = tuple(DEFAULT_CHANNELS if channels is None else channels)
        # same rejections, in the same order, as connect6/model.py:40-47
        if len(ks) != len(cs):
            raise ValueError("kernels and channels must have the same number of entries")
        if len(ks) == 0:
            raise ValueError("the CNN needs at least one layer")
        if any(k <= 0 or k % 2 == 0 for k in ks):
            raise ValueError("every kernel must be a positive odd number")
        if any(c <= 0 for c in cs):
            raise ValueError("channel counts must be greater than zero")
        self.kernels = ks
        self.channels = cs
        self.engine_precision = engine_precision
        # True: in the grad-enabled forward (the PPO update) the backward of every 3x3 layer of up to 128
        # channels runs on the library's tensor-core kernels (train_ops.SiluConv3x3) instead of cuDNN's
        self.engine_backward = bool(engine_backward)

        widths = (self.input_channels,) + cs
        self.convs = nn.ModuleList(
            nn.Conv2d(widths[i], widths[i + 1], kernel_size=ks[i], stride=1, padding=ks[i] // 2, bias=True)
            for i in range(len(ks))
        )
        self.activation = nn.SiLU(inplace=True)
        self.policy_output = nn.Conv2d(cs[-1], 1, kernel_size=1, bias=True)
        self.value_output = nn.Conv2d(cs[-1], 1, kernel_size=1, bias=True)
        self.value_tanh = nn.Tanh()
        self._reset_parameters()

        # engine state: never part of state_dict
        self._engines: dict[tuple, Engine] = {}
        self._packed_versions: dict[tuple, tuple] = {}

    def __getstate__(self):
        # engines hold device handles: copies and pickles of the module start without them
        state = self.__dict__.copy()
        state["_engines"] = {}
        state["_packed_versions"] = {}
        return state

    # ---- reference-compatible surface -----------------------------------------------------------
    @property
    def receptive_field(self) -> int:
        return 1 + sum(k - 1 for k in self.kernels)

    def _reset_parameters(self) -> None:
        """Same initialisers in the same order as connect6/model.py:83-94, so a given
        torch seed yields the same weights as the reference module."""
        for conv in self.convs:
            nn.init.kaiming_normal_(conv.weight, nonlinearity="relu")
            nn.init.zeros_(conv.bias)
        for head in (self.policy_output, self.value_output):
            nn.init.normal_(head.weight, mean=0.0, std=0.01)
            nn.init.zeros_(head.bias)

    def _check_input(self, x: torch.Tensor) -> None:
        want = (self.input_channels, self.board_size, self.board_size)
        if x.ndim != 4 or tuple(x.shape[1:]) != want:
            raise ValueError(
                f"model input must have shape [B, {want[0]}, {want[1]}, {want[2]}], got {tuple(x.shape)}."
            )

    def forward(self, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        self._check_input(x)
        if torch.is_grad_enabled() and any(p.requires_grad for p in self.parameters()):
            return self.forward_autograd(x)
        logits, value = self.engine_for(x.device).forward(self._as_engine_input(x))
        return logits, value

    def forward_autograd(self, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """Differentiable forward (training only; not the inference engine).  By default on the PyTorch modules; with
        `engine_backward=True` and CUDA tensors the layers the library supports -- for the default architecture the whole
        network: stem, 3x3 layers, heads -- run forward and backward on its kernels (train_ops.PolicyValueStack), the
        parameters staying ordinary nn.Parameters whose .grad the backward fills."""
        feats = x
        use_engine = self.engine_backward and x.is_cuda
        convs = list(self.convs)
        if use_engine:
            from .train_ops import SiluConv3x3, SiluConvStack, supports_layer, supports_stem
            # the longest run of library-supported 3x3 layers that ends at the last layer goes through the library as
            # ONE operator (forward and backward, activations kept in the kernels' layout) -- together with the stem
            # when the run starts right behind it and the stem qualifies; layers before the run go one by one
            first = len(convs)
            while first > 0 and supports_layer(convs[first - 1], self.board_size):
                first -= 1
            if first == 1 and len(convs) >= 2 and supports_stem(convs[0], self.board_size) and x.dtype == torch.float32:
                first = 0
        for i, conv in enumerate(convs):
            if use_engine and i == first and len(convs) - first >= 2 and x.shape[0] > 0:
                params = [p for c in convs[first:] for p in (c.weight, c.bias)]
                if self.policy_output.bias is not None and self.value_output.bias is not None:
                    # ... and both heads with them: the features stay in the kernels' layout
                    from .train_ops import PolicyValueStack
                    return PolicyValueStack.apply(feats, *params, self.policy_output.weight, self.policy_output.bias,
                                                  self.value_output.weight, self.value_output.bias)
                feats = SiluConvStack.apply(feats, *params)
                break
            if use_engine and supports_layer(conv, self.board_size):
                feats = SiluConv3x3.apply(feats, conv.weight, conv.bias)
            else:
                feats = self.activation(conv(feats))
        logits = self.policy_output(feats).flatten(1)
        value = self.value_tanh(self.value_output(feats).mean(dim=(-2, -1))).squeeze(1)
        return logits, value

    # ---- engine management --------------------------------------------------------------------
    @staticmethod
    def _as_engine_input(x: torch.Tensor) -> torch.Tensor:
        if x.dtype in (torch.float32, torch.bfloat16):
            return x
        return x.float()

    def _param_versions(self) -> tuple:
        return tuple((p.data_ptr(), p._version) for p in self.parameters())

    def engine_for(self, device: torch.device | str) -> Engine:
        """Engine on `device` with weights matching the current parameters.  Parameters are
        re-packed whenever one of them was modified in place (optimizer step,
        load_state_dict) or re-allocated (.to())."""
        device = torch.device(device)
        if device.type != "cuda":
            raise RuntimeError(
                "PolicyValueNet inference runs on the CUDA engine only; got a tensor on "
                f"{device}. (Enable grad for the PyTorch training path.)"
            )
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        key = (device.index, self.engine_precision)
        eng = self._engines.get(key)
        if eng is None:
            eng = Engine(device, self.board_size, self.kernels, self.channels, 1, self.engine_precision)
            self._engines[key] = eng
            self._packed_versions.pop(key, None)
        versions = self._param_versions()
        if self._packed_versions.get(key) != versions:
            eng.load_state_dict({k: v for k, v in self.state_dict().items()}, group=0)
            self._packed_versions[key] = versions
        return eng

    # ---- fused entry points beyond the reference signature ----------------------------------------
    @torch.no_grad()
    def forward_masked(self, x: torch.Tensor, orient: torch.Tensor | None = None, inverse_map: bool = False):
        """forward + mask_logits (+ per-board D4 view and inverse map) in one engine call."""
        self._check_input(x)
        return self.engine_for(x.device).forward(self._as_engine_input(x), orient, mask=True,
                                                 inverse_map=inverse_map)

    @torch.no_grad()
    def selfplay_step(self, x: torch.Tensor, *, temperature: float = 1.0, seed: int = 0, offset: int = 0,
                      board_index0: int = 0, orient: torch.Tensor | None = None, inverse_map: bool = False,
                      want_logits: bool = False):
        """One self-play inference step (connect6/train.py:792-795): forward, masked
        log-softmax and one categorical draw per board.  Returns (actions int64 [B],
        logprob fp32 [B], value fp32 [B], masked logits or None)."""
        self._check_input(x)
        return self.engine_for(x.device).forward_step(
            self._as_engine_input(x), temperature=temperature, seed=seed, offset=offset,
            board_index0=board_index0, orient=orient, inverse_map=inverse_map, want_logits=want_logits)


    def forward_from_boards(self, boards: torch.Tensor, current_player: torch.Tensor, stones_left: torch.Tensor,
                            index: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
        """forward(canonical_network_input(boards[index], current_player[index], stones_left[index])) -- what the PPO
        minibatch computes from its buffer (connect6/train.py:1038-1048) -- without materialising the gathered state or
        the planes when the grad-enabled forward runs on the library's kernels (`engine_backward=True`): the first kernel
        reads the int8 state directly.  Otherwise the planes are built and `forward` is called."""
        convs = list(self.convs)
        if (self.engine_backward and boards.is_cuda and torch.is_grad_enabled() and any(p.requires_grad for p in self.parameters())
                and boards.dtype == torch.int8 and len(convs) >= 2):
            from .train_ops import PolicyValueStackFromBoards, supports_layer, supports_stem
            if supports_stem(convs[0], self.board_size) and all(supports_layer(c, self.board_size) for c in convs[1:]) \
                    and (index is None or index.numel() > 0) and boards.shape[0] > 0:
                params = [p for c in convs for p in (c.weight, c.bias)]
                idx = (torch.empty(0, dtype=torch.int64, device=boards.device) if index is None
                       else index.to(device=boards.device, dtype=torch.int64))
                return PolicyValueStackFromBoards.apply(
                    boards, current_player.to(device=boards.device, dtype=torch.int8),
                    stones_left.to(device=boards.device, dtype=torch.int8), idx, *params, self.policy_output.weight,
                    self.policy_output.bias, self.value_output.weight, self.value_output.bias)
        from .selfplay import canonical_network_input
        if index is not None:
            boards, current_player, stones_left = boards[index], current_player[index], stones_left[index]
        return self.forward(canonical_network_input(boards, current_player, stones_left))

    @torch.no_grad()
    def selfplay_step_from_boards(self, boards: torch.Tensor, current_player: torch.Tensor, stones_left: torch.Tensor,
                                  index: torch.Tensor | None = None, **kwargs):
        """The same step fed with the environment's raw int8 state (boards [E,n,n], current_player [E],
        stones_left [E]) and an optional int64 index vector selecting the boards to evaluate: fuses
        canonical_network_input (connect6/vector_env.py:196-218) and the gather of
        connect6/train.py:793 into the first kernel."""
        return self.engine_for(boards.device).forward_step_boards(boards, current_player, stones_left, index, **kwargs)


def build_model(model_cfg: dict[str, Any], board_size: int) -> PolicyValueNet:
    """Build the network from the `model` section of the YAML config (connect6/model.py:114-120):
    bookkeeping keys are dropped, the rest are constructor arguments."""
    cfg = {k: v for k, v in dict(model_cfg).items()
           if k not in ("compile", "compile_mode", "architecture_version")}
    return PolicyValueNet(board_size=board_size, **cfg)


def mask_logits(logits: torch.Tensor, legal_mask: torch.Tensor) -> torch.Tensor:
    """Occupied cells get the dtype's most negative finite value (connect6/model.py:123-125)."""
    fill = torch.finfo(logits.dtype).min
    needs_grad = torch.is_grad_enabled() and logits.requires_grad
    if logits.is_cuda and logits.dtype == torch.float32 and legal_mask.dtype == torch.bool \
            and logits.shape == legal_mask.shape and not needs_grad:
        src = logits.contiguous()
        legal = legal_mask.contiguous()
        out = torch.empty_like(src)
        with torch.cuda.device(src.device):
            L.check(L.load().c6_mask_logits(src.data_ptr(), legal.data_ptr(), src.numel(), float(fill),
                                            out.data_ptr(), torch.cuda.current_stream(src.device).cuda_stream),
                    None, "c6_mask_logits")
        return out
    # other dtypes / broadcast masks / autograd (PPO update path): torch operator
    return logits.masked_fill(~legal_mask, fill)
