"""Drop-ins for the inference helpers of the reference's self-play loop
(`connect6/train.py:195-277`) and for `canonical_network_input`
(`connect6/vector_env.py:196-218`), under the reference's own names.

CUDA tensors go through the engine library's kernels; anything else raises (these are the
GPU operators of the hot path -- there is no CPU implementation in this package).
"""
from __future__ import annotations

import torch

from . import _lib as L

# Random stream of the drop-in samplers when the caller passes no seed / offset / board_index0.
# The reference draws from torch's per-process generator (connect6/train.py:195-213), so runs follow
# torch.manual_seed and every rank of a multi-process job draws its own numbers.  Here the Philox key
# is torch.initial_seed() -- the value torch.manual_seed / seed_everything last set -- unless set_seed()
# overrides it, the offset is a process-wide call counter, and the board index starts at
# rank * 2^40 so that local board i of two ranks never shares a uniform.
_RANK_STRIDE = 1 << 40
_stream_state = {"seed": None, "board_index0": None}
_offset_counter = [0]


def set_seed(seed: int | None, board_index0: int | None = None) -> None:
    """Fix the samplers' Philox key (None: follow torch.initial_seed() again) and, optionally, the
    first board index of this process (None: rank * 2^40).  Resets the call counter."""
    _stream_state["seed"] = None if seed is None else int(seed) & 0xFFFFFFFFFFFFFFFF
    _stream_state["board_index0"] = None if board_index0 is None else int(board_index0)
    _offset_counter[0] = 0


def default_stream() -> tuple[int, int]:
    """(seed, board_index0) the samplers use when the caller passes none."""
    seed = _stream_state["seed"]
    if seed is None:
        seed = int(torch.initial_seed()) & 0xFFFFFFFFFFFFFFFF
    base = _stream_state["board_index0"]
    if base is None:
        import torch.distributed as dist
        rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
        base = rank * _RANK_STRIDE
    return seed, base


def _require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what}: expected a CUDA tensor, got {t.device} (no CPU path in this package)")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _next_offset() -> int:
    _offset_counter[0] += 1
    return _offset_counter[0]


def _sample(logits: torch.Tensor, legal: torch.Tensor, temperature: float, want_logprob: bool,
            seed: int | None, offset: int | None, board_index0: int | None):
    _require_cuda(logits, "_sample_actions")
    d_seed, d_base = default_stream()
    lead = logits.shape[:-1]
    A = logits.shape[-1]
    z = logits.float().reshape(-1, A).contiguous()
    lg = legal.reshape(-1, A).to(device=z.device, dtype=torch.bool).contiguous()
    B = z.shape[0]
    actions = torch.empty((B,), device=z.device, dtype=torch.int64)
    logprob = torch.empty((B,), device=z.device, dtype=torch.float32) if want_logprob else None
    with torch.cuda.device(z.device):
        L.check(L.load().c6_sample_actions(
            z.data_ptr(), lg.data_ptr(), B, A, float(temperature),
            int(d_seed if seed is None else seed), int(_next_offset() if offset is None else offset),
            int(d_base if board_index0 is None else board_index0), actions.data_ptr(), L.ptr(logprob), _stream(z)),
            None, "c6_sample_actions")
    actions = actions.reshape(lead)
    return actions, (logprob.reshape(lead) if want_logprob else None)


def _sample_actions(logits: torch.Tensor, legal: torch.Tensor, temperature: float, *, seed: int | None = None,
                    offset: int | None = None, board_index0: int | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """connect6/train.py:195-203: draw from Categorical(mask(logits.float()) / max(T, 1e-4)) and
    return (actions int64, log-prob of the drawn action fp32).  Randomness comes from the engine's
    own Philox4x32-10 stream keyed (seed, offset, board index), not from torch's generator state.
    Defaults: seed = torch.initial_seed() (so torch.manual_seed selects the stream, see set_seed),
    offset = a process-wide counter that advances once per call, board_index0 = rank * 2^40 (every
    rank of a torch.distributed job draws different numbers)."""
    return _sample(logits, legal, temperature, True, seed, offset, board_index0)


def _sample_actions_only(logits: torch.Tensor, legal: torch.Tensor, temperature: float, *,
                         seed: int | None = None, offset: int | None = None,
                         board_index0: int | None = None) -> torch.Tensor:
    """connect6/train.py:206-213: the same draw without the log-probability."""
    return _sample(logits, legal, temperature, False, seed, offset, board_index0)[0]


def _symmetry_for_phase(phase: int) -> tuple[int, bool]:
    """connect6/train.py:216-219: the 8-step D4 cycle -> (quarter turns, mirrored)."""
    p = int(phase) % 8
    return p % 4, p >= 4


def _phase_of(k: int, flip: bool) -> int:
    return (int(k) % 4) + (4 if flip else 0)


def _transform_boards(boards: torch.Tensor, k: int, flip: bool) -> torch.Tensor:
    """connect6/train.py:222-230 for int8 boards [..., n, n] on the GPU."""
    _require_cuda(boards, "_transform_boards")
    if boards.dtype != torch.int8:
        raise TypeError("_transform_boards expects int8 boards")
    n = boards.shape[-1]
    src = boards.contiguous()
    out = torch.empty_like(src)
    B = src.numel() // (n * n)
    with torch.cuda.device(src.device):
        L.check(L.load().c6_transform_boards(src.data_ptr(), B, n, None, _phase_of(k, flip), out.data_ptr(),
                                             _stream(src)), None, "c6_transform_boards")
    return out


def _map_actions(actions: torch.Tensor, board_size: int, k: int, flip: bool, inverse: int) -> torch.Tensor:
    _require_cuda(actions, "_transform_actions")
    src = actions.to(torch.int64).contiguous()
    out = torch.empty_like(src)
    with torch.cuda.device(src.device):
        L.check(L.load().c6_transform_actions(src.data_ptr(), src.numel(), int(board_size), None,
                                              _phase_of(k, flip), inverse, out.data_ptr(), _stream(src)),
                None, "c6_transform_actions")
    return out


def _transform_actions(actions: torch.Tensor, board_size: int, k: int, flip: bool) -> torch.Tensor:
    """connect6/train.py:233-252: canonical action index -> index in the transformed view."""
    return _map_actions(actions, board_size, k, flip, 0)


def _inverse_transform_actions(actions: torch.Tensor, board_size: int, k: int, flip: bool) -> torch.Tensor:
    """connect6/train.py:255-277: view action index -> canonical index."""
    return _map_actions(actions, board_size, k, flip, 1)


def transform_actions_per_board(actions: torch.Tensor, board_size: int, phase: torch.Tensor,
                                inverse: bool = False) -> torch.Tensor:
    """Per-action D4 phase (uint8 [B]) variant of the two maps above."""
    _require_cuda(actions, "transform_actions_per_board")
    src = actions.to(torch.int64).contiguous()
    ph = phase.to(device=src.device, dtype=torch.uint8).contiguous()
    out = torch.empty_like(src)
    with torch.cuda.device(src.device):
        L.check(L.load().c6_transform_actions(src.data_ptr(), src.numel(), int(board_size), ph.data_ptr(), 0,
                                              1 if inverse else 0, out.data_ptr(), _stream(src)),
                None, "c6_transform_actions")
    return out


def canonical_network_input(boards: torch.Tensor, current_player: torch.Tensor,
                            stones_left: torch.Tensor) -> torch.Tensor:
    """connect6/vector_env.py:196-218: int8 boards [B,n,n] -> fp32 planes [B,3,n,n]
    (mine, opponent, last-stone-of-turn)."""
    _require_cuda(boards, "canonical_network_input")
    if boards.dtype != torch.int8:
        raise TypeError("canonical_network_input expects int8 boards")
    B, n = boards.shape[0], boards.shape[-1]
    b = boards.contiguous()
    p = current_player.to(device=b.device, dtype=torch.int8).contiguous()
    s = stones_left.to(device=b.device, dtype=torch.int8).contiguous()
    out = torch.empty((B, 3, n, n), device=b.device, dtype=torch.float32)
    with torch.cuda.device(b.device):
        L.check(L.load().c6_network_input(b.data_ptr(), p.data_ptr(), s.data_ptr(), B, n, out.data_ptr(),
                                          _stream(b)), None, "c6_network_input")
    return out
