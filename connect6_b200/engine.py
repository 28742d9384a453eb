"""Thin object wrapper over the C ABI: one `Engine` owns one C6Engine handle.

PyTorch is used only for device memory (inputs, outputs) and for the current stream.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import torch

from . import _lib as L

_PREC = {"bf16": L.C6_PREC_BF16, "fp32": L.C6_PREC_FP32, "f16": L.C6_PREC_F16}


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _x_dtype(x: torch.Tensor) -> int:
    if x.dtype == torch.float32:
        return L.C6_X_F32
    if x.dtype == torch.bfloat16:
        return L.C6_X_BF16
    raise TypeError(f"network input must be float32 or bfloat16, got {x.dtype}")


class Engine:
    """One architecture, `groups` weight sets, one arithmetic mode, one CUDA device."""

    def __init__(self, device: torch.device | str, board_size: int, kernels: Sequence[int],
                 channels: Sequence[int], groups: int = 1, precision: str = "bf16", max_chunk: int = 0):
        device = torch.device(device)
        if device.type != "cuda":
            raise RuntimeError("the Connect6 engine runs on CUDA devices only (there is no CPU path)")
        if not torch.cuda.is_available():
            raise RuntimeError("CUDA is not available; the Connect6 engine has no CPU path")
        if precision not in _PREC:
            raise ValueError(f"precision must be one of {sorted(_PREC)}, got {precision!r}")
        if len(kernels) != len(channels) or not kernels or len(kernels) > L.C6_MAX_LAYERS:
            raise ValueError("kernels and channels must have the same length in 1..16")
        self.device = torch.device("cuda", device.index if device.index is not None else torch.cuda.current_device())
        self.board_size = int(board_size)
        self.kernels = tuple(int(k) for k in kernels)
        self.channels = tuple(int(c) for c in channels)
        self.groups = int(groups)
        self.precision = precision
        self.n_actions = self.board_size * self.board_size
        self._lib = L.load()
        desc = L.C6Desc()
        desc.device = self.device.index
        desc.board_size = self.board_size
        desc.n_layers = len(self.kernels)
        for i, (k, c) in enumerate(zip(self.kernels, self.channels)):
            desc.kernels[i] = k
            desc.channels[i] = c
        desc.groups = self.groups
        desc.precision = _PREC[precision]
        desc.max_chunk = int(max_chunk)
        handle = C.c_void_p()
        L.check(self._lib.c6_create(C.byref(desc), C.byref(handle)), None, "c6_create")
        self._h = handle

    # -- lifetime -------------------------------------------------------------------------------
    def close(self) -> None:
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.c6_destroy(h)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- weights --------------------------------------------------------------------------------
    def _dev_f32(self, t: torch.Tensor | None) -> torch.Tensor | None:
        if t is None:
            return None
        return t.detach().to(device=self.device, dtype=torch.float32).contiguous()

    def set_layer(self, group: int, layer_or_head: int, weight: torch.Tensor, bias: torch.Tensor | None) -> None:
        w = self._dev_f32(weight)
        b = self._dev_f32(bias)
        with torch.cuda.device(self.device):
            L.check(self._lib.c6_set_weights(self._h, group, layer_or_head, L.ptr(w), L.ptr(b),
                                             _stream_ptr(self.device)), self._h, "c6_set_weights")
        # w and b may be temporaries: the packing kernels were enqueued on the current stream, and
        # the caching allocator only reuses their memory for later work on that same stream.

    def load_state_dict(self, state: dict, group: int = 0, need_value: bool = True) -> None:
        """Pack one reference state_dict (connect6/model.py layout) into weight set `group`."""
        for i in range(len(self.kernels)):
            try:
                w = state[f"convs.{i}.weight"]
            except KeyError as exc:
                raise KeyError(f"missing parameter convs.{i}.weight") from exc
            expect = (self.channels[i], 3 if i == 0 else self.channels[i - 1], self.kernels[i], self.kernels[i])
            if tuple(w.shape) != expect:
                raise ValueError(f"convs.{i}.weight has shape {tuple(w.shape)}, expected {expect}")
            self.set_layer(group, i, w, state.get(f"convs.{i}.bias"))
        if "policy_output.weight" not in state:
            raise KeyError("missing parameter policy_output.weight")
        self.set_layer(group, L.C6_HEAD_POLICY, state["policy_output.weight"], state.get("policy_output.bias"))
        if "value_output.weight" in state:
            self.set_layer(group, L.C6_HEAD_VALUE, state["value_output.weight"], state.get("value_output.bias"))
        elif need_value:
            raise KeyError("missing parameter value_output.weight")
        else:
            self.set_layer(group, L.C6_HEAD_VALUE, torch.zeros_like(state["policy_output.weight"]), None)

    def reserve(self, boards: int) -> None:
        L.check(self._lib.c6_reserve(self._h, int(boards)), self._h, "c6_reserve")

    # -- checks ---------------------------------------------------------------------------------
    def _check_x(self, x: torch.Tensor, lead: int) -> torch.Tensor:
        """x must be [lead dims..., 3, n, n] on the engine's device (the kernels index it unchecked)."""
        if x.device != self.device:
            raise RuntimeError(f"input lives on {x.device}, engine on {self.device} (no CPU path)")
        tail = (3, self.board_size, self.board_size)
        if x.ndim != lead + 3 or tuple(x.shape[lead:]) != tail:
            raise ValueError(f"network input must have {lead} leading dimension(s) followed by "
                             f"[{tail[0]}, {tail[1]}, {tail[2]}], got {tuple(x.shape)}")
        return x if x.is_contiguous() else x.contiguous()

    def _check_orient(self, orient: torch.Tensor | None, boards: int) -> torch.Tensor | None:
        if orient is None:
            return None
        if orient.dtype != torch.uint8 or orient.numel() != boards or orient.device != self.device:
            raise ValueError("orient must be a uint8 tensor with one D4 phase per board on the engine's device")
        return orient.contiguous()

    # -- forward --------------------------------------------------------------------------------
    def forward(self, x: torch.Tensor, orient: torch.Tensor | None = None, *, mask: bool = False,
                inverse_map: bool = False, want_value: bool = True):
        x = self._check_x(x, 1)
        B = x.shape[0]
        orient = self._check_orient(orient, B)
        logits = torch.empty((B, self.n_actions), device=self.device, dtype=torch.float32)
        value = torch.empty((B,), device=self.device, dtype=torch.float32) if want_value else None
        flags = (L.C6_FLAG_MASK_LOGITS if mask else 0) | (L.C6_FLAG_INVERSE_MAP if inverse_map else 0)
        with torch.cuda.device(self.device):
            L.check(self._lib.c6_forward(self._h, L.ptr(x), _x_dtype(x), B, L.ptr(orient), L.ptr(logits),
                                         L.ptr(value), flags, _stream_ptr(self.device)), self._h, "c6_forward")
        return logits, value

    def forward_step(self, x: torch.Tensor, *, temperature: float = 1.0, seed: int = 0, offset: int = 0,
                     board_index0: int = 0, orient: torch.Tensor | None = None, inverse_map: bool = False,
                     want_logits: bool = False, want_logprob: bool = True, want_value: bool = True):
        x = self._check_x(x, 1)
        B = x.shape[0]
        orient = self._check_orient(orient, B)
        action = torch.empty((B,), device=self.device, dtype=torch.int64)
        logprob = torch.empty((B,), device=self.device, dtype=torch.float32) if want_logprob else None
        value = torch.empty((B,), device=self.device, dtype=torch.float32) if want_value else None
        logits = torch.empty((B, self.n_actions), device=self.device, dtype=torch.float32) if want_logits else None
        flags = L.C6_FLAG_INVERSE_MAP if inverse_map else 0
        with torch.cuda.device(self.device):
            L.check(self._lib.c6_forward_step(self._h, L.ptr(x), _x_dtype(x), B, L.ptr(orient), flags,
                                              float(temperature), int(seed), int(offset), int(board_index0),
                                              L.ptr(action), L.ptr(logprob), L.ptr(value), L.ptr(logits),
                                              _stream_ptr(self.device)), self._h, "c6_forward_step")
        return action, logprob, value, logits

    def forward_step_boards(self, boards: torch.Tensor, current_player: torch.Tensor, stones_left: torch.Tensor,
                            index: torch.Tensor | None = None, *, temperature: float = 1.0, seed: int = 0,
                            offset: int = 0, board_index0: int = 0, orient: torch.Tensor | None = None,
                            inverse_map: bool = False, want_logits: bool = False, want_logprob: bool = True,
                            want_value: bool = True):
        """Self-play step straight from the environment's int8 state (no fp32 planes)."""
        for t, name in ((boards, "boards"), (current_player, "current_player"), (stones_left, "stones_left")):
            if t.dtype != torch.int8 or t.device != self.device:
                raise ValueError(f"{name} must be an int8 tensor on {self.device}")
        n = self.board_size
        if boards.ndim != 3 or tuple(boards.shape[1:]) != (n, n):
            raise ValueError(f"boards must have shape [envs, {n}, {n}], got {tuple(boards.shape)}")
        envs = int(boards.shape[0])
        if tuple(current_player.shape) != (envs,) or tuple(stones_left.shape) != (envs,):
            raise ValueError(f"current_player and stones_left must have shape [{envs}], got "
                             f"{tuple(current_player.shape)} and {tuple(stones_left.shape)}")
        boards, current_player, stones_left = boards.contiguous(), current_player.contiguous(), stones_left.contiguous()
        if index is not None:
            if index.dtype != torch.int64 or index.device != self.device or index.ndim != 1:
                raise ValueError("index must be a one-dimensional int64 tensor on the engine's device")
            index = index.contiguous()
        # the values of `index` stay on the device: the kernel skips entries outside [0, envs), evaluates
        # an empty board for them and raises C6_STATUS_BAD_INDEX in the status word
        B = int(index.numel()) if index is not None else envs
        orient = self._check_orient(orient, B)
        action = torch.empty((B,), device=self.device, dtype=torch.int64)
        logprob = torch.empty((B,), device=self.device, dtype=torch.float32) if want_logprob else None
        value = torch.empty((B,), device=self.device, dtype=torch.float32) if want_value else None
        logits = torch.empty((B, self.n_actions), device=self.device, dtype=torch.float32) if want_logits else None
        flags = L.C6_FLAG_INVERSE_MAP if inverse_map else 0
        with torch.cuda.device(self.device):
            L.check(self._lib.c6_forward_step_boards(self._h, L.ptr(boards), L.ptr(current_player), L.ptr(stones_left),
                                                     envs, L.ptr(index), B, L.ptr(orient), flags, float(temperature), int(seed),
                                                     int(offset), int(board_index0), L.ptr(action), L.ptr(logprob),
                                                     L.ptr(value), L.ptr(logits), _stream_ptr(self.device)),
                    self._h, "c6_forward_step_boards")
        return action, logprob, value, logits

    def forward_grouped(self, x: torch.Tensor, *, want_value: bool = False, mask: bool = False):
        x = self._check_x(x, 2)
        G, T = x.shape[0], x.shape[1]
        if G != self.groups:
            raise ValueError(f"grouped input has {G} groups, engine has {self.groups}")
        logits = torch.empty((G, T, self.n_actions), device=self.device, dtype=torch.float32)
        value = torch.empty((G, T), device=self.device, dtype=torch.float32) if want_value else None
        flags = L.C6_FLAG_MASK_LOGITS if mask else 0
        with torch.cuda.device(self.device):
            L.check(self._lib.c6_forward_grouped(self._h, L.ptr(x), _x_dtype(x), T, L.ptr(logits), L.ptr(value),
                                                 flags, _stream_ptr(self.device)), self._h, "c6_forward_grouped")
        return logits, value

    def layer_output(self, x: torch.Tensor, layer: int, orient: torch.Tensor | None = None) -> torch.Tensor:
        """Test aid: fp32 activation [boards, channels[layer], n, n] after backbone layer `layer`."""
        x = self._check_x(x, x.ndim - 3)
        lead = x.shape[:-3]
        boards = 1
        for s in lead:
            boards *= int(s)
        T = boards // self.groups
        out = torch.empty((boards, self.channels[layer], self.board_size, self.board_size), device=self.device,
                          dtype=torch.float32)
        orient = self._check_orient(orient, boards)
        with torch.cuda.device(self.device):
            L.check(self._lib.c6_debug_layer_output(self._h, L.ptr(x), _x_dtype(x), T, L.ptr(orient), int(layer),
                                                    L.ptr(out), _stream_ptr(self.device)), self._h,
                    "c6_debug_layer_output")
        return out

    # -- per-kernel timing ------------------------------------------------------------------
    def profile(self, on: bool | int) -> None:
        """0/False off, 1/True per-launch events, 2 events plus in-kernel pipeline wait counters."""
        L.check(self._lib.c6_profile_enable(self._h, int(on)), self._h, "c6_profile_enable")

    def profile_read(self) -> dict[str, tuple[float, int]]:
        """{kernel kind: (total ms, launches)} since the last read; waits for the recorded events."""
        ms = (C.c_float * L.C6_KIND_COUNT)()
        cnt = (C.c_int64 * L.C6_KIND_COUNT)()
        L.check(self._lib.c6_profile_read(self._h, ms, cnt, L.C6_KIND_COUNT), self._h, "c6_profile_read")
        names = {L.C6_KIND_PACK: "pack_input", L.C6_KIND_STEM: "stem", L.C6_KIND_FINISH: "finish",
                 L.C6_KIND_OTHER: "head_maps"}
        out = {}
        for k in range(L.C6_KIND_COUNT):
            if cnt[k]:
                out[names.get(k, f"conv{k - L.C6_KIND_CONV0}")] = (float(ms[k]), int(cnt[k]))
        return out

    def wait_cycles(self, reset: bool = True) -> dict[str, int]:
        """Pipeline wait counters of CTA 0 of the conv kernel (accumulated while profiling is on)."""
        buf = (C.c_int64 * 8)()
        L.check(self._lib.c6_debug_wait_cycles(self._h, buf, 1 if reset else 0), self._h, "c6_debug_wait_cycles")
        return dict(zip(("producer_wait_empty", "mma_wait_full", "mma_wait_acc", "epilogue_wait_acc", "mma_issue", "mma_loop_total", "epilogue_tmem_fetch", "epilogue_math"), map(int, buf)))

    def cta_times(self, n_ctas: int = 148) -> list[tuple[int, int]]:
        """(entry, exit, MMA loop begin, MMA loop end) in ns for each CTA of the last profiled conv launch."""
        buf = (C.c_int64 * (4 * n_ctas))()
        L.check(self._lib.c6_debug_cta_times(self._h, buf, n_ctas), self._h, "c6_debug_cta_times")
        return [tuple(int(buf[4 * i + j]) for j in range(4)) for i in range(n_ctas)]

    # -- introspection --------------------------------------------------------------------------
    def status(self) -> int:
        """Device status word; synchronises the engine's device first. Raises if non-zero."""
        torch.cuda.synchronize(self.device)
        st = C.c_int(0)
        L.check(self._lib.c6_status(self._h, C.byref(st)), self._h, "c6_status")
        return st.value

    def clear_status(self) -> None:
        L.check(self._lib.c6_clear_status(self._h), self._h, "c6_clear_status")

    def expire_wait_selftest(self) -> None:
        """Enqueue the bounded-wait self-test kernel (its wait runs out by design)."""
        with torch.cuda.device(self.device):
            L.check(self._lib.c6_debug_expire_wait(self._h, _stream_ptr(self.device)), self._h, "c6_debug_expire_wait")

    @property
    def launch_count(self) -> int:
        return int(self._lib.c6_launch_count(self._h))

    @property
    def device_bytes(self) -> int:
        return int(self._lib.c6_device_bytes(self._h))
