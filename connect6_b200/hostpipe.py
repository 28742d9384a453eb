"""Host-buffer front end for self-play inference: pinned host planes in, pinned host results out.

The reference's rollout loop builds its network input on the device; a caller that keeps boards on
the host pays one host->device copy per step.  `HostStepPipeline` hides that copy behind the
previous step's kernels: inputs are double-buffered on the device and uploaded on a side stream,
results come back through pinned buffers.  Every step still performs its own upload and its own
download; only their overlap with compute changes.
"""
from __future__ import annotations

import torch

from .model import PolicyValueNet


class HostStepPipeline:
    """Two-deep pipeline around `PolicyValueNet.selfplay_step` for host-resident inputs.

    submit(x_host)  -- enqueue the upload of one batch of fp32/bf16 planes [B,3,n,n] (pinned memory
                       for a truly asynchronous copy); at most two batches may be in flight.
    step(**kw)      -- run the self-play step on the oldest submitted batch, download
                       (actions int64, logprob fp32, value fp32) into pinned buffers, wait for them
                       and return them (views that stay valid until the next step()).
    """

    def __init__(self, model: PolicyValueNet, batch: int, device: torch.device | str, dtype=torch.float32):
        self.model = model
        self.device = torch.device(device)
        n = model.board_size
        self._x = [torch.empty((batch, 3, n, n), device=self.device, dtype=dtype) for _ in range(2)]
        self._uploaded = [torch.cuda.Event() for _ in range(2)]
        self._consumed = [torch.cuda.Event() for _ in range(2)]
        self._copy_stream = torch.cuda.Stream(self.device)
        self._head = 0      # next buffer to fill
        self._tail = 0      # next buffer to consume
        self._inflight = 0
        self._sizes = [0, 0]
        self.actions = torch.empty(batch, dtype=torch.int64).pin_memory()
        self.logprob = torch.empty(batch, dtype=torch.float32).pin_memory()
        self.value = torch.empty(batch, dtype=torch.float32).pin_memory()
        for ev in self._consumed:
            ev.record(torch.cuda.current_stream(self.device))

    def submit(self, x_host: torch.Tensor) -> None:
        if self._inflight >= 2:
            raise RuntimeError("two batches are already in flight: call step() first")
        k = self._head
        b = x_host.shape[0]
        with torch.cuda.stream(self._copy_stream):
            self._copy_stream.wait_event(self._consumed[k])      # the kernels that read this buffer are done
            self._x[k][:b].copy_(x_host, non_blocking=True)
            self._uploaded[k].record(self._copy_stream)
        self._sizes[k] = b
        self._head ^= 1
        self._inflight += 1

    def step(self, **kwargs):
        if self._inflight == 0:
            raise RuntimeError("nothing submitted")
        k = self._tail
        b = self._sizes[k]
        stream = torch.cuda.current_stream(self.device)
        stream.wait_event(self._uploaded[k])
        action, logprob, value, _ = self.model.selfplay_step(self._x[k][:b], **kwargs)
        self._consumed[k].record(stream)
        self.actions[:b].copy_(action, non_blocking=True)
        self.logprob[:b].copy_(logprob, non_blocking=True)
        self.value[:b].copy_(value, non_blocking=True)
        self._tail ^= 1
        self._inflight -= 1
        stream.synchronize()                                       # the caller reads the results now
        return self.actions[:b], self.logprob[:b], self.value[:b]
