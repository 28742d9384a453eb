"""Small, self-ending workload for profilers: `python -m connect6_b200.profile_case [boards] [steps]`.

Runs `steps` bf16 self-play inference steps of the default network on `boards` generated boards
(default 2048: the widest activations exceed L2 while the process holds well under 1 GB on the
device), prints a checksum and the device status word.  With more than one step it also prints the
mean step time between CUDA events (after the first step, which includes workspace allocation).
"""
from __future__ import annotations

import sys

import torch

from .boards import generate_planes
from .model import PolicyValueNet


def main() -> None:
    boards = int(sys.argv[1]) if len(sys.argv) > 1 else 2048
    steps = int(sys.argv[2]) if len(sys.argv) > 2 else 1
    dev = torch.device("cuda", 0)
    torch.manual_seed(42)
    model = PolicyValueNet(19).to(dev).eval()
    x = torch.from_numpy(generate_planes(0, boards)).to(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(steps):
        if i == 1:
            e0.record()
        actions, logprob, value, _ = model.selfplay_step(x, seed=1, offset=i)
    e1.record()
    torch.cuda.synchronize()
    print("ok", int(actions.sum()), float(value.sum()), model.engine_for(dev).status())
    if steps > 1:
        us = e0.elapsed_time(e1) * 1e3 / (steps - 1)
        print(f"boards {boards}: {us:.1f} us per step, {boards / us:.3f} M boards/s")


if __name__ == "__main__":
    main()
