"""Small, self-ending workload for profilers: `python -m connect6_b200.profile_case [boards] [steps]`.

Runs `steps` bf16 self-play inference steps of the default network on `boards` generated boards
(default 2048: the widest activations exceed L2 while the process holds well under 1 GB on the
device), prints a checksum and the device status word.
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
    for i in range(steps):
        actions, logprob, value, _ = model.selfplay_step(x, seed=1, offset=i)
    torch.cuda.synchronize()
    print("ok", int(actions.sum()), float(value.sum()), model.engine_for(dev).status())


if __name__ == "__main__":
    main()
