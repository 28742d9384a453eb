"""Torch-CPU restatement of the reference forward (TEST INFRASTRUCTURE ONLY).

The reference runs its CNN through torch.nn.Conv2d / torch.nn.functional.conv2d;
on the host that dispatches to PyTorch's own CPU convolution.  This port issues
the same library calls from functional code so that (a) large parity cases
finish in seconds and (b) the benchmark can time "the reference's CPU path" on
the GPU box, where the reference sources are not present.  It is checked against
the numpy oracle and the golden fixtures in tests/test_oracle.py.

Only tests/, the smoke test and the CPU-baseline / reference legs of bench.py
may import this module.

Reference citations: connect6/model.py:96-111 (forward), connect6/history.py:251-303
(grouped forward), connect6/train.py:195-203 (masked Categorical).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def n_layers_of(params: dict) -> int:
    n = 0
    while f"convs.{n}.weight" in params:
        n += 1
    return n


@torch.inference_mode()
def policy_value_forward(x: torch.Tensor, params: dict) -> tuple[torch.Tensor, torch.Tensor]:
    """connect6/model.py:96-111 on CPU tensors, dtype of x (fp32 or fp64)."""
    f = x
    for i in range(n_layers_of(params)):
        w = params[f"convs.{i}.weight"].to(x.dtype)
        b = params[f"convs.{i}.bias"].to(x.dtype)
        f = F.silu(F.conv2d(f, w, b, stride=1, padding=w.shape[-1] // 2))
    logits = F.conv2d(f, params["policy_output.weight"].to(x.dtype), params["policy_output.bias"].to(x.dtype)).flatten(1)
    vmap = F.conv2d(f, params["value_output.weight"].to(x.dtype), params["value_output.bias"].to(x.dtype))
    value = torch.tanh(vmap.mean(dim=(-2, -1))).squeeze(1)
    return logits, value


@torch.inference_mode()
def grouped_policy_value_forward(x: torch.Tensor, params_list: list[dict]):
    """M independent forwards == the grouped convolution of connect6/history.py:251-303."""
    outs = [policy_value_forward(x[m], params_list[m]) for m in range(len(params_list))]
    return torch.stack([o[0] for o in outs]), torch.stack([o[1] for o in outs])


@torch.inference_mode()
def masked_log_softmax(logits: torch.Tensor, legal: torch.Tensor, temperature: float = 1.0) -> torch.Tensor:
    """Normalised logits of Categorical(logits=mask_logits(logits.float(), legal)/max(T,1e-4))."""
    z = logits.float().masked_fill(~legal, torch.finfo(torch.float32).min) / max(float(temperature), 1e-4)
    return z - z.logsumexp(dim=-1, keepdim=True)
