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
(grouped forward), connect6/train.py:195-203 (masked Categorical), connect6/train.py:1047-1119 with
connect6/model.py:104-106 (autograd backward of one backbone layer -> layer_backward; pinned by
tests/golden/layer_backward.npz, recorded from a loss.backward() through the reference's own modules).
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


# ---- environment step (connect6/vector_env.py:106-193) with stock torch ops -----------------------
# Restated over a zero-padded board (no bounds masks needed: the padding never equals a player) with
# one gather for all probe cells; the result is the same integer state.  Works on CPU and CUDA
# tensors: on the GPU it serves as the "stock PyTorch" timing bar for the environment kernels, on the
# CPU as a fast checker for large batches (it is itself checked against the numpy oracle and the
# recorded reference games).
_ENV_DIRECTIONS = ((1, 0), (0, 1), (1, 1), (1, -1))
_probe_cache: dict = {}


def _probe_offsets(n: int, win_length: int, device) -> torch.Tensor:
    """Flat offsets, inside the padded (n + 2*reach)^2 board, of the probe cells around a stone:
    [8 rays, reach] ordered near to far; rays 2d and 2d+1 are the two halves of line direction d."""
    key = (n, win_length, str(device))
    if key not in _probe_cache:
        reach, pitch = win_length - 1, n + 2 * (win_length - 1)
        rays = []
        for dr, dc in _ENV_DIRECTIONS:
            for sgn in (1, -1):
                rays.append([sgn * s * (dr * pitch + dc) for s in range(1, reach + 1)])
        _probe_cache[key] = torch.tensor(rays, dtype=torch.long, device=device).reshape(8, reach)
    return _probe_cache[key]


@torch.no_grad()
def env_step_torch(boards: torch.Tensor, current_player: torch.Tensor, stones_left: torch.Tensor,
                   empty_count: torch.Tensor, move_count: torch.Tensor, actions: torch.Tensor, win_length: int = 6):
    """In-place step of the five state tensors; returns (reward, done, winner, transition_sign,
    game_lengths) with the reference's dtypes."""
    E, n, _ = boards.shape
    reach, pitch = win_length - 1, n + 2 * (win_length - 1)
    env_ids = torch.arange(E, device=boards.device)
    r, c = actions // n, actions % n
    actor = current_player.clone()
    boards[env_ids, r, c] = actor
    empty_count -= 1
    move_count += 1
    if reach > 0:
        padded = torch.nn.functional.pad(boards, (reach, reach, reach, reach)).reshape(E, -1)
        centre = (r + reach) * pitch + (c + reach)
        probes = centre.view(E, 1, 1) + _probe_offsets(n, win_length, boards.device)
        same = padded.gather(1, probes.reshape(E, -1)).reshape(E, 8, reach) == actor.view(E, 1, 1)
        runs = same.to(torch.int16).cumprod(-1).sum(-1)              # contiguous stones along each ray
        won = ((1 + runs[:, 0::2] + runs[:, 1::2]) >= win_length).any(1)
    else:
        won = torch.ones(E, dtype=torch.bool, device=boards.device)
    done = won | (empty_count == 0)
    winner = torch.where(won, actor, torch.zeros_like(actor))
    remaining = stones_left - 1
    stay = ~done & (remaining > 0)
    switch = ~done & ~(remaining > 0)
    stones_left.copy_(torch.where(stay, remaining, torch.where(switch, torch.full_like(remaining, 2), stones_left)))
    current_player.copy_(torch.where(switch, -current_player, current_player))
    sign = stay.to(torch.int8) - switch.to(torch.int8)
    return won.to(torch.float32), done, winner, sign, move_count.clone()


def layer_backward(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, grad_out: torch.Tensor):
    """What autograd computes for one backbone layer y = silu(conv2d(x, W, b, padding=k//2)) inside the
    reference's PPO update (connect6/train.py:1047-1119 differentiating connect6/model.py:104-106):
    (dL/dx, dL/dW, dL/db) from dL/dy, in the dtype of the arguments (use float64 for an oracle)."""
    x = x.detach().clone().requires_grad_(True)
    weight = weight.detach().clone().requires_grad_(True)
    bias = bias.detach().clone().requires_grad_(True)
    y = F.silu(F.conv2d(x, weight, bias, padding=weight.shape[-1] // 2))
    y.backward(grad_out.to(y.dtype))
    return x.grad, weight.grad, bias.grad


def stack_backward(x: torch.Tensor, weights, biases, grad_out: torch.Tensor):
    """What autograd computes for a run of backbone layers y_l = silu(conv2d(y_{l-1}, W_l, b_l, padding=k//2))
    (the loop of connect6/model.py:104-106 differentiated by connect6/train.py:1115-1119):
    (y, dL/dx, [dL/dW_l], [dL/db_l]) from dL/dy, in the dtype of the arguments (use float64 for an oracle)."""
    x = x.detach().clone().requires_grad_(True)
    weights = [w.detach().clone().requires_grad_(True) for w in weights]
    biases = [b.detach().clone().requires_grad_(True) for b in biases]
    y = x
    for w, b in zip(weights, biases):
        y = F.silu(F.conv2d(y, w, b, padding=w.shape[-1] // 2))
    y.backward(grad_out.to(y.dtype))
    return y.detach(), x.grad, [w.grad for w in weights], [b.grad for b in biases]


def ppo_loss(logits: torch.Tensor, legal: torch.Tensor, actions: torch.Tensor, old_logprob: torch.Tensor,
             advantages: torch.Tensor, returns: torch.Tensor, values: torch.Tensor, temperature: float, clip_coef: float,
             value_coef: float, entropy_coef: float) -> dict:
    """The loss of one PPO minibatch as connect6/train.py:1047-1094 computes it from the network outputs, and what
    loss.backward() (connect6/train.py:1115-1119) hands back to them: dict with loss, policy_loss, value_loss, entropy,
    approx_kl, clipfrac (scalars) and dlogits, dvalues.  dtype of `logits` (use float64 for an oracle)."""
    from torch.distributions import Categorical
    logits = logits.detach().clone().requires_grad_(True)
    values = values.detach().clone().requires_grad_(True)
    z = logits.masked_fill(~legal, torch.finfo(logits.dtype).min) / max(temperature, 1e-4)
    dist = Categorical(logits=z)
    new_logprob = dist.log_prob(actions)
    entropy = dist.entropy().mean()
    logratio = new_logprob - old_logprob
    ratio = logratio.exp()
    pg1 = -advantages * ratio
    pg2 = -advantages * torch.clamp(ratio, 1.0 - clip_coef, 1.0 + clip_coef)
    policy_loss = torch.maximum(pg1, pg2).mean()
    value_loss = 0.5 * (values - returns).pow(2).mean()
    loss = policy_loss + value_coef * value_loss - entropy_coef * entropy
    loss.backward()
    with torch.no_grad():
        approx_kl = ((ratio - 1.0) - logratio).mean()
        clipfrac = ((ratio - 1.0).abs() > clip_coef).to(logits.dtype).mean()
    return {"loss": loss.detach(), "policy_loss": policy_loss.detach(), "value_loss": value_loss.detach(),
            "entropy": entropy.detach(), "approx_kl": approx_kl, "clipfrac": clipfrac, "dlogits": logits.grad,
            "dvalues": values.grad}
