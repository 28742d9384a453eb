"""Generate the golden fixtures in this directory from the UNMODIFIED reference.

Run where the reference checkout is importable:
    python tests/golden/make_golden.py [/path/to/reference]
It imports `connect6.*` from that path (or from $C6_REFERENCE), runs the
reference's own functions on seeded inputs and stores inputs, weights and outputs as .npz.
The tests only read the .npz files; they never need the reference.
"""
from __future__ import annotations

import hashlib
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
if len(sys.argv) < 2 and "C6_REFERENCE" not in os.environ:
    raise SystemExit("usage: python " + sys.argv[0] + " /path/to/the/reference/checkout   (or set C6_REFERENCE)")
REF = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ["C6_REFERENCE"])
sys.path.insert(0, str(REF))
sys.path.insert(1, str(REPO))

from connect6.history import HistoricalCheckpoint, HistoricalPolicyEnsemble  # noqa: E402
from connect6.model import PolicyValueNet, build_model, mask_logits  # noqa: E402
from connect6.train import (  # noqa: E402
    _inverse_transform_actions, _sample_actions, _symmetry_for_phase, _transform_actions, _transform_boards)
from connect6.vector_env import canonical_network_input  # noqa: E402

from connect6_b200.boards import generate_planes  # noqa: E402


def state_np(model) -> dict:
    return {k: v.detach().cpu().numpy().copy() for k, v in model.state_dict().items()}


def state_hash(state: dict) -> str:
    h = hashlib.sha256()
    for k in sorted(state):
        h.update(k.encode())
        h.update(np.ascontiguousarray(state[k], dtype=np.float32).tobytes())
    return h.hexdigest()


def layer_backward_fixture() -> None:
    """One PPO-style backward through the reference's own modules (connect6/train.py:1047-1119): the
    reference network in train mode, a loss on logits and values, loss.backward(); a hook on backbone layer
    2 records what autograd hands that layer (its input, the gradient at its output) and what it produces
    (gradients of its input, weight and bias)."""
    torch.manual_seed(11)
    net = PolicyValueNet(board_size=7, kernels=[5, 3, 3, 3], channels=[16, 24, 40, 16]).train()
    with torch.no_grad():
        for p in net.parameters():
            if p.ndim == 1:
                p.uniform_(-0.3, 0.3)
    x = torch.from_numpy(generate_planes(0, 6, board_size=7, max_stones=30))
    layer = net.convs[2]
    grabbed = {}

    def fwd_hook(mod, inp, out):
        grabbed["x_in"] = inp[0].detach().clone()
        inp[0].register_hook(lambda g: grabbed.__setitem__("dx", g.detach().clone()))

    h1 = layer.register_forward_hook(fwd_hook)
    # the SiLU module acts in place (connect6/model.py:67), so the gradient at the layer's OUTPUT is the gradient
    # of the activation's result: hook the activation call that follows convs[2]
    feats = x
    acts = []
    for i, conv in enumerate(net.convs):
        feats = net.activation(conv(feats))
        if i == 2:
            feats.register_hook(lambda g: grabbed.__setitem__("dy", g.detach().clone()))
        acts.append(feats)
    logits = net.policy_output(feats).flatten(1)
    value = net.value_tanh(net.value_output(feats).mean(dim=(-2, -1))).squeeze(1)
    ref_logits, ref_value = net(x)                       # the reference's own forward gives the same numbers
    assert torch.allclose(ref_logits, logits) and torch.allclose(ref_value, value)
    target = torch.arange(6) * 7 % 49
    loss = torch.nn.functional.cross_entropy(logits, target) + 0.5 * (value - 0.25).pow(2).mean()
    net.zero_grad()
    loss.backward()
    h1.remove()
    np.savez_compressed(HERE / "layer_backward.npz", x_in=grabbed["x_in"].numpy(), dy=grabbed["dy"].numpy(),
                        dx=grabbed["dx"].numpy(), weight=layer.weight.detach().numpy(), bias=layer.bias.detach().numpy(),
                        dw=layer.weight.grad.numpy(), db=layer.bias.grad.numpy(), torch_version=torch.__version__)
    print("layer_backward: x_in", tuple(grabbed["x_in"].shape), "dy", tuple(grabbed["dy"].shape),
          "|dw| max", float(layer.weight.grad.abs().max()))


def network_backward_fixture() -> None:
    """Parameter gradients of one PPO-style loss.backward() through the reference's own network (a 9x9 net with a
    5x5 stem and four 3x3 layers, 8 boards): every parameter's gradient, the weights and the inputs."""
    torch.manual_seed(23)
    kernels, channels = [5, 3, 3, 3, 3], [16, 24, 40, 32, 24]
    net = PolicyValueNet(board_size=9, kernels=kernels, channels=channels).train()
    with torch.no_grad():
        for p in net.parameters():
            if p.ndim == 1:
                p.uniform_(-0.3, 0.3)
        net.policy_output.weight.mul_(30.0)      # default-init heads (std 0.01) would leave the gradients tiny
        net.value_output.weight.mul_(30.0)
    x = torch.from_numpy(generate_planes(0, 8, board_size=9, max_stones=50))
    logits, value = net(x)
    target = torch.arange(8) * 11 % 81
    loss = torch.nn.functional.cross_entropy(logits, target) + 0.5 * (value - 0.25).pow(2).mean()
    net.zero_grad()
    loss.backward()
    np.savez_compressed(HERE / "network_backward.npz", x=x.numpy(), target=target.numpy(), loss=float(loss),
                        kernels=np.array(kernels), channels=np.array(channels), board_size=9,
                        torch_version=torch.__version__,
                        **{"w::" + k: v for k, v in state_np(net).items()},
                        **{"g::" + k: p.grad.numpy() for k, p in net.named_parameters()})
    print("network_backward: loss", float(loss), "|g| max per tensor",
          [round(float(p.grad.abs().max()), 5) for p in net.parameters()][:6])


def reference_ppo_loss_code():
    """Code objects compiled from the reference's own statements inside train() (connect6/train.py): the body of the
    autocast block of the PPO minibatch after the model call (masked logits ... loss) and the two statistics of the
    no_grad block behind it.  Nothing of the reference's text is stored: the statements are found by their shape."""
    import ast
    tree = ast.parse((REF / "connect6" / "train.py").read_text())
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "train")
    loss_with = stats_with = None
    for node in ast.walk(fn):
        if isinstance(node, ast.With) and node.body and isinstance(node.body[0], ast.Assign):
            first = ast.unparse(node.body[0])
            if first.startswith("new_logits, new_values = model("):
                loss_with = node
            elif first.startswith("approx_kl_tensor ="):
                stats_with = node
    assert loss_with is not None and stats_with is not None
    loss_nodes = loss_with.body[1:]
    stats_nodes = [n for n in stats_with.body if isinstance(n, ast.Assign) and ast.unparse(n.targets[0]) in ("approx_kl_tensor", "clipfrac_tensor")]
    assert ast.unparse(loss_nodes[-1].targets[0]) == "loss" and len(stats_nodes) == 2
    print(f"ppo loss statements: lines {loss_nodes[0].lineno}-{loss_nodes[-1].end_lineno} and {stats_nodes[0].lineno}-"
          f"{stats_nodes[-1].end_lineno} of connect6/train.py")

    def code(nodes, tag):
        mod = ast.Module(body=list(nodes), type_ignores=[])
        return compile(ast.fix_missing_locations(mod), f"<reference train.py: {tag}>", "exec")

    return code(loss_nodes, "ppo loss"), code(stats_nodes, "ppo statistics")


def ppo_loss_fixture() -> None:
    """The reference's own PPO-loss statements run on random network outputs (two cases: temperature 1 and 0.7), with
    loss.backward() to the logits and values."""
    import types
    import connect6.train as RT
    loss_code, stats_code = reference_ppo_loss_code()
    out = {}
    for case, (B, A, temperature, clip_coef, value_coef, entropy_coef, seed) in enumerate(
            [(48, 361, 1.0, 0.2, 0.5, 0.01, 5), (31, 81, 0.7, 0.1, 1.0, 0.02, 6)]):
        g = torch.Generator().manual_seed(seed)
        logits = (torch.randn(B, A, generator=g) * 1.5).requires_grad_(True)
        values = torch.tanh(torch.randn(B, generator=g)).requires_grad_(True)
        legal = torch.rand(B, A, generator=g) < 0.7
        actions = torch.stack([torch.nonzero(legal[b]).flatten()[int(torch.randint(int(legal[b].sum()), (1,), generator=g))] for b in range(B)])
        with torch.no_grad():
            lp = torch.log_softmax(logits.masked_fill(~legal, torch.finfo(torch.float32).min) / temperature, -1)
            old = lp.gather(1, actions[:, None]).squeeze(1) + 0.3 * torch.randn(B, generator=g)   # ratios on both sides of the clip range
        adv, ret = torch.randn(B, generator=g), torch.tanh(torch.randn(B, generator=g))
        ns = {"torch": torch, "Categorical": RT.Categorical, "mask_logits": RT.mask_logits, "new_logits": logits, "new_values": values,
              "mb_legal": legal, "mb_actions": actions, "temperature": temperature, "buffer": types.SimpleNamespace(logprobs=old),
              "idx": torch.arange(B), "local_idx": torch.arange(B), "advantages": adv, "returns": ret, "clip_coef": clip_coef,
              "value_coef": value_coef, "entropy_coef": entropy_coef}
        exec(loss_code, ns)
        ns["loss"].backward()
        with torch.no_grad():
            exec(stats_code, ns)
        p = f"c{case}_"
        out.update({p + "logits": logits.detach().numpy(), p + "values": values.detach().numpy(), p + "legal": legal.numpy(),
                    p + "actions": actions.numpy(), p + "old_logprob": old.numpy(), p + "advantages": adv.numpy(), p + "returns": ret.numpy(),
                    p + "coefs": np.array([temperature, clip_coef, value_coef, entropy_coef], dtype=np.float64),
                    p + "stats": np.array([float(ns[k]) for k in ("loss", "policy_loss", "value_loss", "entropy", "approx_kl_tensor", "clipfrac_tensor")]),
                    p + "dlogits": logits.grad.numpy(), p + "dvalues": values.grad.numpy()})
        print(f"ppo_loss case {case}: loss {float(ns['loss']):.6f}, clipfrac {float(ns['clipfrac_tensor']):.3f}")
    np.savez_compressed(HERE / "ppo_loss.npz", ncases=2, torch_version=torch.__version__, **out)


def main() -> None:
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    layer_backward_fixture()
    network_backward_fixture()
    ppo_loss_fixture()

    # 1. small net with an even-wider-than-board stem: weights stored, random real-valued input
    torch.manual_seed(7)
    small = PolicyValueNet(board_size=7, kernels=[9, 3, 3], channels=[8, 8, 16]).eval()
    with torch.no_grad():
        for p in small.parameters():  # non-zero biases so that bias handling is pinned too
            if p.ndim == 1:
                p.uniform_(-0.2, 0.2)
        small.policy_output.weight.mul_(30.0)
        small.value_output.weight.mul_(30.0)
    xs = torch.randn(5, 3, 7, 7)
    with torch.inference_mode():
        ls, vs = small(xs)
    np.savez_compressed(HERE / "small_net.npz", x=xs.numpy(), logits=ls.numpy(), value=vs.numpy(),
                        kernels=np.array([9, 3, 3]), channels=np.array([8, 8, 16]), board_size=7,
                        **{"w::" + k: v for k, v in state_np(small).items()})

    # 2. default v4 net, torch seed 42 (configs/train.yaml:8), generated boards 0..5
    torch.manual_seed(42)
    net = PolicyValueNet(board_size=19).eval()
    st = state_np(net)
    xd = torch.from_numpy(generate_planes(0, 6))
    with torch.inference_mode():
        ld, vd = net(xd)
        feats = xd
        layer_stats = []
        for conv in net.convs:
            feats = torch.nn.functional.silu(conv(feats))
            layer_stats.append([float(feats.mean()), float(feats.std()), float(feats.abs().max())])
    np.savez_compressed(HERE / "default_net_seed42.npz", logits=ld.numpy(), value=vd.numpy(),
                        weights_sha256=state_hash(st), layer_stats=np.array(layer_stats),
                        first_board_indices=np.arange(6), torch_version=torch.__version__,
                        first_weights=st["convs.0.weight"][:2, :, :2, :2],
                        policy_weight=st["policy_output.weight"].reshape(-1))

    # 3. D4 tables for n = 19 and n = 7, all 8 phases, straight from the reference helpers
    d4 = {}
    for n in (7, 19):
        a = torch.arange(n * n)
        board = torch.arange(n * n, dtype=torch.int16).reshape(1, n, n)
        fwd, inv, views = [], [], []
        for phase in range(8):
            k, flip = _symmetry_for_phase(phase)
            fwd.append(_transform_actions(a, n, k, flip).numpy())
            inv.append(_inverse_transform_actions(a, n, k, flip).numpy())
            views.append(_transform_boards(board, k, flip).reshape(-1).numpy())
        d4[f"fwd{n}"] = np.stack(fwd).astype(np.int32)
        d4[f"inv{n}"] = np.stack(inv).astype(np.int32)
        d4[f"view{n}"] = np.stack(views).astype(np.int32)
    d4["phases"] = np.array([list(map(int, _symmetry_for_phase(p))) for p in range(10)])
    np.savez_compressed(HERE / "d4_tables.npz", **d4)

    # 4. grouped ensemble on the reference test's own configuration
    #    (tests/test_training_features.py:120-151), three models
    torch.manual_seed(123)
    cfg = {"architecture_version": 4, "kernels": [3, 3, 3], "channels": [8, 8, 16], "compile": False,
           "compile_mode": "default"}
    game = {"board_size": 5, "win_length": 3}
    models = [build_model(cfg, 5) for _ in range(3)]
    cps = [HistoricalCheckpoint(path=Path(f"model_update_{i + 1:08d}.pt"), update=i + 1,
                                model_state=m.state_dict(), model_config=cfg, game_config=game)
           for i, m in enumerate(models)]
    ens = HistoricalPolicyEnsemble(cps, torch.device("cpu"))
    xg = torch.randn(3, 4, 3, 5, 5)
    with torch.inference_mode():
        lg = ens.forward_grouped(xg)
        vg = torch.stack([m.eval()(xg[i])[1] for i, m in enumerate(models)])
    blob = {"x": xg.numpy(), "logits": lg.numpy(), "value": vg.numpy(), "kernels": np.array([3, 3, 3]),
            "channels": np.array([8, 8, 16]), "board_size": 5}
    for i, m in enumerate(models):
        blob.update({f"w{i}::" + k: v for k, v in state_np(m).items()})
    np.savez_compressed(HERE / "grouped_small.npz", **blob)

    # 5. masking and the masked categorical's log-probabilities
    torch.manual_seed(5)
    lo = torch.randn(6, 361) * 2.0
    legal = torch.rand(6, 361) > 0.4
    legal[4] = False
    legal[4, 17] = True      # a single legal move
    legal[5] = False         # no legal move at all: torch yields a uniform distribution
    masked = mask_logits(lo, legal)
    masked_bf16 = mask_logits(lo.bfloat16(), legal).float()
    out = {"logits": lo.numpy(), "legal": legal.numpy(), "masked": masked.numpy(), "masked_bf16": masked_bf16.numpy()}
    for T in (1.0, 0.5, 2.0):
        # with T < 1 the fill overflows to -inf and torch rejects the all-occupied row (NaN), so
        # that row is pinned for T >= 1 only
        rows = slice(0, 5) if T < 1.0 else slice(0, 6)
        z = mask_logits(lo.float(), legal)[rows] / max(T, 1e-4)
        dist = torch.distributions.Categorical(logits=z)
        out[f"logp_T{T}"] = dist.logits.numpy()
    torch.manual_seed(11)
    acts, lps = _sample_actions(lo[:4], legal[:4], 1.0)
    out["sampled_actions"] = acts.numpy()
    out["sampled_logprob"] = lps.numpy()
    np.savez_compressed(HERE / "masking.npz", **out)

    # 6. network planes from raw boards
    torch.manual_seed(3)
    boards = torch.randint(-1, 2, (5, 19, 19), dtype=torch.int8)
    player = torch.tensor([1, -1, 1, -1, 1], dtype=torch.int8)
    stones_left = torch.tensor([1, 2, 2, 1, 1], dtype=torch.int8)
    planes = canonical_network_input(boards, player, stones_left)
    np.savez_compressed(HERE / "network_input.npz", boards=boards.numpy(), player=player.numpy(),
                        stones_left=stones_left.numpy(), planes=planes.numpy())
    print("fixtures written to", HERE)
    for f in sorted(HERE.glob("*.npz")):
        print(f"  {f.name}: {f.stat().st_size} bytes")


if __name__ == "__main__":
    main()
