"""Backward of one backbone layer through the C ABI (include/c6_train.h) against PyTorch autograd in fp64.

The reference's PPO update differentiates y = silu(conv2d(x, W, b)) with autograd (connect6/train.py:1047-1119,
connect6/model.py:104-106); the oracle (oracle/torch_port.py:layer_backward) is exactly that, on CPU in float64,
pinned by gradients recorded from a loss.backward() through the reference's own modules
(tests/golden/layer_backward.npz).  The operator computes in bf16
with fp32 accumulation, so the tolerance is stated relative to the spread of each gradient: dX carries one bf16
rounding of dL/d(pre-activation), of the filter and of the result (measured ~5e-3 of the gradient's standard
deviation at worst); dW and db are sums over every position of the batch, where the rounding errors average out.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

import torch_port as TP
from conftest import load_golden

pytestmark = pytest.mark.gpu

DX_TOL = 3e-2     # max |error| / std(dX)
DW_TOL = 2e-2     # max |error| / std(dW)
DB_TOL = 2e-2     # max |error| / max(std(db), |db| scale)


def _oracle(x, w, b, dy):
    return TP.layer_backward(x.double(), w.double(), b.double(), dy.double())


def test_conv_layer_backward_golden(cuda_device):
    """Gradients recorded from loss.backward() through the reference's own network (one backbone layer of a
    7x7 net, 24 -> 40 channels, 6 boards): the operator reproduces them within the bf16 tolerances."""
    from connect6_b200.train_ops import backward_status, conv_layer_backward
    g = load_golden("layer_backward.npz")
    t = lambda k: torch.from_numpy(g[k]).to(cuda_device)
    dx, dw, db = conv_layer_backward(t("x_in"), t("weight"), t("bias"), t("dy"))
    assert backward_status(dx) == 0
    assert np.abs(dx.cpu().numpy() - g["dx"]).max() < DX_TOL * g["dx"].std()
    # only 6 x 49 positions are summed here, so the bf16 rounding of the operands averages out less than in a
    # real batch: twice the large-batch tolerance (measured 0.021 of the gradient's standard deviation)
    assert np.abs(dw.cpu().numpy() - g["dw"]).max() < 2 * DW_TOL * g["dw"].std()
    assert np.abs(db.cpu().numpy() - g["db"]).max() < 2 * DB_TOL * np.abs(g["db"]).max()


def _case(B, cin, cout, n, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.nn.functional.silu(torch.randn(B, cin, n, n, generator=g))            # like a previous layer's output
    w = torch.randn(cout, cin, 3, 3, generator=g) * (2.0 / (9 * cin)) ** 0.5          # kaiming scale
    b = 0.1 * torch.randn(cout, generator=g)
    dy = torch.randn(B, cout, n, n, generator=g) * 1e-3
    return x, w, b, dy


@pytest.mark.parametrize("B,cin,cout,n", [(37, 64, 96, 19), (5, 32, 32, 19), (16, 96, 96, 19), (9, 24, 40, 7), (3, 64, 64, 19)])
def test_conv_layer_backward_against_autograd(cuda_device, B, cin, cout, n):
    from connect6_b200.train_ops import backward_status, conv_layer_backward
    x, w, b, dy = _case(B, cin, cout, n, seed=B + cin)
    rx, rw, rb = _oracle(x, w, b, dy)
    for _ in range(2):                                      # second call reuses the workspace
        dx, dw, db = conv_layer_backward(x.to(cuda_device), w.to(cuda_device), b.to(cuda_device), dy.to(cuda_device))
    assert backward_status(dx) == 0
    ex = (dx.cpu().double() - rx).abs().max().item() / rx.std().item()
    ew = (dw.cpu().double() - rw).abs().max().item() / rw.std().item()
    eb = (db.cpu().double() - rb).abs().max().item() / max(rb.std().item(), rb.abs().max().item())
    assert ex < DX_TOL, f"dX: {ex}"
    assert ew < DW_TOL, f"dW: {ew}"
    assert eb < DB_TOL, f"db: {eb}"
    # without dX (first trainable layer) the other two are unchanged
    none, dw2, db2 = conv_layer_backward(x.to(cuda_device), w.to(cuda_device), b.to(cuda_device), dy.to(cuda_device),
                                         need_dx=False)
    assert none is None and torch.equal(dw2, dw) and torch.equal(db2, db)


def test_conv_layer_backward_is_linear_in_the_output_gradient(cuda_device):
    """Size-independent property at a larger batch: the backward is linear in dy (up to bf16 rounding of dy)."""
    from connect6_b200.train_ops import conv_layer_backward
    x, w, b, dy = _case(512, 64, 96, 19, seed=3)
    xd, wd, bd, dyd = (t.to(cuda_device) for t in (x, w, b, dy))
    dx1, dw1, db1 = conv_layer_backward(xd, wd, bd, dyd)
    dx2, dw2, db2 = conv_layer_backward(xd, wd, bd, 2.0 * dyd)      # exact in bf16: a power of two
    assert torch.equal(dx2, 2.0 * dx1) and torch.allclose(dw2, 2.0 * dw1, rtol=1e-5, atol=0) and torch.allclose(db2, 2.0 * db1, rtol=1e-5)
    zx, zw, zb = conv_layer_backward(xd, wd, bd, torch.zeros_like(dyd))
    assert not zx.any() and not zw.any() and not zb.any()


def test_autograd_function_trains_a_layer(cuda_device):
    from connect6_b200.train_ops import SiluConv3x3
    torch.manual_seed(0)
    conv = torch.nn.Conv2d(64, 96, 3, padding=1).to(cuda_device)
    x = torch.nn.functional.silu(torch.randn(8, 64, 19, 19, device=cuda_device)).requires_grad_(True)
    y = SiluConv3x3.apply(x, conv.weight, conv.bias)
    loss = (y * torch.linspace(-1, 1, 96, device=cuda_device).view(1, 96, 1, 1)).sum() * 1e-3
    loss.backward()
    gx, gw, gb = x.grad.clone(), conv.weight.grad.clone(), conv.bias.grad.clone()
    x.grad = None
    conv.zero_grad()
    y2 = torch.nn.functional.silu(conv(x))
    ((y2 * torch.linspace(-1, 1, 96, device=cuda_device).view(1, 96, 1, 1)).sum() * 1e-3).backward()
    assert (gx - x.grad).abs().max().item() < DX_TOL * x.grad.std().item()
    assert (gw - conv.weight.grad).abs().max().item() < DW_TOL * conv.weight.grad.std().item()
    assert (gb - conv.bias.grad).abs().max().item() < DB_TOL * conv.bias.grad.abs().max().item()


def test_conv_layer_backward_rejects_what_it_does_not_support(cuda_device):
    from connect6_b200.train_ops import conv_layer_backward
    dev = cuda_device
    with pytest.raises(ValueError):     # 5x5 filter
        conv_layer_backward(torch.zeros(2, 8, 19, 19, device=dev), torch.zeros(8, 8, 5, 5, device=dev), None,
                            torch.zeros(2, 8, 19, 19, device=dev))
    with pytest.raises(ValueError):     # too wide
        conv_layer_backward(torch.zeros(2, 192, 19, 19, device=dev), torch.zeros(8, 192, 3, 3, device=dev), None,
                            torch.zeros(2, 8, 19, 19, device=dev))
    with pytest.raises(ValueError):     # shapes of different layers
        conv_layer_backward(torch.zeros(2, 8, 19, 19, device=dev), torch.zeros(8, 16, 3, 3, device=dev), None,
                            torch.zeros(2, 8, 19, 19, device=dev))
    with pytest.raises(RuntimeError):
        conv_layer_backward(torch.zeros(2, 8, 19, 19), torch.zeros(8, 8, 3, 3), None, torch.zeros(2, 8, 19, 19))
    dx, dw, db = conv_layer_backward(torch.zeros(0, 8, 19, 19, device=dev), torch.zeros(8, 8, 3, 3, device=dev), None,
                                     torch.zeros(0, 8, 19, 19, device=dev))
    assert dx.shape == (0, 8, 19, 19) and not dw.any() and not db.any()


STACK_RMS_TOL = 2e-2    # rms error / scale of each gradient, through up to seven bf16 layer backwards
STACK_MAX_TOL = 1e-1    # worst element / scale


def _check_stack(got, ref, name):
    ref = ref.double()
    scale = max(ref.std().item(), ref.abs().max().item() * 0.1) if ref.numel() > 1 else abs(ref.item())
    err = (got.cpu().double() - ref).abs().max().item()
    rms = (got.cpu().double() - ref).pow(2).mean().sqrt().item()
    assert err < STACK_MAX_TOL * scale and rms < STACK_RMS_TOL * scale, f"{name}: max {err}, rms {rms} vs scale {scale}"


@pytest.mark.parametrize("B,n,channels,stem", [(37, 19, (32, 32, 64, 64, 64, 96, 96, 96), 0), (5, 19, (32, 64), 0),
                                               (9, 7, (24, 40, 16), 0), (300, 19, (64, 96, 96), 0),
                                               (37, 19, (3, 32, 32, 64), 23), (6, 9, (3, 16, 24), 5), (130, 19, (3, 64, 32), 23),
                                               (4, 13, (3, 24, 24), 17)])
def test_layer_stack_forward_backward_against_autograd(cuda_device, B, n, channels, stem):
    """c6_backbone_forward / c6_backbone_backward (a whole run of layers, activations and gradients kept in the
    kernels' plane layout between layers; stem > 0: the run starts with the network's stem x stem first layer on the
    3 input planes) against autograd in fp64 (oracle/torch_port.py:stack_backward)."""
    from connect6_b200.train_ops import stack_backward, stack_forward, stack_status
    gen = torch.Generator().manual_seed(B + n)
    if stem:
        x = (torch.rand(B, 3, n, n, generator=gen) < 0.3).float()            # 0/1 planes like the network input
    else:
        x = torch.nn.functional.silu(torch.randn(B, channels[0], n, n, generator=gen))
    ks = [stem if (stem and l == 0) else 3 for l in range(len(channels) - 1)]
    ws = [torch.randn(channels[l + 1], channels[l], ks[l], ks[l], generator=gen) * (2.0 / (ks[l] ** 2 * channels[l])) ** 0.5
          for l in range(len(channels) - 1)]
    bs = [0.1 * torch.randn(channels[l + 1], generator=gen) for l in range(len(channels) - 1)]
    dy = torch.randn(B, channels[-1], n, n, generator=gen) * 1e-3
    ry, rx, rws, rbs = TP.stack_backward(x.double(), [w.double() for w in ws], [b.double() for b in bs], dy.double())
    dev = cuda_device
    for _ in range(2):                                      # the second round reuses the workspace
        y, lease = stack_forward(x.to(dev), [w.to(dev) for w in ws], [b.to(dev) for b in bs])
        dx, dws, dbs = stack_backward(lease, dy.to(dev))
        assert stack_status(lease) == 0
        del lease
    # forward: one bf16 rounding per layer (relative 2^-9 of a value) on top of bf16 weights and inputs
    assert (y.cpu().double() - ry).abs().max().item() < 2.0 ** -7 * ry.abs().max().item() * len(ws) ** 0.5 + 1e-3
    if stem:
        assert dx is None                                   # the network input has no gradient
    else:
        _check_stack(dx, rx, "dx")
    for l in range(len(ws)):
        _check_stack(dws[l], rws[l], f"dw[{l}]")
        _check_stack(dbs[l], rbs[l], f"db[{l}]")
    # without dX the parameter gradients are unchanged
    y2, lease = stack_forward(x.to(dev), [w.to(dev) for w in ws], [b.to(dev) for b in bs])
    none, dws2, dbs2 = stack_backward(lease, dy.to(dev), need_dx=False)
    assert none is None and torch.equal(y2, y)
    assert all(torch.equal(a, b) for a, b in zip(dws2, dws)) and all(torch.equal(a, b) for a, b in zip(dbs2, dbs))


@pytest.mark.parametrize("B,n,channels,stem", [(33, 19, (3, 32, 64, 96), 23), (7, 9, (16, 24), 0), (700, 19, (32, 40), 0)])
def test_heads_on_the_stack_against_autograd(cuda_device, B, n, channels, stem):
    """heads_forward / heads_backward (the two 1x1 heads of connect6/model.py:70-75,108-110 on features that never
    leave the plane layout) chained with the layer stack, against autograd in fp64 on the same expression."""
    from connect6_b200.train_ops import heads_backward, heads_forward, stack_backward, stack_forward, stack_status
    gen = torch.Generator().manual_seed(B)
    x = (torch.rand(B, 3, n, n, generator=gen) < 0.3).float() if stem else torch.nn.functional.silu(torch.randn(B, channels[0], n, n, generator=gen))
    ks = [stem if (stem and l == 0) else 3 for l in range(len(channels) - 1)]
    ws = [torch.randn(channels[l + 1], channels[l], ks[l], ks[l], generator=gen) * (2.0 / (ks[l] ** 2 * channels[l])) ** 0.5
          for l in range(len(channels) - 1)]
    bs = [0.1 * torch.randn(channels[l + 1], generator=gen) for l in range(len(channels) - 1)]
    C_ = channels[-1]
    pw, vw = 0.3 * torch.randn(1, C_, 1, 1, generator=gen), 0.3 * torch.randn(1, C_, 1, 1, generator=gen)
    pb, vb = torch.tensor([0.2]), torch.tensor([-0.1])
    r1, r2 = torch.randn(B, n * n, generator=gen) * 1e-3, torch.randn(B, generator=gen) * 1e-2
    # oracle: the same expression in float64 under autograd
    leaves = [t.double().requires_grad_(True) for t in ws + bs + [pw, pb, vw, vb]]
    ows, obs, (opw, opb, ovw, ovb) = leaves[:len(ws)], leaves[len(ws):2 * len(ws)], leaves[2 * len(ws):]
    f = x.double()
    for w, b in zip(ows, obs):
        f = torch.nn.functional.silu(torch.nn.functional.conv2d(f, w, b, padding=w.shape[-1] // 2))
    rl = torch.nn.functional.conv2d(f, opw, opb).flatten(1)
    rv = torch.tanh(torch.nn.functional.conv2d(f, ovw, ovb).mean(dim=(-2, -1))).squeeze(1)
    ((rl * r1.double()).sum() + (rv * r2.double()).sum()).backward()
    dev = cuda_device
    d = lambda t: t.to(dev)
    for _ in range(2):
        _, lease = stack_forward(d(x), [d(w) for w in ws], [d(b) for b in bs], want_features=False)
        logits, value = heads_forward(lease, d(pw), d(pb), d(vw), d(vb))
        dpw, dpb, dvw, dvb = heads_backward(lease, d(pw), d(vw), d(r1), d(r2), value)
        dx, dws, dbs = stack_backward(lease, None, need_dx=False)
        assert stack_status(lease) == 0
        del lease
    assert (logits.cpu().double() - rl.detach()).abs().max().item() < 2.0 ** -7 * rl.detach().abs().max().item() * (len(ws) + 1) ** 0.5 + 1e-3
    assert (value.cpu().double() - rv.detach()).abs().max().item() < 5e-3
    for got, ref, name in ((dpw, opw.grad, "policy w"), (dpb, opb.grad, "policy b"), (dvw, ovw.grad, "value w"), (dvb, ovb.grad, "value b")):
        _check_stack(got.reshape(ref.shape), ref, name)
    for l in range(len(ws)):
        _check_stack(dws[l], ows[l].grad, f"dw[{l}]")
        _check_stack(dbs[l], obs[l].grad, f"db[{l}]")


def test_layer_stack_rejects_what_it_does_not_support(cuda_device):
    from connect6_b200.train_ops import stack_forward
    dev = cuda_device
    z = lambda *s: torch.zeros(*s, device=dev)
    with pytest.raises(ValueError):     # 5x5 filter that is not a stem on 3 planes
        stack_forward(z(2, 8, 19, 19), [z(8, 8, 5, 5), z(8, 8, 3, 3)], [None, None])
    with pytest.raises(ValueError):     # a stem with nothing behind it
        stack_forward(z(2, 3, 19, 19), [z(8, 3, 5, 5)], [None])
    with pytest.raises(ValueError):     # a wide filter in the middle
        stack_forward(z(2, 3, 19, 19), [z(8, 3, 5, 5), z(8, 8, 5, 5)], [None, None])
    with pytest.raises(ValueError):     # layers that do not chain
        stack_forward(z(2, 8, 19, 19), [z(16, 8, 3, 3), z(8, 8, 3, 3)], [None, None])
    with pytest.raises(ValueError):     # too wide
        stack_forward(z(2, 8, 19, 19), [z(192, 8, 3, 3)], [None])
    with pytest.raises(RuntimeError):   # no CPU path
        stack_forward(torch.zeros(2, 8, 19, 19), [torch.zeros(8, 8, 3, 3)], [None])
    y, lease = stack_forward(z(0, 8, 19, 19), [z(8, 8, 3, 3)], [None])
    assert y.shape == (0, 8, 19, 19) and lease is None


def test_network_gradients_golden(cuda_device):
    """Every parameter gradient of a PPO-style loss.backward() recorded from the reference's own network
    (tests/golden/network_backward.npz: 9x9 board, 5x5 stem, four 3x3 layers, 8 boards), reproduced by
    PolicyValueNet(engine_backward=True): the stem, the four 3x3 layers and both heads run forward and backward on the
    library's kernels (train_ops.PolicyValueStack)."""
    from connect6_b200.model import PolicyValueNet
    g = load_golden("network_backward.npz")
    net = PolicyValueNet(int(g["board_size"]), [int(k) for k in g["kernels"]], [int(c) for c in g["channels"]],
                         engine_backward=True).to(cuda_device).train()
    net.load_state_dict({k[3:]: torch.from_numpy(g[k]) for k in g if k.startswith("w::")})
    logits, value = net(torch.from_numpy(g["x"]).to(cuda_device))
    loss = torch.nn.functional.cross_entropy(logits, torch.from_numpy(g["target"]).to(cuda_device)) + 0.5 * (value - 0.25).pow(2).mean()
    assert abs(float(loss) - float(g["loss"])) < 2e-2 * abs(float(g["loss"]))
    net.zero_grad()
    loss.backward()
    for name, p in net.named_parameters():
        # 8 x 81 positions only: the bf16 roundings average out less than in a real batch (twice the tolerances)
        ref = torch.from_numpy(g["g::" + name]).double()
        scale = max(ref.std().item(), ref.abs().max().item() * 0.1) if ref.numel() > 1 else abs(ref.item())
        # the policy head's bias gradient is a sum of (softmax - one-hot) over the actions: zero but for rounding (5e-8
        # in the recording), so it only has an absolute bound
        scale = max(scale, 1e-5)
        err = (p.grad.cpu().double() - ref).abs().max().item()
        rms = (p.grad.cpu().double() - ref).pow(2).mean().sqrt().item()
        assert err < 2 * STACK_MAX_TOL * scale and rms < 2 * STACK_RMS_TOL * scale, f"{name}: max {err}, rms {rms} vs {scale}"


def test_whole_network_gradients_with_engine_backward(cuda_device):
    """PolicyValueNet(engine_backward=True): a PPO-style loss.backward() whose stem, seven 3x3 layers and heads run
    forward and backward on the library's kernels (train_ops.PolicyValueStack) gives the parameter gradients of plain
    autograd (fp32 on the same GPU).  The gradient passes through up to seven bf16 layer backwards before it reaches the early layers
    (one bf16 rounding of dL/dx per layer), so the bound is on the root-mean-square error (2 % of each gradient's
    scale) and, for the worst of the thousands of elements of a tensor, 10 %."""
    from connect6_b200.boards import generate_planes
    from connect6_b200.model import PolicyValueNet
    torch.manual_seed(3)
    plain = PolicyValueNet(19).to(cuda_device).train()
    ours = PolicyValueNet(19, engine_backward=True).to(cuda_device).train()
    ours.load_state_dict(plain.state_dict())
    with torch.no_grad():                       # default-init heads (std 0.01) would leave the gradients tiny
        for m in (plain, ours):
            m.policy_output.weight.mul_(30.0)
            m.value_output.weight.mul_(30.0)
    x = torch.from_numpy(generate_planes(0, 48)).to(cuda_device)
    target = (torch.arange(48, device=cuda_device) * 37) % 361
    grads = []
    for m in (plain, ours):
        logits, value = m(x)
        assert logits.requires_grad
        loss = torch.nn.functional.cross_entropy(logits, target) + 0.5 * (value - 0.3).pow(2).mean()
        m.zero_grad()
        loss.backward()
        grads.append({k: p.grad.detach().clone() for k, p in m.named_parameters()})
    for name, ref in grads[0].items():
        got = grads[1][name]
        scale = max(ref.std().item(), ref.abs().max().item() * 0.1) if ref.numel() > 1 else abs(ref.item())
        scale = max(scale, 1e-5)    # the policy bias gradient is zero but for rounding (a sum of softmax - one-hot)
        err = (got - ref).abs().max().item()
        rms = (got - ref).pow(2).mean().sqrt().item()
        assert err < 0.1 * scale and rms < 0.02 * scale, f"{name}: max {err}, rms {rms} vs scale {scale}"


def test_ppo_loss_golden_and_oracle(cuda_device):
    """c6_ppo_loss (one kernel: loss components, statistics, gradients at the network outputs) against the values the
    reference's own statements gave (tests/golden/ppo_loss.npz) and, on a larger random minibatch, the float64 oracle."""
    from connect6_b200.train_ops import ppo_loss
    dev = cuda_device
    g = load_golden("ppo_loss.npz")
    for case in range(int(g["ncases"])):
        p = f"c{case}_"
        t = lambda k: torch.from_numpy(g[p + k]).to(dev)
        coefs = [float(v) for v in g[p + "coefs"]]
        logits, values = t("logits").requires_grad_(True), t("values").requires_grad_(True)
        loss, stats = ppo_loss(logits, values, t("legal"), t("actions"), t("old_logprob"), t("advantages"), t("returns"), *coefs)
        loss.backward()
        assert np.abs(stats.cpu().numpy() - g[p + "stats"]).max() < 2e-5
        assert abs(float(loss) - g[p + "stats"][0]) < 2e-5
        assert np.abs(logits.grad.cpu().numpy() - g[p + "dlogits"]).max() < 1e-6 + 1e-4 * np.abs(g[p + "dlogits"]).max()
        assert np.abs(values.grad.cpu().numpy() - g[p + "dvalues"]).max() < 1e-7
    # larger case against the oracle, with one board whose ratio is far outside the range
    gen = torch.Generator().manual_seed(9)
    B, A = 1000, 361
    logits = torch.randn(B, A, generator=gen) * 2.0
    legal = torch.rand(B, A, generator=gen) < 0.6
    actions = torch.stack([torch.nonzero(legal[b]).flatten()[0] if legal[b].any() else torch.tensor(0) for b in range(B)])
    lp = torch.log_softmax(logits.masked_fill(~legal, torch.finfo(torch.float32).min), -1).gather(1, actions[:, None]).squeeze(1)
    old = lp + 0.3 * torch.randn(B, generator=gen)
    old[11] -= 3.0
    adv, ret, values = torch.randn(B, generator=gen), torch.tanh(torch.randn(B, generator=gen)), torch.tanh(torch.randn(B, generator=gen))
    r = TP.ppo_loss(logits.double(), legal, actions, old.double(), adv.double(), ret.double(), values.double(), 1.0, 0.2, 0.5, 0.01)
    lg, vv = logits.to(dev).requires_grad_(True), values.to(dev).requires_grad_(True)
    loss, stats = ppo_loss(lg, vv, legal.to(dev), actions.to(dev), old.to(dev), adv.to(dev), ret.to(dev), 1.0, 0.2, 0.5, 0.01)
    (2.0 * loss).backward()                                 # the gradients scale with what flows into the loss
    want = np.array([float(r[k]) for k in ("loss", "policy_loss", "value_loss", "entropy", "approx_kl", "clipfrac")])
    assert np.abs(stats.cpu().numpy() - want).max() < 5e-5
    assert (lg.grad.cpu().double() - 2.0 * r["dlogits"]).abs().max().item() < 1e-7 + 1e-4 * r["dlogits"].abs().max().item()
    assert (vv.grad.cpu().double() - 2.0 * r["dvalues"]).abs().max().item() < 1e-8
    # A board without any legal action (terminal: never part of a real minibatch) gets the uniform distribution and no
    # gradient; the reference's own arithmetic degenerates there (its fill value absorbs the normaliser), so only
    # finiteness is checked.
    legal2 = legal.clone()
    legal2[7] = False
    lg2 = logits.to(dev).requires_grad_(True)
    loss2, stats2 = ppo_loss(lg2, vv.detach(), legal2.to(dev), actions.to(dev), old.to(dev), adv.to(dev), ret.to(dev), 1.0, 0.2, 0.5, 0.01)
    loss2.backward()
    assert torch.isfinite(stats2).all() and not lg2.grad[7].any() and torch.isfinite(lg2.grad).all()
    with pytest.raises(RuntimeError):
        ppo_loss(logits, values, legal, actions, old, adv, ret)
    with pytest.raises(ValueError):
        ppo_loss(lg, vv[:5], legal.to(dev), actions.to(dev), old.to(dev), adv.to(dev), ret.to(dev))


def test_ppo_updates_track_the_autograd_path(cuda_device):
    """Five optimizer steps of a PPO minibatch loop (forward under bf16 autocast, ppo_loss, backward, gradient clipping,
    AdamW) with the network and the loss on the library's kernels against the same loop through the PyTorch modules and
    the reference's loss statements: the losses stay together, and the parameters end up close."""
    from torch.distributions import Categorical
    from connect6_b200.boards import generate_planes
    from connect6_b200.model import PolicyValueNet
    from connect6_b200.train_ops import ppo_loss
    dev = cuda_device
    torch.manual_seed(5)
    plain = PolicyValueNet(19).to(dev).train()
    ours = PolicyValueNet(19, engine_backward=True).to(dev).train()
    ours.load_state_dict(plain.state_dict())
    B = 64
    x = torch.from_numpy(generate_planes(0, B)).to(dev)
    gen = torch.Generator(device=dev).manual_seed(1)
    legal = (x[:, 0] + x[:, 1]).reshape(B, -1).eq(0)
    actions = torch.multinomial(legal.float(), 1, generator=gen).squeeze(1)
    old = -torch.log(legal.sum(1).float()) + 0.1 * torch.randn(B, device=dev, generator=gen)
    adv, ret = torch.randn(B, device=dev, generator=gen), torch.tanh(torch.randn(B, device=dev, generator=gen))
    losses = {}
    for name, m in (("plain", plain), ("ours", ours)):
        opt = torch.optim.AdamW(m.parameters(), lr=3e-4)
        losses[name] = []
        for _ in range(5):
            with torch.autocast("cuda", dtype=torch.bfloat16):
                logits, value = m(x)
                if m is ours:
                    loss, stats = ppo_loss(logits, value, legal, actions, old, adv, ret, 1.0, 0.2, 0.5, 0.01)
                else:
                    z = logits.masked_fill(~legal, torch.finfo(logits.dtype).min)
                    dist = Categorical(logits=z.float())
                    ratio = (dist.log_prob(actions) - old).exp()
                    pg = torch.maximum(-adv * ratio, -adv * torch.clamp(ratio, 0.8, 1.2)).mean()
                    loss = pg + 0.5 * 0.5 * (value.float() - ret).pow(2).mean() - 0.01 * dist.entropy().mean()
            opt.zero_grad(set_to_none=True)
            loss.backward()
            torch.nn.utils.clip_grad_norm_(m.parameters(), 0.5)
            opt.step()
            losses[name].append(float(loss))
    assert all(abs(a - b) < 5e-3 + 0.02 * abs(a) for a, b in zip(losses["plain"], losses["ours"])), losses
    for (k, p), (_, q) in zip(plain.named_parameters(), ours.named_parameters()):
        # AdamW's first steps move every parameter by about lr per step whatever the gradient's size: the two runs may
        # differ by a few lr where a gradient component is noise-sized, never by more
        assert (p - q).abs().max().item() <= 5 * 2 * 3e-4 + 1e-6, k


def test_training_step_under_a_cuda_graph(cuda_device):
    """Forward + ppo_loss + backward of PolicyValueNet(engine_backward=True) captured once in a CUDA graph and replayed:
    the library's training entry points only enqueue work on the stream they are given (no allocation, no
    synchronisation), so the whole step is capturable; the replayed gradients equal the eager ones bit for bit (every
    reduction runs in a fixed order)."""
    from connect6_b200.boards import generate_planes
    from connect6_b200.model import PolicyValueNet
    from connect6_b200.train_ops import ppo_loss
    dev = cuda_device
    torch.manual_seed(2)
    m = PolicyValueNet(19, engine_backward=True).to(dev).train()
    B = 32
    x = torch.from_numpy(generate_planes(0, B)).to(dev)
    gen = torch.Generator(device=dev).manual_seed(1)
    legal = (x[:, 0] + x[:, 1]).reshape(B, -1).eq(0)
    actions = torch.multinomial(legal.float(), 1, generator=gen).squeeze(1)
    old = -torch.log(legal.sum(1).float())
    adv, ret = torch.randn(B, device=dev, generator=gen), torch.zeros(B, device=dev)

    def step():
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits, value = m(x)
            loss, _ = ppo_loss(logits, value, legal, actions, old, adv, ret)
        loss.backward()
        return loss

    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        for _ in range(2):
            m.zero_grad(set_to_none=True)
            eager_loss = step()
    torch.cuda.current_stream(dev).wait_stream(side)
    torch.cuda.synchronize(dev)
    eager = [p.grad.detach().clone() for p in m.parameters()]
    m.zero_grad(set_to_none=True)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        graph_loss = step()
    for _ in range(2):
        for p in m.parameters():
            p.grad.zero_()          # the captured backward accumulates into these very tensors
        graph.replay()
    torch.cuda.synchronize(dev)
    assert float(graph_loss) == float(eager_loss)
    for p, ref in zip(m.parameters(), eager):
        assert torch.equal(p.grad, ref)


def test_clip_adamw_matches_torch(cuda_device):
    """train_ops.ClipAdamW (c6_clip_adamw_step: global-norm clipping + AdamW in two launches) against
    nn.utils.clip_grad_norm_ + torch.optim.AdamW with the reference's hyper-parameters (connect6/train.py:476-481,
    configs/train.yaml:55-62) over four steps, two of them with gradients large enough to be clipped; then the state
    moves into a torch.optim.AdamW and both continue in step."""
    from connect6_b200.model import PolicyValueNet
    from connect6_b200.train_ops import ClipAdamW
    dev = cuda_device
    torch.manual_seed(4)
    a = PolicyValueNet(19).to(dev)
    b = PolicyValueNet(19).to(dev)
    b.load_state_dict(a.state_dict())
    kw = dict(lr=2.5e-4, weight_decay=1e-4, eps=1e-5)
    ref = torch.optim.AdamW(a.parameters(), **kw)
    ours = ClipAdamW(b.parameters(), max_grad_norm=2.0, **kw)
    gen = torch.Generator(device=dev).manual_seed(1)
    for it in range(4):
        scale = 10.0 if it % 2 else 1e-2               # clipped / not clipped
        for pa, pb in zip(a.parameters(), b.parameters()):
            g = scale * torch.randn(pa.shape, device=dev, generator=gen)
            pa.grad, pb.grad = g.clone(), g.clone()
        want_norm = torch.nn.utils.clip_grad_norm_(a.parameters(), 2.0, error_if_nonfinite=True)
        ref.step()
        got_norm = ours.step()
        assert abs(float(got_norm) - float(want_norm)) < 1e-4 * float(want_norm)
        for pa, pb in zip(a.parameters(), b.parameters()):
            assert torch.allclose(pb.grad, pa.grad, rtol=1e-5, atol=1e-9)            # clipped in place like clip_grad_norm_
            assert (pa - pb).abs().max().item() < 2e-7 + 1e-6 * pa.abs().max().item()
    # the state has AdamW's layout: a torch optimizer continues from it
    cont = torch.optim.AdamW(b.parameters(), **kw)
    sd = ours.state_dict()
    for g_ in sd["param_groups"]:
        g_.pop("max_grad_norm")
    cont.load_state_dict(sd)
    for pa, pb in zip(a.parameters(), b.parameters()):
        g = 1e-2 * torch.randn(pa.shape, device=dev, generator=gen)
        pa.grad, pb.grad = g.clone(), g.clone()
    ref.step()
    cont.step()
    for pa, pb in zip(a.parameters(), b.parameters()):
        assert (pa - pb).abs().max().item() < 4e-7 + 1e-6 * pa.abs().max().item()
    # a non-finite gradient: the norm says so, nothing moves
    before = [p.detach().clone() for p in b.parameters()]
    next(iter(b.parameters())).grad[0, 0, 0, 0] = float("inf")
    n = ours.step()
    assert not torch.isfinite(n)
    assert all(torch.equal(p, q) for p, q in zip(b.parameters(), before))
    cpu_p = torch.nn.Parameter(torch.zeros(3))
    cpu_p.grad = torch.zeros(3)
    with pytest.raises(RuntimeError):       # no CPU path
        ClipAdamW([cpu_p], lr=1e-3).step()


def test_training_forward_from_the_buffer_state(cuda_device):
    """PolicyValueNet.forward_from_boards with engine_backward=True (the stem kernel reads the int8 state and the
    minibatch index directly) gives the logits, values and parameter gradients of the same network fed with
    canonical_network_input(boards[index], ...) -- bit for bit: the planes are 0/1 either way."""
    from connect6_b200.model import PolicyValueNet
    from connect6_b200.selfplay import canonical_network_input
    dev = cuda_device
    torch.manual_seed(8)
    m = PolicyValueNet(19, engine_backward=True).to(dev).train()
    gen = torch.Generator().manual_seed(3)
    E = 50
    boards = torch.randint(-1, 2, (E, 19, 19), generator=gen).to(torch.int8).to(dev)
    player = (torch.randint(0, 2, (E,), generator=gen) * 2 - 1).to(torch.int8).to(dev)
    stones = torch.randint(1, 3, (E,), generator=gen).to(torch.int8).to(dev)
    index = torch.randperm(E, generator=gen)[:21].to(dev)
    results = []
    for from_state in (True, False):
        m.zero_grad(set_to_none=True)
        if from_state:
            logits, value = m.forward_from_boards(boards, player, stones, index)
        else:
            logits, value = m(canonical_network_input(boards[index], player[index], stones[index]))
        (logits.square().mean() + value.sum()).backward()
        results.append((logits.detach().clone(), value.detach().clone(), [p.grad.detach().clone() for p in m.parameters()]))
    assert torch.equal(results[0][0], results[1][0]) and torch.equal(results[0][1], results[1][1])
    assert all(torch.equal(a, b) for a, b in zip(results[0][2], results[1][2]))
    # no index: every environment; no grad: the inference engine
    logits, _ = m.forward_from_boards(boards, player, stones)
    assert logits.shape == (E, 361) and logits.requires_grad
    with torch.no_grad():
        lg, _ = m.forward_from_boards(boards, player, stones, index)
    assert lg.shape == (21, 361) and not lg.requires_grad


def test_ppo_minibatch_update_helper(cuda_device):
    """train_ops.ppo_minibatch_update (the body of the reference's minibatch loop as one call) run on a buffer-shaped
    state: three updates with PolicyValueNet(engine_backward=True) + ClipAdamW against the same helper driving the plain
    model with torch.optim.AdamW -- statistics and gradient norms stay together."""
    from connect6_b200.model import PolicyValueNet
    from connect6_b200.train_ops import ClipAdamW, ppo_minibatch_update
    dev = cuda_device
    torch.manual_seed(6)
    plain = PolicyValueNet(19).to(dev).train()
    ours = PolicyValueNet(19, engine_backward=True).to(dev).train()
    ours.load_state_dict(plain.state_dict())
    gen = torch.Generator().manual_seed(2)
    N = 96
    boards = torch.randint(-1, 2, (N, 19, 19), generator=gen).to(torch.int8).to(dev)
    players = (torch.randint(0, 2, (N,), generator=gen) * 2 - 1).to(torch.int8).to(dev)
    stones = torch.randint(1, 3, (N,), generator=gen).to(torch.int8).to(dev)
    legal = boards.reshape(N, -1).eq(0)
    actions = torch.multinomial(legal.float().cpu(), 1, generator=gen).squeeze(1).to(dev)
    old = (-torch.log(legal.sum(1).float())).to(dev)
    adv, ret = torch.randn(N, generator=gen).to(dev), torch.tanh(torch.randn(N, generator=gen)).to(dev)
    kw = dict(lr=2.5e-4, weight_decay=1e-4, eps=1e-5)
    o_plain = torch.optim.AdamW(plain.parameters(), **kw)
    o_plain.param_groups[0]["max_grad_norm"] = 2.0
    o_ours = ClipAdamW(ours.parameters(), max_grad_norm=2.0, **kw)
    for it in range(3):
        idx = torch.randperm(N, generator=gen)[:32].to(dev)
        s1, n1 = ppo_minibatch_update(plain, o_plain, boards, players, stones, actions, old, adv, ret, idx)
        s2, n2 = ppo_minibatch_update(ours, o_ours, boards, players, stones, actions, old, adv, ret, idx)
        assert (s1 - s2).abs().max().item() < 5e-3 + 0.02 * s1.abs().max().item(), (it, s1, s2)
        assert abs(float(n1) - float(n2)) < 0.05 * float(n1) + 1e-4


def test_network_backward_properties_at_4096_boards(cuda_device):
    """Size-independent properties of the whole-network backward at a batch the fp64 oracle cannot afford: the parameter
    gradients of a batch are the sums of the gradients of its halves (fp32 sums in another order: 1e-3 of each tensor's
    scale, the bf16 operands being the same numbers either way), they are linear in the output gradients (a factor 2
    is exact in bf16 up to the fp32 roundings of the sums), and a zero output gradient gives zero everywhere."""
    from connect6_b200.boards import generate_planes
    from connect6_b200.train_ops import heads_backward, heads_forward, stack_backward, stack_forward, stack_status
    dev = cuda_device
    torch.manual_seed(12)
    from connect6_b200.model import PolicyValueNet
    net = PolicyValueNet(19).to(dev)
    ws = [c.weight.detach() for c in net.convs]
    bs = [c.bias.detach() + 0.05 for c in net.convs]
    pw, pb, vw, vb = (net.policy_output.weight.detach() * 30, net.policy_output.bias.detach(), net.value_output.weight.detach() * 30,
                      net.value_output.bias.detach())
    B = 4096
    x = torch.from_numpy(generate_planes(0, B)).to(dev)
    gen = torch.Generator(device=dev).manual_seed(1)
    dl = torch.randn(B, 361, device=dev, generator=gen) * 1e-3
    dv = torch.randn(B, device=dev, generator=gen) * 1e-2

    def grads(sl, scale=1.0):
        _, lease = stack_forward(x[sl], ws, bs, want_features=False)
        _, value = heads_forward(lease, pw, pb, vw, vb)
        hg = heads_backward(lease, pw, vw, scale * dl[sl], scale * dv[sl], value)
        _, dws, dbs = stack_backward(lease, None, need_dx=False)
        assert stack_status(lease) == 0
        return [g.clone() for g in list(hg) + dws + dbs]

    whole = grads(slice(0, B))
    first, second = grads(slice(0, B // 2)), grads(slice(B // 2, B))
    for w, a, b in zip(whole, first, second):
        scale = max(w.abs().max().item(), 1e-6)
        assert (w - (a + b)).abs().max().item() < 1e-3 * scale
    doubled = grads(slice(0, B), 2.0)
    for w, d in zip(whole, doubled):
        scale = max(w.abs().max().item(), 1e-6)
        assert (d - 2.0 * w).abs().max().item() < 1e-4 * scale
    zero = grads(slice(0, B), 0.0)
    assert all(not z.any() for z in zero)


def test_whole_update_under_a_cuda_graph_with_clip_adamw(cuda_device):
    """ClipAdamW(capturable=True) keeps its update count on the device: forward + ppo_loss + backward + clipping + AdamW
    captured once and replayed three times moves the parameters exactly like three eager updates of a twin model (bias
    corrections included: they change with every replay)."""
    from connect6_b200.boards import generate_planes
    from connect6_b200.model import PolicyValueNet
    from connect6_b200.train_ops import ClipAdamW, ppo_loss
    dev = cuda_device
    torch.manual_seed(9)
    a = PolicyValueNet(19, engine_backward=True).to(dev).train()
    b = PolicyValueNet(19, engine_backward=True).to(dev).train()
    b.load_state_dict(a.state_dict())
    B = 32
    x = torch.from_numpy(generate_planes(0, B)).to(dev)
    gen = torch.Generator(device=dev).manual_seed(1)
    legal = (x[:, 0] + x[:, 1]).reshape(B, -1).eq(0)
    actions = torch.multinomial(legal.float(), 1, generator=gen).squeeze(1)
    old = -torch.log(legal.sum(1).float())
    adv, ret = torch.randn(B, device=dev, generator=gen), torch.zeros(B, device=dev)
    kw = dict(lr=2.5e-4, weight_decay=1e-4, eps=1e-5, max_grad_norm=2.0)
    # both with the device-side update count: the same arithmetic eagerly and replayed (the host-side count rounds its
    # bias corrections in double precision, and training amplifies even that difference within a few updates)
    oa, ob = ClipAdamW(a.parameters(), capturable=True, **kw), ClipAdamW(b.parameters(), capturable=True, **kw)

    def update(m, opt):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits, value = m(x)
            loss, _ = ppo_loss(logits, value, legal, actions, old, adv, ret)
        loss.backward()
        return opt.step()

    for _ in range(4):                        # eager: four updates
        oa.zero_grad(set_to_none=True)
        update(a, oa)
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        ob.zero_grad(set_to_none=True)
        update(b, ob)                         # the first update runs eagerly on the side stream (allocates the state)
    torch.cuda.current_stream(dev).wait_stream(side)
    torch.cuda.synchronize(dev)
    for p in b.parameters():
        p.grad.zero_()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        update(b, ob)                         # captured, not executed
    for _ in range(3):
        for p in b.parameters():
            p.grad.zero_()
        graph.replay()
    torch.cuda.synchronize(dev)
    assert float(ob.state[next(iter(b.parameters()))]["step"]) == 4.0
    for pa, pb in zip(a.parameters(), b.parameters()):
        assert torch.equal(pa, pb)
