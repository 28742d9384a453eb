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


@pytest.mark.parametrize("B,n,channels", [(37, 19, (32, 32, 64, 64, 64, 96, 96, 96)), (5, 19, (32, 64)), (9, 7, (24, 40, 16)),
                                          (300, 19, (64, 96, 96))])
def test_layer_stack_forward_backward_against_autograd(cuda_device, B, n, channels):
    """c6_backbone_forward / c6_backbone_backward (a whole run of 3x3 layers, activations and gradients kept in the
    kernels' plane layout between layers) against autograd in fp64 (oracle/torch_port.py:stack_backward)."""
    from connect6_b200.train_ops import stack_backward, stack_forward, stack_status
    gen = torch.Generator().manual_seed(B + n)
    x = torch.nn.functional.silu(torch.randn(B, channels[0], n, n, generator=gen))
    ws = [torch.randn(channels[l + 1], channels[l], 3, 3, generator=gen) * (2.0 / (9 * channels[l])) ** 0.5 for l in range(len(channels) - 1)]
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
    _check_stack(dx, rx, "dx")
    for l in range(len(ws)):
        _check_stack(dws[l], rws[l], f"dw[{l}]")
        _check_stack(dbs[l], rbs[l], f"db[{l}]")
    # without dX the parameter gradients are unchanged
    y2, lease = stack_forward(x.to(dev), [w.to(dev) for w in ws], [b.to(dev) for b in bs])
    none, dws2, dbs2 = stack_backward(lease, dy.to(dev), need_dx=False)
    assert none is None and torch.equal(y2, y)
    assert all(torch.equal(a, b) for a, b in zip(dws2, dws)) and all(torch.equal(a, b) for a, b in zip(dbs2, dbs))


def test_layer_stack_rejects_what_it_does_not_support(cuda_device):
    from connect6_b200.train_ops import stack_forward
    dev = cuda_device
    z = lambda *s: torch.zeros(*s, device=dev)
    with pytest.raises(ValueError):     # 5x5 filter
        stack_forward(z(2, 8, 19, 19), [z(8, 8, 5, 5)], [None])
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
    PolicyValueNet(engine_backward=True): the four 3x3 layers run forward and backward as one library operator, the
    stem and heads on autograd."""
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
    """PolicyValueNet(engine_backward=True): a PPO-style loss.backward() whose seven 3x3 layers run forward and
    backward as one library operator (train_ops.SiluConvStack) gives the parameter gradients of plain autograd (fp32
    on the same GPU); the stem and the heads stay on autograd.  The gradient passes through up to seven bf16 layer backwards before it reaches the early layers
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
