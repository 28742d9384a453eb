"""Training-side operators on the engine library's own kernels (include/c6_train.h).

The reference differentiates its network with PyTorch autograd inside the PPO minibatch update
(connect6/train.py:1032-1147).  `conv_layer_backward` does the backward of ONE backbone layer
y = silu(conv2d(x, W, b)) (connect6/model.py:104-106) on tcgen05 tensor cores: dX, dW and db from x, W, b
and dL/dy.  `SiluConv3x3` wraps it as a torch.autograd.Function whose forward is PyTorch's own (the
parameters stay ordinary nn.Parameters), so a layer can be switched over without touching the optimizer.
CUDA only: there is no CPU implementation in this package.
"""
from __future__ import annotations

import torch

from . import _lib as L

_workspaces: dict[tuple, torch.Tensor] = {}


def _workspace(device: torch.device, n: int, k: int, cin: int, cout: int, B: int) -> torch.Tensor:
    """Zero-filled scratch for one shape, kept and reused: the operator maintains the zero padding it
    relies on, so the buffer is cleared only once."""
    key = (device.index, n, k, cin, cout, B)
    ws = _workspaces.get(key)
    if ws is None:
        need = int(L.load().c6_conv_layer_backward_workspace_bytes(n, k, cin, cout, B))
        if need == 0:
            raise ValueError(f"conv_layer_backward supports k = 3, board size <= 32, cin and cout <= 128; got n={n}, "
                             f"k={k}, cin={cin}, cout={cout}")
        if len(_workspaces) >= 8:
            _workspaces.clear()
        ws = torch.zeros((need + 7) // 8, dtype=torch.int64, device=device)
        _workspaces[key] = ws
    return ws


def conv_layer_backward(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, grad_out: torch.Tensor,
                        need_dx: bool = True):
    """(dx or None, dw, db) for y = silu(conv2d(x, weight, bias, padding=k//2)) given grad_out = dL/dy.
    x [B, cin, n, n], weight [cout, cin, 3, 3], grad_out [B, cout, n, n]; fp32 CUDA tensors in, fp32 out
    (bf16 operands and fp32 accumulation inside)."""
    if not x.is_cuda:
        raise RuntimeError(f"conv_layer_backward: expected CUDA tensors, got {x.device} (no CPU path in this package)")
    if x.ndim != 4 or weight.ndim != 4 or grad_out.ndim != 4 or x.shape[2] != x.shape[3]:
        raise ValueError("conv_layer_backward: x [B,cin,n,n], weight [cout,cin,k,k], grad_out [B,cout,n,n]")
    B, cin, n, _ = x.shape
    cout, cin_w, k, k2 = weight.shape
    if cin_w != cin or k != k2 or tuple(grad_out.shape) != (B, cout, n, n) or (bias is not None and tuple(bias.shape) != (cout,)):
        raise ValueError("conv_layer_backward: shapes of x, weight, bias and grad_out do not belong to one layer")
    dev = x.device
    f32 = lambda t: None if t is None else t.detach().to(device=dev, dtype=torch.float32).contiguous()
    x, weight, bias, grad_out = f32(x), f32(weight), f32(bias), f32(grad_out)
    dx = torch.empty_like(x) if need_dx else None
    dw = torch.empty_like(weight)
    db = torch.empty(cout, device=dev, dtype=torch.float32)
    ws = _workspace(dev, n, k, cin, cout, B) if B else torch.zeros(32, dtype=torch.int64, device=dev)
    with torch.cuda.device(dev):
        rc = L.load().c6_conv_layer_backward(dev.index, n, k, cin, cout, B, x.data_ptr(), weight.data_ptr(), L.ptr(bias),
                                             grad_out.data_ptr(), L.ptr(dx), dw.data_ptr(), db.data_ptr(), ws.data_ptr(),
                                             ws.numel() * 8, torch.cuda.current_stream(dev).cuda_stream)
    if rc != L.C6_OK:
        msg = L.load().c6_train_last_error().decode("utf-8", "replace")
        raise (ValueError if rc in (L.C6_ERR_ARG, L.C6_ERR_UNSUPPORTED) else RuntimeError)(f"c6_conv_layer_backward failed: {msg}")
    return dx, dw, db


def backward_status(x: torch.Tensor) -> int:
    """Status word of the most recently used workspace on x's device for x's shape family (synchronises)."""
    torch.cuda.synchronize(x.device)
    return max((int(ws[0].item()) & 0xFFFFFFFF for key, ws in _workspaces.items() if key[0] == x.device.index), default=0)


class SiluConv3x3(torch.autograd.Function):
    """y = silu(conv2d(x, weight, bias, padding=1)) whose backward runs on the library's tensor-core kernels."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        ctx.save_for_backward(x, weight, bias)
        return torch.nn.functional.silu(torch.nn.functional.conv2d(x, weight, bias, padding=1))

    @staticmethod
    def backward(ctx, grad_out):
        x, weight, bias = ctx.saved_tensors
        dx, dw, db = conv_layer_backward(x, weight, bias, grad_out, need_dx=ctx.needs_input_grad[0])
        # autograd wants each gradient in its tensor's own dtype (bf16 activations under autocast, fp32 parameters)
        return (None if dx is None else dx.to(x.dtype)), dw.to(weight.dtype), (db.to(bias.dtype) if bias is not None else None)


def supports_layer(conv: torch.nn.Conv2d, board_size: int) -> bool:
    """Whether `conv_layer_backward` covers this layer: 3x3, stride 1, 'same' padding, at most 128 channels."""
    return (tuple(conv.kernel_size) == (3, 3) and tuple(conv.stride) == (1, 1) and tuple(conv.padding) == (1, 1)
            and tuple(conv.dilation) == (1, 1) and conv.groups == 1 and conv.in_channels <= 128
            and conv.out_channels <= 128 and board_size <= 32)
