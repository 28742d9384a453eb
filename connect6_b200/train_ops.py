"""Training-side operators on the engine library's own kernels (include/c6_train.h).

The reference differentiates its network with PyTorch autograd inside the PPO minibatch update
(connect6/train.py:1032-1147).  `conv_layer_backward` does the backward of ONE backbone layer
y = silu(conv2d(x, W, b)) (connect6/model.py:104-106) on tcgen05 tensor cores: dX, dW and db from x, W, b
and dL/dy.  `SiluConv3x3` wraps it as a torch.autograd.Function whose forward is PyTorch's own (the
parameters stay ordinary nn.Parameters), so a layer can be switched over without touching the optimizer.
`SiluConvStack` does forward AND backward of a whole run of consecutive 3x3 layers in the library: the
forward keeps every layer's input in the kernels' own 16-bit plane layout, the backward walks the stack
with the gradient in that layout, and only the ends of the stack are NCHW tensors.
CUDA only: there is no CPU implementation in this package.
"""
from __future__ import annotations

import ctypes as C

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


# ---- a stack of 3x3 layers ---------------------------------------------------------------------------
_stack_pool: dict[tuple, list[torch.Tensor]] = {}


class _StackLease:
    """A zero-initialised workspace of one stack shape, taken from a pool for the time between a forward call
    and the end of its autograd graph; handed back when the lease is garbage-collected.  The operators keep the
    zero padding they rely on intact, so a returned buffer is reused without clearing."""

    def __init__(self, device: torch.device, n: int, channels: tuple[int, ...], B: int) -> None:
        self.key = (device.index, n, channels, B)
        pool = _stack_pool.setdefault(self.key, [])
        if pool:
            self.ws = pool.pop()
        else:
            arr = (C.c_int32 * len(channels))(*channels)
            need = int(L.load().c6_backbone_workspace_bytes(n, len(channels) - 1, arr, B))
            if need == 0:
                raise ValueError(f"SiluConvStack supports 1..16 layers of 3x3, board size <= 32, at most 128 channels; "
                                 f"got n={n}, channels={channels}")
            self.ws = torch.zeros((need + 7) // 8, dtype=torch.int64, device=device)

    def __del__(self) -> None:
        try:
            pool = _stack_pool.setdefault(self.key, [])
            if len(pool) < 2:
                pool.append(self.ws)
        except Exception:   # interpreter shutdown
            pass


def _ptr_array(tensors) -> "C.Array":
    return (C.c_void_p * len(tensors))(*[None if t is None else t.data_ptr() for t in tensors])


def _train_fail(rc: int, what: str):
    msg = L.load().c6_train_last_error().decode("utf-8", "replace")
    return (ValueError if rc in (L.C6_ERR_ARG, L.C6_ERR_UNSUPPORTED) else RuntimeError)(f"{what} failed: {msg}")


def stack_forward(x: torch.Tensor, weights, biases):
    """y = the layers y_l = silu(conv2d(y_{l-1}, weights[l], biases[l], padding=1)) applied in turn to x
    [B, c0, n, n]; returns (y fp32 [B, cL, n, n], lease) -- the lease holds the saved activations for
    `stack_backward`."""
    if not x.is_cuda:
        raise RuntimeError(f"stack_forward: expected CUDA tensors, got {x.device} (no CPU path in this package)")
    if x.ndim != 4 or x.shape[2] != x.shape[3] or len(weights) != len(biases) or not weights:
        raise ValueError("stack_forward: x [B,c0,n,n], one weight [c_out,c_in,3,3] and one bias (or None) per layer")
    B, c0, n, _ = x.shape
    channels = [c0]
    for w, b in zip(weights, biases):
        if w.ndim != 4 or tuple(w.shape[1:]) != (channels[-1], 3, 3) or (b is not None and tuple(b.shape) != (w.shape[0],)):
            raise ValueError("stack_forward: the layers' shapes do not chain (3x3 filters, c_in of a layer = c_out of the one before)")
        channels.append(int(w.shape[0]))
    if B == 0:
        return x.new_zeros((0, channels[-1], n, n), dtype=torch.float32), None
    dev = x.device
    f32 = lambda t: None if t is None else t.detach().to(device=dev, dtype=torch.float32).contiguous()
    x = f32(x)
    ws_ = [f32(w) for w in weights]
    bs_ = [f32(b) for b in biases]
    lease = _StackLease(dev, n, tuple(channels), B)
    y = torch.empty((B, channels[-1], n, n), device=dev, dtype=torch.float32)
    arr = (C.c_int32 * len(channels))(*channels)
    with torch.cuda.device(dev):
        rc = L.load().c6_backbone_forward(dev.index, n, len(ws_), arr, B, x.data_ptr(), _ptr_array(ws_), _ptr_array(bs_),
                                          y.data_ptr(), lease.ws.data_ptr(), lease.ws.numel() * 8,
                                          torch.cuda.current_stream(dev).cuda_stream)
    if rc != L.C6_OK:
        raise _train_fail(rc, "c6_backbone_forward")
    return y, lease


def stack_backward(lease: _StackLease, grad_out: torch.Tensor, need_dx: bool = True):
    """(dx or None, [dw_l], [db_l]) of the stack whose forward produced `lease`, given grad_out = dL/dy."""
    dev_index, n, channels, B = lease.key
    dev = grad_out.device
    if not grad_out.is_cuda or dev.index != dev_index or tuple(grad_out.shape) != (B, channels[-1], n, n):
        raise ValueError("stack_backward: grad_out does not belong to this forward call")
    grad_out = grad_out.detach().to(dtype=torch.float32).contiguous()
    dx = torch.empty((B, channels[0], n, n), device=dev, dtype=torch.float32) if need_dx else None
    dws = [torch.empty((channels[l + 1], channels[l], 3, 3), device=dev, dtype=torch.float32) for l in range(len(channels) - 1)]
    dbs = [torch.empty(channels[l + 1], device=dev, dtype=torch.float32) for l in range(len(channels) - 1)]
    arr = (C.c_int32 * len(channels))(*channels)
    with torch.cuda.device(dev):
        rc = L.load().c6_backbone_backward(dev_index, n, len(dws), arr, B, grad_out.data_ptr(), L.ptr(dx), _ptr_array(dws),
                                           _ptr_array(dbs), lease.ws.data_ptr(), lease.ws.numel() * 8,
                                           torch.cuda.current_stream(dev).cuda_stream)
    if rc != L.C6_OK:
        raise _train_fail(rc, "c6_backbone_backward")
    return dx, dws, dbs


def stack_status(lease: _StackLease) -> int:
    """Device status word of a stack workspace (synchronises)."""
    return int(lease.ws[0].item()) & 0xFFFFFFFF


class SiluConvStack(torch.autograd.Function):
    """features = the 3x3 backbone layers applied to x, forward and backward on the library's tensor-core kernels.
    Call as SiluConvStack.apply(x, w_1, b_1, w_2, b_2, ...)."""

    @staticmethod
    def forward(ctx, x, *params):
        weights, biases = list(params[0::2]), list(params[1::2])
        y, lease = stack_forward(x, weights, biases)
        ctx.lease = lease
        ctx.dtypes = (x.dtype, [p.dtype for p in params])
        ctx.nparams = len(params)
        return y.to(x.dtype) if x.dtype != torch.float32 else y

    @staticmethod
    def backward(ctx, grad_out):
        if ctx.lease is None:   # empty batch
            return (None,) * (1 + ctx.nparams)
        dx, dws, dbs = stack_backward(ctx.lease, grad_out, need_dx=ctx.needs_input_grad[0])
        xdt, pdts = ctx.dtypes
        grads = [None if dx is None else dx.to(xdt)]
        for l, (dw, db) in enumerate(zip(dws, dbs)):
            grads.append(dw.to(pdts[2 * l]) if ctx.needs_input_grad[1 + 2 * l] else None)
            grads.append(db.to(pdts[2 * l + 1]) if ctx.needs_input_grad[2 + 2 * l] else None)
        return tuple(grads)
