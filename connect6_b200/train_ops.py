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


def _f32(t: torch.Tensor | None, dev: torch.device) -> torch.Tensor | None:
    """t as a contiguous fp32 tensor on dev without autograd history; t itself when it already is one (the usual case:
    no dispatcher call on the hot path of a 256-board minibatch, which is bound by host time)."""
    if t is None:
        return None
    if t.dtype is torch.float32 and t.device == dev and t.is_contiguous():
        return t.detach() if t.requires_grad else t
    return t.detach().to(device=dev, dtype=torch.float32).contiguous()


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
    f32 = lambda t: _f32(t, dev)
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


def supports_stem(conv: torch.nn.Conv2d, board_size: int) -> bool:
    """Whether `SiluConvStack` can start with this layer: k x k (odd k <= 31) on 3 planes, stride 1, 'same' padding, at
    most 64 output channels."""
    k = conv.kernel_size[0]
    return (conv.kernel_size[0] == conv.kernel_size[1] and k % 2 == 1 and 3 < k <= 31 and tuple(conv.stride) == (1, 1)
            and tuple(conv.padding) == (k // 2, k // 2) and tuple(conv.dilation) == (1, 1) and conv.groups == 1
            and conv.in_channels == 3 and conv.out_channels <= 64 and board_size <= 32)


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

    def __init__(self, device: torch.device, n: int, channels: tuple[int, ...], B: int, stem_k: int = 0) -> None:
        self.key = (device.index, n, channels, B, stem_k)
        pool = _stack_pool.setdefault(self.key, [])
        if pool:
            self.ws = pool.pop()
        else:
            arr = (C.c_int32 * len(channels))(*channels)
            need = int(L.load().c6_backbone_workspace_bytes(n, len(channels) - 1, arr, stem_k, B))
            if need == 0:
                raise ValueError(f"SiluConvStack supports 1..16 layers of 3x3 with at most 128 channels on boards up to 32x32, "
                                 f"optionally behind an odd k x k stem (k <= 31) from 3 planes to at most 64 channels; "
                                 f"got n={n}, channels={channels}, stem {stem_k}")
            self.ws = torch.zeros((need + 7) // 8, dtype=torch.int64, device=device)

    def __del__(self) -> None:
        try:
            pool = _stack_pool.pop(self.key, [])          # re-inserted last: the dict keeps the keys in order of use
            if len(pool) < 2:
                pool.append(self.ws)
            _stack_pool[self.key] = pool
            while len(_stack_pool) > 4:                   # shapes no longer in use give their memory back
                _stack_pool.pop(next(iter(_stack_pool)))
        except Exception:   # interpreter shutdown
            pass


def _ptr_array(tensors) -> "C.Array":
    return (C.c_void_p * len(tensors))(*[None if t is None else t.data_ptr() for t in tensors])


def _train_fail(rc: int, what: str):
    msg = L.load().c6_train_last_error().decode("utf-8", "replace")
    return (ValueError if rc in (L.C6_ERR_ARG, L.C6_ERR_UNSUPPORTED) else RuntimeError)(f"{what} failed: {msg}")


def stack_forward(x: torch.Tensor, weights, biases, want_features: bool = True):
    """y = the layers y_l = silu(conv2d(y_{l-1}, weights[l], biases[l], padding=k_l//2)) applied in turn to x
    [B, c0, n, n]; returns (y fp32 [B, cL, n, n], lease) -- the lease holds the saved activations for
    `stack_backward`.  Every filter is 3x3, except that the first may be the network's k x k stem on the 3 input
    planes (then x is the network input).  want_features=False returns y = None: the features stay in the lease only,
    for `heads_forward`."""
    if not x.is_cuda:
        raise RuntimeError(f"stack_forward: expected CUDA tensors, got {x.device} (no CPU path in this package)")
    if x.ndim != 4 or x.shape[2] != x.shape[3] or len(weights) != len(biases) or not weights:
        raise ValueError("stack_forward: x [B,c0,n,n], one weight [c_out,c_in,3,3] and one bias (or None) per layer")
    B, c0, n, _ = x.shape
    channels = [c0]
    stem_k = 0
    for l, (w, b) in enumerate(zip(weights, biases)):
        k = int(w.shape[-1]) if w.ndim == 4 else 0
        if l == 0 and k != 3 and c0 == 3 and len(weights) > 1:
            stem_k = k
        if (w.ndim != 4 or tuple(w.shape[1:]) != (channels[-1], k, k) or (k != 3 and not (l == 0 and stem_k))
                or (b is not None and tuple(b.shape) != (w.shape[0],))):
            raise ValueError("stack_forward: the layers' shapes do not chain (3x3 filters -- the first may be a k x k stem on "
                             "3 planes --, c_in of a layer = c_out of the one before)")
        channels.append(int(w.shape[0]))
    if B == 0:
        return x.new_zeros((0, channels[-1], n, n), dtype=torch.float32), None
    dev = x.device
    f32 = lambda t: _f32(t, dev)
    x = f32(x)
    ws_ = [f32(w) for w in weights]
    bs_ = [f32(b) for b in biases]
    lease = _StackLease(dev, n, tuple(channels), B, stem_k)
    y = torch.empty((B, channels[-1], n, n), device=dev, dtype=torch.float32) if want_features else None
    arr = (C.c_int32 * len(channels))(*channels)
    with torch.cuda.device(dev):
        rc = L.load().c6_backbone_forward(dev.index, n, len(ws_), arr, stem_k, B, x.data_ptr(), _ptr_array(ws_), _ptr_array(bs_),
                                          L.ptr(y), lease.ws.data_ptr(), lease.ws.numel() * 8,
                                          torch.cuda.current_stream(dev).cuda_stream)
    if rc != L.C6_OK:
        raise _train_fail(rc, "c6_backbone_forward")
    return y, lease


def stack_backward(lease: _StackLease, grad_out: torch.Tensor | None, need_dx: bool = True):
    """(dx or None, [dw_l], [db_l]) of the stack whose forward produced `lease`, given grad_out = dL/dy (None: the
    gradient of the features was left in the lease by `heads_backward`).  A stack that starts with the stem has no dx
    (its input is the network input)."""
    dev_index, n, channels, B, stem_k = lease.key
    need_dx = need_dx and not stem_k
    dev = lease.ws.device
    if grad_out is not None:
        if not grad_out.is_cuda or grad_out.device.index != dev_index or tuple(grad_out.shape) != (B, channels[-1], n, n):
            raise ValueError("stack_backward: grad_out does not belong to this forward call")
        grad_out = grad_out.detach().to(dtype=torch.float32).contiguous()
    dx = torch.empty((B, channels[0], n, n), device=dev, dtype=torch.float32) if need_dx else None
    dws = [torch.empty((channels[l + 1], channels[l], stem_k if (stem_k and l == 0) else 3, stem_k if (stem_k and l == 0) else 3),
                       device=dev, dtype=torch.float32) for l in range(len(channels) - 1)]
    dbs = [torch.empty(channels[l + 1], device=dev, dtype=torch.float32) for l in range(len(channels) - 1)]
    arr = (C.c_int32 * len(channels))(*channels)
    with torch.cuda.device(dev):
        rc = L.load().c6_backbone_backward(dev_index, n, len(dws), arr, stem_k, B, L.ptr(grad_out), L.ptr(dx), _ptr_array(dws),
                                           _ptr_array(dbs), lease.ws.data_ptr(), lease.ws.numel() * 8,
                                           torch.cuda.current_stream(dev).cuda_stream)
    if rc != L.C6_OK:
        raise _train_fail(rc, "c6_backbone_backward")
    return dx, dws, dbs


def heads_forward(lease: _StackLease, pw: torch.Tensor, pb: torch.Tensor, vw: torch.Tensor, vb: torch.Tensor):
    """(logits [B, n*n], value [B]) of the two 1x1 heads (connect6/model.py:70-75,108-110) on the features that
    `stack_forward` left in the lease.  pw, vw: the [1, C, 1, 1] filters; pb, vb: [1]."""
    dev_index, n, channels, B, stem_k = lease.key
    dev = lease.ws.device
    f32 = lambda t: _f32(t, dev)
    pw, pb, vw, vb = f32(pw).reshape(-1), f32(pb).reshape(-1), f32(vw).reshape(-1), f32(vb).reshape(-1)
    if pw.numel() != channels[-1] or vw.numel() != channels[-1] or pb.numel() != 1 or vb.numel() != 1:
        raise ValueError("heads_forward: head parameters do not fit the features' channel count")
    logits = torch.empty((B, n * n), device=dev, dtype=torch.float32)
    value = torch.empty(B, device=dev, dtype=torch.float32)
    arr = (C.c_int32 * len(channels))(*channels)
    with torch.cuda.device(dev):
        rc = L.load().c6_backbone_heads_forward(dev_index, n, len(channels) - 1, arr, stem_k, B, pw.data_ptr(), pb.data_ptr(),
                                                vw.data_ptr(), vb.data_ptr(), logits.data_ptr(), value.data_ptr(),
                                                lease.ws.data_ptr(), lease.ws.numel() * 8,
                                                torch.cuda.current_stream(dev).cuda_stream)
    if rc != L.C6_OK:
        raise _train_fail(rc, "c6_backbone_heads_forward")
    return logits, value


def heads_backward(lease: _StackLease, pw: torch.Tensor, vw: torch.Tensor, dlogits: torch.Tensor, dvalue: torch.Tensor,
                   value: torch.Tensor):
    """(dpw, dpb, dvw, dvb) of the heads; the gradient of the features goes into the lease, where
    `stack_backward(lease, None)` picks it up."""
    dev_index, n, channels, B, stem_k = lease.key
    dev = lease.ws.device
    f32 = lambda t: _f32(t, dev)
    pwf, vwf, dlogits, dvalue, value = f32(pw).reshape(-1), f32(vw).reshape(-1), f32(dlogits), f32(dvalue), f32(value)
    if tuple(dlogits.shape) != (B, n * n) or tuple(dvalue.shape) != (B,) or tuple(value.shape) != (B,):
        raise ValueError("heads_backward: gradients do not belong to this forward call")
    Cc = channels[-1]
    dpw, dvw = torch.empty(Cc, device=dev, dtype=torch.float32), torch.empty(Cc, device=dev, dtype=torch.float32)
    dpb, dvb = torch.empty(1, device=dev, dtype=torch.float32), torch.empty(1, device=dev, dtype=torch.float32)
    arr = (C.c_int32 * len(channels))(*channels)
    with torch.cuda.device(dev):
        rc = L.load().c6_backbone_heads_backward(dev_index, n, len(channels) - 1, arr, stem_k, B, pwf.data_ptr(), vwf.data_ptr(),
                                                 dlogits.data_ptr(), dvalue.data_ptr(), value.data_ptr(), dpw.data_ptr(),
                                                 dpb.data_ptr(), dvw.data_ptr(), dvb.data_ptr(), lease.ws.data_ptr(),
                                                 lease.ws.numel() * 8, torch.cuda.current_stream(dev).cuda_stream)
    if rc != L.C6_OK:
        raise _train_fail(rc, "c6_backbone_heads_backward")
    return dpw.view_as(pw), dpb, dvw.view_as(vw), dvb


def stack_forward_boards(boards: torch.Tensor, current_player: torch.Tensor, stones_left: torch.Tensor,
                         index: torch.Tensor | None, weights, biases, want_features: bool = True):
    """`stack_forward` for a stack that starts with the network's stem, fed with the environment's raw int8 state
    (boards [E, n, n], current_player [E], stones_left [E]) and an optional int64 index [B] selecting the boards --
    what the PPO minibatch holds in its buffer (connect6/train.py:1038-1046): the gather and canonical_network_input
    (connect6/vector_env.py:196-218) happen inside the first kernel."""
    if not boards.is_cuda:
        raise RuntimeError(f"stack_forward_boards: expected CUDA tensors, got {boards.device} (no CPU path in this package)")
    if boards.ndim != 3 or boards.shape[1] != boards.shape[2] or boards.dtype != torch.int8:
        raise ValueError("stack_forward_boards: boards must be int8 [E, n, n]")
    E, n, _ = boards.shape
    for name, v in (("current_player", current_player), ("stones_left", stones_left)):
        if tuple(v.shape) != (E,) or v.dtype != torch.int8 or v.device != boards.device:
            raise ValueError(f"stack_forward_boards: {name} must be int8 [E] on the boards' device")
    if index is not None and (index.ndim != 1 or index.dtype != torch.int64 or index.device != boards.device):
        raise ValueError("stack_forward_boards: index must be int64 [B] on the boards' device")
    if len(weights) != len(biases) or len(weights) < 2 or weights[0].ndim != 4 or weights[0].shape[1] != 3:
        raise ValueError("stack_forward_boards: the stack must start with the stem on the 3 input planes and have a 3x3 layer behind it")
    B = E if index is None else int(index.shape[0])
    stem_k = int(weights[0].shape[-1])
    channels = [3]
    for l, (w, b) in enumerate(zip(weights, biases)):
        k = stem_k if l == 0 else 3
        if w.ndim != 4 or tuple(w.shape[1:]) != (channels[-1], k, k) or (b is not None and tuple(b.shape) != (w.shape[0],)):
            raise ValueError("stack_forward_boards: the layers' shapes do not chain (a k x k stem on 3 planes, then 3x3 filters)")
        channels.append(int(w.shape[0]))
    dev = boards.device
    if B == 0:
        return torch.zeros((0, channels[-1], n, n), device=dev), None
    f32 = lambda t: _f32(t, dev)
    ws_ = [f32(w) for w in weights]
    bs_ = [f32(b) for b in biases]
    boards, current_player, stones_left = boards.contiguous(), current_player.contiguous(), stones_left.contiguous()
    index = None if index is None else index.contiguous()
    lease = _StackLease(dev, n, tuple(channels), B, stem_k)
    y = torch.empty((B, channels[-1], n, n), device=dev, dtype=torch.float32) if want_features else None
    arr = (C.c_int32 * len(channels))(*channels)
    with torch.cuda.device(dev):
        rc = L.load().c6_backbone_forward_boards(dev.index, n, len(ws_), arr, stem_k, B, boards.data_ptr(), current_player.data_ptr(),
                                                 stones_left.data_ptr(), E, L.ptr(index), _ptr_array(ws_), _ptr_array(bs_), L.ptr(y),
                                                 lease.ws.data_ptr(), lease.ws.numel() * 8,
                                                 torch.cuda.current_stream(dev).cuda_stream)
    if rc != L.C6_OK:
        raise _train_fail(rc, "c6_backbone_forward_boards")
    return y, lease


def stack_status(lease: _StackLease) -> int:
    """Device status word of a stack workspace (synchronises)."""
    return int(lease.ws[0].item()) & 0xFFFFFFFF


class SiluConvStack(torch.autograd.Function):
    """features = the backbone layers applied to x, forward and backward on the library's tensor-core kernels: 3x3
    layers, optionally starting with the network's k x k stem on the 3 input planes.
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


class PolicyValueStack(torch.autograd.Function):
    """(logits, value) = the whole network -- stem or first 3x3 layer, the 3x3 layers, both heads -- forward and
    backward on the library's kernels; the features never leave the kernels' plane layout.
    Call as PolicyValueStack.apply(x, w_1, b_1, ..., w_L, b_L, policy_w, policy_b, value_w, value_b)."""

    @staticmethod
    def forward(ctx, x, *params):
        conv_params, (pw, pb, vw, vb) = params[:-4], params[-4:]
        weights, biases = list(conv_params[0::2]), list(conv_params[1::2])
        _, lease = stack_forward(x, weights, biases, want_features=False)
        logits, value = heads_forward(lease, pw, pb, vw, vb)
        ctx.lease = lease
        ctx.save_for_backward(pw, vw, value)
        ctx.dtypes = (x.dtype, [p.dtype for p in params])
        return logits, value

    @staticmethod
    def backward(ctx, dlogits, dvalue):
        pw, vw, value = ctx.saved_tensors
        lease = ctx.lease
        B = lease.key[3]
        if dlogits is None:
            dlogits = torch.zeros((B, lease.key[1] ** 2), device=value.device)
        if dvalue is None:
            dvalue = torch.zeros(B, device=value.device)
        dpw, dpb, dvw, dvb = heads_backward(lease, pw, vw, dlogits, dvalue, value)
        dx, dws, dbs = stack_backward(lease, None, need_dx=ctx.needs_input_grad[0])
        xdt, pdts = ctx.dtypes
        grads = [None if dx is None else dx.to(xdt)]
        for l, (dw, db) in enumerate(zip(dws, dbs)):
            grads.append(dw.to(pdts[2 * l]))
            grads.append(db.to(pdts[2 * l + 1]))
        n = len(pdts)
        grads += [dpw.to(pdts[n - 4]), dpb.to(pdts[n - 3]), dvw.to(pdts[n - 2]), dvb.to(pdts[n - 1])]
        return tuple(grads)


# ---- PPO minibatch loss ------------------------------------------------------------------------------
class _PpoLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, values, legal, actions, old_logprob, advantages, returns, temperature, clip_coef, value_coef,
                entropy_coef):
        if not logits.is_cuda:
            raise RuntimeError(f"ppo_loss: expected CUDA tensors, got {logits.device} (no CPU path in this package)")
        if logits.ndim != 2 or tuple(legal.shape) != tuple(logits.shape):
            raise ValueError("ppo_loss: logits and legal must be [B, A]")
        B, A = logits.shape
        for name, v in (("values", values), ("actions", actions), ("old_logprob", old_logprob), ("advantages", advantages), ("returns", returns)):
            if tuple(v.shape) != (B,):
                raise ValueError(f"ppo_loss: {name} must be [B]")
        dev = logits.device
        f32 = lambda v: _f32(v, dev)
        lg, vv, old, adv, ret = f32(logits), f32(values), f32(old_logprob), f32(advantages), f32(returns)
        lm = legal.detach().to(device=dev, dtype=torch.uint8).contiguous()
        act = actions.detach().to(device=dev, dtype=torch.int64).contiguous()
        stats = torch.empty(6, device=dev, dtype=torch.float32)
        dlogits = torch.empty_like(lg)
        dvalues = torch.empty_like(vv)
        if B == 0:
            raise ValueError("ppo_loss: empty minibatch")
        ws = torch.empty(B * 5, device=dev, dtype=torch.float32)
        with torch.cuda.device(dev):
            rc = L.load().c6_ppo_loss(dev.index, B, A, lg.data_ptr(), lm.data_ptr(), act.data_ptr(), old.data_ptr(), adv.data_ptr(),
                                      ret.data_ptr(), vv.data_ptr(), float(temperature), float(clip_coef), float(value_coef),
                                      float(entropy_coef), stats.data_ptr(), dlogits.data_ptr(), dvalues.data_ptr(), ws.data_ptr(),
                                      ws.numel() * 4, torch.cuda.current_stream(dev).cuda_stream)
        if rc != L.C6_OK:
            raise _train_fail(rc, "c6_ppo_loss")
        ctx.save_for_backward(dlogits, dvalues)
        ctx.dtypes = (logits.dtype, values.dtype)
        ctx.mark_non_differentiable(stats)
        return stats[0].clone(), stats

    @staticmethod
    def backward(ctx, grad_loss, _grad_stats):
        dlogits, dvalues = ctx.saved_tensors
        return ((grad_loss * dlogits).to(ctx.dtypes[0]), (grad_loss * dvalues).to(ctx.dtypes[1])) + (None,) * 9


def ppo_loss(logits: torch.Tensor, values: torch.Tensor, legal: torch.Tensor, actions: torch.Tensor, old_logprob: torch.Tensor,
             advantages: torch.Tensor, returns: torch.Tensor, temperature: float = 1.0, clip_coef: float = 0.2,
             value_coef: float = 0.5, entropy_coef: float = 0.01):
    """(loss, stats) of one PPO minibatch from the network's outputs, as connect6/train.py:1047-1094 computes them:
    loss = clipped-ratio policy loss + value_coef * 0.5 (v - ret)^2 - entropy_coef * entropy over the masked,
    temperature-scaled action distribution; stats = [loss, policy loss, value loss, entropy, approx_kl, clipfrac]
    (a device tensor: no synchronisation).  `loss` is differentiable with respect to logits and values: one kernel
    computes the loss and both gradients, `loss.backward()` only scales them."""
    return _PpoLoss.apply(logits, values, legal, actions, old_logprob, advantages, returns, temperature, clip_coef,
                          value_coef, entropy_coef)


# ---- gradient clipping + AdamW -----------------------------------------------------------------------
class ClipAdamW(torch.optim.Optimizer):
    """torch.optim.AdamW with nn.utils.clip_grad_norm_ folded in, for a model's whole parameter list in two kernel
    launches (connect6/train.py:476-481 sets the optimizer up, :1121-1145 clips and steps).  `step()` returns the total
    gradient norm BEFORE clipping as a device tensor (what clip_grad_norm_ returns) without synchronising; a
    non-finite norm leaves the parameters untouched.  The state (`step`, `exp_avg`, `exp_avg_sq` per parameter) and
    `state_dict()` have torch.optim.AdamW's layout, so checkpoints move between the two.  One parameter group per
    call of the kernel; fp32 CUDA parameters only."""

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 1e-2,
                 max_grad_norm: float = 0.0, capturable: bool = False) -> None:
        if lr < 0 or eps < 0 or not 0 <= betas[0] < 1 or not 0 <= betas[1] < 1 or weight_decay < 0:
            raise ValueError("ClipAdamW: invalid hyper-parameter")
        # capturable=True keeps the update count on the device (like torch.optim.AdamW's flag of that name), so that a
        # step captured in a CUDA graph can be replayed; the learning rate then is the value at capture time
        super().__init__(params, dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay, max_grad_norm=max_grad_norm,
                                      amsgrad=False, maximize=False, foreach=None, capturable=bool(capturable), differentiable=False,
                                      fused=None))

    @torch.no_grad()
    def step(self, closure=None):
        if closure is not None:
            raise RuntimeError("ClipAdamW.step takes no closure")
        norms = []
        for group in self.param_groups:
            ps = [p for p in group["params"] if p.grad is not None]
            if not ps:
                continue
            dev = ps[0].device
            for p in ps:
                if not p.is_cuda or p.dtype != torch.float32 or p.device != dev or not p.is_contiguous() or not p.grad.is_contiguous() \
                        or p.grad.dtype != torch.float32:
                    raise RuntimeError("ClipAdamW: contiguous fp32 CUDA parameters and gradients on one device only (no CPU path)")
                st = self.state[p]
                if not st:
                    st["step"] = torch.zeros((), device=dev) if group["capturable"] else torch.tensor(0.0)
                    st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
            step_dev = None
            if group["capturable"]:
                # one device counter for the group: every parameter's "step" entry is that tensor
                step_dev = self.state[ps[0]]["step"]
                if not step_dev.is_cuda:
                    step_dev = step_dev.to(dev)
                for p in ps:
                    self.state[p]["step"] = step_dev
                step = 0
            else:
                steps = {int(self.state[p]["step"]) for p in ps}
                if len(steps) != 1:
                    raise RuntimeError("ClipAdamW: the parameters of a group must have been stepped together")
                step = steps.pop() + 1
            norm = torch.empty(1, device=dev, dtype=torch.float32)
            pool = self.__dict__.setdefault("_c6_workspaces", {})
            ws = pool.get(dev)
            if ws is None:
                ws = pool[dev] = torch.empty(148, device=dev, dtype=torch.float32)
            b1, b2 = group["betas"]
            for lo in range(0, len(ps), 48):
                chunk = ps[lo:lo + 48]
                if len(ps) > 48:
                    raise RuntimeError("ClipAdamW: at most 48 parameter tensors per group")
                sizes = (C.c_int64 * len(chunk))(*[p.numel() for p in chunk])
                with torch.cuda.device(dev):
                    rc = L.load().c6_clip_adamw_step(dev.index, len(chunk), sizes, _ptr_array(chunk), _ptr_array([p.grad for p in chunk]),
                                                     _ptr_array([self.state[p]["exp_avg"] for p in chunk]),
                                                     _ptr_array([self.state[p]["exp_avg_sq"] for p in chunk]), float(group["lr"]),
                                                     float(b1), float(b2), float(group["eps"]), float(group["weight_decay"]),
                                                     float(group["max_grad_norm"]), step, L.ptr(step_dev), norm.data_ptr(), ws.data_ptr(),
                                                     ws.numel() * 4, torch.cuda.current_stream(dev).cuda_stream)
                if rc != L.C6_OK:
                    raise _train_fail(rc, "c6_clip_adamw_step")
            if step_dev is None:
                for p in ps:
                    self.state[p]["step"] += 1
            norms.append(norm)
        if not norms:
            return None
        return norms[0][0] if len(norms) == 1 else torch.stack([n[0] for n in norms])


class PolicyValueStackFromBoards(torch.autograd.Function):
    """`PolicyValueStack` fed with the environment's raw int8 state instead of network-input planes (see
    `stack_forward_boards`).  Call as PolicyValueStackFromBoards.apply(boards, current_player, stones_left, index,
    w_1, b_1, ..., policy_w, policy_b, value_w, value_b); index may be an empty tensor for "every board"."""

    @staticmethod
    def forward(ctx, boards, current_player, stones_left, index, *params):
        conv_params, (pw, pb, vw, vb) = params[:-4], params[-4:]
        weights, biases = list(conv_params[0::2]), list(conv_params[1::2])
        _, lease = stack_forward_boards(boards, current_player, stones_left, index if index.numel() else None, weights, biases,
                                        want_features=False)
        logits, value = heads_forward(lease, pw, pb, vw, vb)
        ctx.lease = lease
        ctx.save_for_backward(pw, vw, value)
        ctx.pdtypes = [p.dtype for p in params]
        return logits, value

    @staticmethod
    def backward(ctx, dlogits, dvalue):
        pw, vw, value = ctx.saved_tensors
        lease = ctx.lease
        B = lease.key[3]
        if dlogits is None:
            dlogits = torch.zeros((B, lease.key[1] ** 2), device=value.device)
        if dvalue is None:
            dvalue = torch.zeros(B, device=value.device)
        dpw, dpb, dvw, dvb = heads_backward(lease, pw, vw, dlogits, dvalue, value)
        _, dws, dbs = stack_backward(lease, None, need_dx=False)
        pd = ctx.pdtypes
        grads = [None, None, None, None]
        for l, (dw, db) in enumerate(zip(dws, dbs)):
            grads.append(dw.to(pd[2 * l]))
            grads.append(db.to(pd[2 * l + 1]))
        n = len(pd)
        grads += [dpw.to(pd[n - 4]), dpb.to(pd[n - 3]), dvw.to(pd[n - 2]), dvb.to(pd[n - 1])]
        return tuple(grads)


def ppo_minibatch_update(model, optimizer, boards: torch.Tensor, players: torch.Tensor, stones_left: torch.Tensor,
                         actions: torch.Tensor, old_logprob: torch.Tensor, advantages: torch.Tensor, returns: torch.Tensor,
                         idx: torch.Tensor, local_idx: torch.Tensor | None = None, *, temperature: float = 1.0,
                         clip_coef: float = 0.2, value_coef: float = 0.5, entropy_coef: float = 0.01):
    """One minibatch of the PPO update as the body of the reference's loop does it (connect6/train.py:1036-1145):
    gather the minibatch `idx` from the buffer tensors (boards int8 [N, n, n], players, stones_left int8 [N], actions,
    old_logprob [N]) and `local_idx` (default: idx) from advantages / returns, forward, loss, backward, gradient
    clipping and optimizer step.  With PolicyValueNet(engine_backward=True) and a ClipAdamW optimizer every kernel of
    it is the library's.  Returns (stats, grad_norm): stats = device tensor [loss, policy loss, value loss, entropy,
    approx_kl, clipfrac], grad_norm = the total gradient norm before clipping; nothing is synchronised -- the caller's
    KL watchdog reads stats[4:6] when it wants to."""
    local_idx = idx if local_idx is None else local_idx
    mb_boards = boards[idx]
    legal = mb_boards.reshape(mb_boards.shape[0], -1).eq(0)            # connect6/train.py:1046
    with torch.autocast("cuda", dtype=torch.bfloat16):
        if hasattr(model, "forward_from_boards"):
            logits, values = model.forward_from_boards(boards, players, stones_left, idx)
        else:
            from .selfplay import canonical_network_input
            logits, values = model(canonical_network_input(mb_boards, players[idx], stones_left[idx]))
        loss, stats = ppo_loss(logits.float(), values.float(), legal, actions[idx].long(), old_logprob[idx],
                               advantages[local_idx], returns[local_idx], temperature, clip_coef, value_coef, entropy_coef)
    optimizer.zero_grad(set_to_none=True)
    loss.backward()
    if isinstance(optimizer, ClipAdamW):
        grad_norm = optimizer.step()
    else:
        max_norm = optimizer.param_groups[0].get("max_grad_norm", 0.0)
        params = [p for g in optimizer.param_groups for p in g["params"]]
        grad_norm = torch.nn.utils.clip_grad_norm_(params, max_norm if max_norm > 0 else float("inf"))
        optimizer.step()
    return stats, grad_norm
