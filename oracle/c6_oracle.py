"""CPU oracle for the Connect6 policy/value CNN hot path (TEST INFRASTRUCTURE ONLY).

This module restates, in plain numpy, the arithmetic that the reference project
mgxmateusz/connect6 performs on its inference hot path.  It is the checker that
the parity tests, the smoke test and the CPU-baseline leg of the benchmark use.
Nothing in the shipped package imports it: the product path is the CUDA engine
and fails loudly without it.

The reference is pure Python on top of PyTorch, so the convolution arithmetic
itself lives in a third-party dependency (PyTorch, unpinned in the reference's
requirements.txt; 2.11.0 in this image).  The published algorithm restated here
is the cross-correlation "convolution" of torch.nn.functional.conv2d with
stride 1 and symmetric zero padding k//2.

Pinning: every function below is checked against fixtures under tests/golden/
that were produced by importing the unmodified reference (see
tests/golden/make_golden.py), and against the relational identities the
reference's own tests assert (grouped == per-model, D4 round trips).

Reference citations (paths inside the reference project):
  connect6/model.py:96-111     PolicyValueNet.forward        -> policy_value_forward
  connect6/model.py:123-125    mask_logits                   -> mask_logits
  connect6/history.py:251-303  grouped forward               -> grouped_policy_forward
  connect6/train.py:195-213    _sample_actions(_only)        -> masked_log_softmax / sample_inverse_cdf
  connect6/train.py:216-277    D4 helpers                    -> symmetry_for_phase / transform_*
  connect6/vector_env.py:196-218 canonical_network_input     -> canonical_network_input
"""
from __future__ import annotations

import numpy as np

FP32_MIN = float(np.finfo(np.float32).min)

# --------------------------------------------------------------------------------------
# convolution stack
# --------------------------------------------------------------------------------------


def conv2d_same(x: np.ndarray, w: np.ndarray, b: np.ndarray | None, dtype=np.float64) -> np.ndarray:
    """Stride-1 cross-correlation with zero padding k//2 (torch.nn.functional.conv2d).

    x [B,Cin,H,W], w [Cout,Cin,K,K], b [Cout] -> [B,Cout,H,W].
    Follows the call at connect6/model.py:56-63 (padding=kernel // 2, stride=1).
    """
    x = np.asarray(x, dtype=dtype)
    w = np.asarray(w, dtype=dtype)
    B, Cin, H, W = x.shape
    Cout, Cin2, K, K2 = w.shape
    assert Cin == Cin2 and K == K2 and K % 2 == 1
    p = K // 2
    xp = np.zeros((B, Cin, H + 2 * p, W + 2 * p), dtype=dtype)
    xp[:, :, p:p + H, p:p + W] = x
    out = np.zeros((B, Cout, H, W), dtype=dtype)
    # accumulate one filter tap at a time: out[b,o,r,c] += sum_i w[o,i,dy,dx] * xp[b,i,r+dy,c+dx]
    for dy in range(K):
        for dx in range(K):
            patch = xp[:, :, dy:dy + H, dx:dx + W]            # [B,Cin,H,W]
            out += np.einsum("oi,bihw->bohw", w[:, :, dy, dx], patch, optimize=True)
    if b is not None:
        out += np.asarray(b, dtype=dtype)[None, :, None, None]
    return out


def silu(x: np.ndarray) -> np.ndarray:
    """x * sigmoid(x) (torch.nn.SiLU, connect6/model.py:67)."""
    return x / (1.0 + np.exp(-x))


def n_layers_of(params: dict) -> int:
    n = 0
    while f"convs.{n}.weight" in params:
        n += 1
    return n


def backbone(x: np.ndarray, params: dict, dtype=np.float64) -> np.ndarray:
    """features = SiLU(conv(features)) for every backbone layer (connect6/model.py:104-106)."""
    f = np.asarray(x, dtype=dtype)
    for i in range(n_layers_of(params)):
        f = silu(conv2d_same(f, params[f"convs.{i}.weight"], params[f"convs.{i}.bias"], dtype))
    return f


def policy_value_forward(x: np.ndarray, params: dict, dtype=np.float64):
    """PolicyValueNet.forward (connect6/model.py:96-111).

    x [B,3,H,W]; params uses the reference state_dict keys.  Returns
    (logits [B,H*W] unmasked, value [B]).
    """
    x = np.asarray(x)
    if x.ndim != 4 or x.shape[1] != 3 or x.shape[2] != x.shape[3]:
        raise ValueError(f"model input must be [B,3,H,W], got {x.shape}")
    f = backbone(x, params, dtype)
    wp = np.asarray(params["policy_output.weight"], dtype=dtype).reshape(-1)
    bp = np.asarray(params["policy_output.bias"], dtype=dtype).reshape(())
    wv = np.asarray(params["value_output.weight"], dtype=dtype).reshape(-1)
    bv = np.asarray(params["value_output.bias"], dtype=dtype).reshape(())
    logits = np.einsum("c,bchw->bhw", wp, f).reshape(x.shape[0], -1) + bp      # model.py:108
    vmap = np.einsum("c,bchw->bhw", wv, f) + bv                                 # model.py:109
    value = np.tanh(vmap.mean(axis=(-2, -1)))                                   # model.py:110
    return logits, value


def grouped_policy_forward(x: np.ndarray, params_list: list[dict], dtype=np.float64) -> np.ndarray:
    """HistoricalPolicyEnsemble.forward_grouped (connect6/history.py:276-303).

    x [M,T,3,H,W] -> logits [M,T,H*W].  A grouped convolution with groups=M over
    channel-stacked models is, by definition, M independent convolutions; the
    reference's own test asserts this (tests/test_training_features.py:120-151).
    """
    x = np.asarray(x)
    if x.ndim != 5 or x.shape[0] != len(params_list):
        raise ValueError(f"grouped input must be [M,T,3,H,W] with M={len(params_list)}, got {x.shape}")
    return np.stack([policy_value_forward(x[m], params_list[m], dtype)[0] for m in range(len(params_list))])


def grouped_policy_value_forward(x: np.ndarray, params_list: list[dict], dtype=np.float64):
    """Per-group logits AND values: M independent PolicyValueNet forwards."""
    outs = [policy_value_forward(x[m], params_list[m], dtype) for m in range(len(params_list))]
    return np.stack([o[0] for o in outs]), np.stack([o[1] for o in outs])


# --------------------------------------------------------------------------------------
# masking, log-softmax, sampling
# --------------------------------------------------------------------------------------


def legal_from_planes(x: np.ndarray) -> np.ndarray:
    """legal = board.eq(0) (connect6/vector_env.py:95-96) restated on network planes:
    a cell is empty iff neither plane 0 (mine) nor plane 1 (opponent) is set."""
    x = np.asarray(x)
    return ((x[:, 0] == 0) & (x[:, 1] == 0)).reshape(x.shape[0], -1)


def mask_logits(logits: np.ndarray, legal: np.ndarray, fill: float = FP32_MIN) -> np.ndarray:
    """logits.masked_fill(~legal, finfo(dtype).min) (connect6/model.py:123-125)."""
    out = np.array(logits, dtype=np.float32, copy=True)
    out[~np.asarray(legal, dtype=bool)] = np.float32(fill)
    return out


def masked_log_softmax(logits: np.ndarray, legal: np.ndarray, temperature: float = 1.0) -> np.ndarray:
    """Normalised logits of Categorical(logits=mask(logits)/max(T,1e-4)) (connect6/train.py:200-203),
    i.e. z - logsumexp(z) with logsumexp = max + log(sum(exp(z - max))), in float64.

    Illegal cells come out near -3.4e38 (their exp is exactly 0).  Edge case kept from the
    reference: if NO cell is legal every z equals the fill, log(361) is absorbed when added to
    -3.4e38, and the result is 0 for every cell (torch returns the same); the probabilities
    softmax(z) are still uniform.  A fill that overflowed to -inf (T < 1) is clamped to the most
    negative finite value, where torch would raise for the all-occupied row."""
    z = mask_logits(logits, legal).astype(np.float64) / max(float(temperature), 1e-4)
    z = np.maximum(z, np.finfo(np.float64).min)
    m = z.max(axis=-1, keepdims=True)
    lse = m + np.log(np.exp(z - m).sum(axis=-1, keepdims=True))
    return z - lse


def sample_inverse_cdf(logp: np.ndarray, u: np.ndarray) -> np.ndarray:
    """Inverse-CDF draw: smallest a with cdf[a] > u * cdf[-1], one u per row.  The weights are
    exp(logp - max) so that the degenerate all-occupied row (logp == 0 everywhere) is uniform."""
    p = np.exp(logp - logp.max(axis=-1, keepdims=True))
    cdf = np.cumsum(p, axis=-1)
    target = np.asarray(u, dtype=np.float64)[:, None] * cdf[:, -1:]
    a = (cdf <= target).sum(axis=-1)
    return np.minimum(a, logp.shape[-1] - 1).astype(np.int64)


# Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11).
_PHILOX_M0 = np.uint64(0xD2511F53)
_PHILOX_M1 = np.uint64(0xCD9E8D57)
_PHILOX_W0 = np.uint32(0x9E3779B9)
_PHILOX_W1 = np.uint32(0xBB67AE85)


def philox4x32_10(counter: np.ndarray, key: np.ndarray) -> np.ndarray:
    """counter [...,4] uint32, key [...,2] uint32 -> [...,4] uint32."""
    c = np.array(counter, dtype=np.uint32, copy=True)
    k = np.array(key, dtype=np.uint32, copy=True)
    c, k = np.broadcast_arrays(c, k[..., [0, 1, 0, 1]])
    c = c.copy()
    k0 = k[..., 0].copy()
    k1 = k[..., 1].copy()
    mask32 = np.uint64(0xFFFFFFFF)
    with np.errstate(over="ignore"):
        for _ in range(10):
            p0 = _PHILOX_M0 * c[..., 0].astype(np.uint64)
            p1 = _PHILOX_M1 * c[..., 2].astype(np.uint64)
            hi0 = (p0 >> np.uint64(32)).astype(np.uint32)
            lo0 = (p0 & mask32).astype(np.uint32)
            hi1 = (p1 >> np.uint64(32)).astype(np.uint32)
            lo1 = (p1 & mask32).astype(np.uint32)
            n0 = hi1 ^ c[..., 1] ^ k0
            n1 = lo1
            n2 = hi0 ^ c[..., 3] ^ k1
            n3 = lo0
            c = np.stack([n0, n1, n2, n3], axis=-1)
            k0 = k0 + _PHILOX_W0
            k1 = k1 + _PHILOX_W1
    return c


def board_uniform(seed: int, offset: int, board_index: np.ndarray) -> np.ndarray:
    """The one uniform in [0,1) the engine draws for a board in a self-play step.

    Counter = (board_index lo, board_index hi, offset lo, offset hi), key = seed
    (lo, hi); u = (first output word >> 8) * 2^-24.  Keyed by the GLOBAL board
    index so that sharding boards over GPUs never changes a draw."""
    bi = np.asarray(board_index, dtype=np.uint64)
    ctr = np.stack([
        (bi & np.uint64(0xFFFFFFFF)).astype(np.uint32),
        (bi >> np.uint64(32)).astype(np.uint32),
        np.full(bi.shape, offset & 0xFFFFFFFF, dtype=np.uint32),
        np.full(bi.shape, (offset >> 32) & 0xFFFFFFFF, dtype=np.uint32),
    ], axis=-1)
    key = np.array([seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF], dtype=np.uint32)
    r = philox4x32_10(ctr, key)
    return (r[..., 0] >> np.uint32(8)).astype(np.float32) * np.float32(1.0 / 16777216.0)


# --------------------------------------------------------------------------------------
# D4 symmetries (bit-exact integer work)
# --------------------------------------------------------------------------------------


def symmetry_for_phase(phase: int) -> tuple[int, bool]:
    """connect6/train.py:216-219: phase 0..7 -> (k quarter turns, mirror)."""
    phase = int(phase) % 8
    return phase % 4, phase >= 4


def transform_boards(boards: np.ndarray, k: int, flip: bool) -> np.ndarray:
    """connect6/train.py:222-230: rot90 (counter-clockwise) k times on the last two
    axes, then mirror the columns."""
    out = np.rot90(boards, k=int(k) % 4, axes=(-2, -1))
    return out[..., ::-1] if flip else out


def transform_actions(actions: np.ndarray, n: int, k: int, flip: bool) -> np.ndarray:
    """connect6/train.py:233-252: canonical action index -> index in the view."""
    a = np.asarray(actions, dtype=np.int64)
    r, c = a // n, a % n
    k = int(k) % 4
    if k == 1:
        r, c = n - 1 - c, r
    elif k == 2:
        r, c = n - 1 - r, n - 1 - c
    elif k == 3:
        r, c = c, n - 1 - r
    if flip:
        c = n - 1 - c
    return r * n + c


def inverse_transform_actions(actions: np.ndarray, n: int, k: int, flip: bool) -> np.ndarray:
    """connect6/train.py:255-277: view action index -> canonical index."""
    a = np.asarray(actions, dtype=np.int64)
    r, c = a // n, a % n
    k = int(k) % 4
    if flip:
        c = n - 1 - c
    if k == 1:
        r, c = c, n - 1 - r
    elif k == 2:
        r, c = n - 1 - r, n - 1 - c
    elif k == 3:
        r, c = n - 1 - c, r
    return r * n + c


def d4_forward_table(n: int) -> np.ndarray:
    """[8, n*n] int32: table[p, a] = index in view p of canonical cell a."""
    a = np.arange(n * n)
    return np.stack([transform_actions(a, n, *symmetry_for_phase(p)) for p in range(8)]).astype(np.int32)


def oriented_forward(x: np.ndarray, orient: np.ndarray, params: dict, dtype=np.float64):
    """Per-board D4 inference: plane view -> CNN -> logits mapped back to canonical
    action indices (logits_canon[a] = logits_view[fwd(a)])."""
    x = np.asarray(x)
    B, _, n, _ = x.shape
    xv = np.empty_like(x)
    for p in range(8):
        sel = np.nonzero(np.asarray(orient) == p)[0]
        if sel.size:
            xv[sel] = transform_boards(x[sel], *symmetry_for_phase(p))
    logits_view, value = policy_value_forward(xv, params, dtype)
    table = d4_forward_table(n)
    logits = np.take_along_axis(logits_view, table[np.asarray(orient)].astype(np.int64), axis=1)
    return logits, value, logits_view


# --------------------------------------------------------------------------------------
# network input from raw boards
# --------------------------------------------------------------------------------------


def canonical_network_input(boards: np.ndarray, current_player: np.ndarray, stones_left: np.ndarray) -> np.ndarray:
    """connect6/vector_env.py:196-218: int8 boards [B,H,W] (+1/-1/0), player [B]
    (+1/-1), stones_left [B] -> float32 planes [B,3,H,W]."""
    boards = np.asarray(boards)
    player = np.asarray(current_player).reshape(-1, 1, 1)
    me = (boards == player).astype(np.float32)
    opp = (boards == -player).astype(np.float32)
    last = (np.asarray(stones_left) == 1).astype(np.float32).reshape(-1, 1, 1)
    last = np.broadcast_to(last, boards.shape)
    return np.stack([me, opp, last], axis=1)


# --------------------------------------------------------------------------------------
# bf16 emulation (for the tolerance budget only)
# --------------------------------------------------------------------------------------


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round float32 to the nearest bfloat16 (ties to even), returned as float32."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + np.uint64(0x7FFF) + ((u >> np.uint64(16)) & np.uint64(1))) >> np.uint64(16)) << np.uint64(16)
    return (r & np.uint64(0xFFFFFFFF)).astype(np.uint32).view(np.float32).reshape(np.shape(x))


def policy_value_forward_bf16_emulated(x: np.ndarray, params: dict):
    """The engine's bf16 numerics restated: bf16 weights and bf16 inter-layer
    activations, wide accumulation, bias+SiLU in full precision, heads computed
    from the unrounded last-layer output."""
    f = bf16_round(np.asarray(x, dtype=np.float32)).astype(np.float64)
    L = n_layers_of(params)
    for i in range(L):
        w = bf16_round(params[f"convs.{i}.weight"]).astype(np.float64)
        f = silu(conv2d_same(f, w, params[f"convs.{i}.bias"], np.float64))
        if i < L - 1:
            f = bf16_round(f.astype(np.float32)).astype(np.float64)
    wp = np.asarray(params["policy_output.weight"], dtype=np.float64).reshape(-1)
    wv = np.asarray(params["value_output.weight"], dtype=np.float64).reshape(-1)
    logits = np.einsum("c,bchw->bhw", wp, f).reshape(f.shape[0], -1) + float(np.asarray(params["policy_output.bias"]).reshape(()))
    vmap = np.einsum("c,bchw->bhw", wv, f) + float(np.asarray(params["value_output.bias"]).reshape(()))
    return logits, np.tanh(vmap.mean(axis=(-2, -1)))
