"""GPU tests at the benchmark configurations' own shapes (BASELINE configs 3, 4 and 5).

Small slices are compared with the oracle; the full sizes are checked through size-independent
properties: a fused path must equal the same result assembled from simpler engine calls, bit for
bit (both sides run the same arithmetic), masks and index maps must be exact.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

import c6_oracle as O
import torch_port as TP

pytestmark = pytest.mark.gpu

WIDE_CHANNELS = (64, 64, 128, 128, 128, 192, 192, 192)
KERNELS = (23, 3, 3, 3, 3, 3, 3, 3)


def _state(seed, channels=None):
    from connect6_b200.model import PolicyValueNet
    torch.manual_seed(seed)
    m = PolicyValueNet(19, KERNELS, channels)
    return {k: v.detach().clone() for k, v in m.state_dict().items()}


def test_config5_widened_network_against_oracle(cuda_device):
    """Channels [64,64,128,128,128,192,192,192]: weights no longer fit shared memory (streamed with the
    activation stages), N = 192 uses two TMEM accumulators, boards drawn with up to 200 stones."""
    from connect6_b200.boards import generate_planes
    from connect6_b200.engine import Engine
    state = _state(5, WIDE_CHANNELS)
    eng = Engine(cuda_device, 19, KERNELS, WIDE_CHANNELS, 1, "bf16")
    eng.load_state_dict(state)
    x = torch.from_numpy(generate_planes(0, 160, max_stones=200))
    rl, rv = TP.policy_value_forward(x.double(), {k: v.double() for k, v in state.items()})
    f = x.double()
    for i in range(8):
        w, b = state[f"convs.{i}.weight"].double(), state[f"convs.{i}.bias"].double()
        f = torch.nn.functional.silu(torch.nn.functional.conv2d(f, w, b, padding=w.shape[-1] // 2))
        if i in (0, 1, 4, 7):
            got = eng.layer_output(x.to(cuda_device), i).cpu().double()
            err = (got - f).abs().max().item() / f.abs().max().item()
            assert err < 2e-2, f"layer {i}: relative error {err}"
    logits, value = eng.forward(x.to(cuda_device), mask=True)
    legal = O.legal_from_planes(x.numpy())
    lg = logits.cpu().numpy()
    assert np.array_equal(lg == O.FP32_MIN, ~legal)
    dl = np.abs(lg - rl.numpy())[legal].max()
    assert dl < 3e-2 and dl < 0.12 * rl.std().item()
    assert (value.cpu().double() - rv).abs().max().item() < 3e-2
    assert eng.status() == 0


def test_config5_full_batch_properties(cuda_device):
    """B = 32768 boards of the widened network in 4 internal passes: equal to the same boards run in
    separate calls, draws legal and reproducible."""
    from connect6_b200.boards import generate_planes
    from connect6_b200.engine import Engine
    state = _state(5, WIDE_CHANNELS)
    eng = Engine(cuda_device, 19, KERNELS, WIDE_CHANNELS, 1, "bf16")
    eng.load_state_dict(state)
    B = 32768
    x = torch.from_numpy(generate_planes(0, B, max_stones=200)).to(cuda_device)
    a, lp, v, _ = eng.forward_step(x, seed=11, offset=3)
    legal = ((x[:, 0] == 0) & (x[:, 1] == 0)).reshape(B, -1)
    assert bool(legal.gather(1, a[:, None]).all())
    for lo in (0, 8192 * 2 + 100, B - 777):
        hi = min(B, lo + 777)
        a2, lp2, v2, _ = eng.forward_step(x[lo:hi], seed=11, offset=3, board_index0=lo)
        assert torch.equal(a2, a[lo:hi]) and torch.equal(lp2, lp[lo:hi]) and torch.equal(v2, v[lo:hi])
    assert eng.status() == 0


def test_config4_d4_inference_65536_boards(cuda_device):
    """65536 boards, orientation i mod 8, logits mapped back to canonical indices: must equal (bit for
    bit) transforming the planes up front, running the plain forward and permuting with the oracle's
    index tables; masks exact."""
    from connect6_b200.boards import generate_planes
    from connect6_b200.engine import Engine
    from connect6_b200.model import PolicyValueNet
    state = _state(42)
    eng = Engine(cuda_device, 19, KERNELS, PolicyValueNet.DEFAULT_CHANNELS, 1, "bf16")
    eng.load_state_dict(state)
    B = 65536
    xh = generate_planes(0, B)
    orient = (np.arange(B) % 8).astype(np.uint8)
    x = torch.from_numpy(xh).to(cuda_device)
    od = torch.from_numpy(orient).to(cuda_device)
    logits, value = eng.forward(x, od, mask=True, inverse_map=True)
    # reference route inside the engine: explicit views, plain forward
    xv = np.empty_like(xh)
    for p in range(8):
        xv[p::8] = O.transform_boards(xh[p::8], *O.symmetry_for_phase(p))
    lv, vv = eng.forward(torch.from_numpy(xv).to(cuda_device), mask=False)
    table = torch.from_numpy(O.d4_forward_table(19).astype(np.int64)).to(cuda_device)
    canon = torch.gather(lv, 1, table[od.long()])
    legal = ((x[:, 0] == 0) & (x[:, 1] == 0)).reshape(B, -1)
    assert torch.equal(logits == O.FP32_MIN, ~legal)
    assert torch.equal(torch.where(legal, logits, torch.zeros_like(logits)), torch.where(legal, canon, torch.zeros_like(canon)))
    assert torch.equal(value, vv)
    assert eng.status() == 0


def test_config3_grouped_16x512(cuda_device):
    """G = 16 stacked checkpoints x 512 boards: every group equals a single-model engine with that
    group's weights on that group's boards, logits and values, bit for bit."""
    from connect6_b200.boards import generate_planes
    from connect6_b200.engine import Engine
    from connect6_b200.model import PolicyValueNet
    G, T = 16, 512
    states = [_state(1000 + g) for g in range(G)]
    eng = Engine(cuda_device, 19, KERNELS, PolicyValueNet.DEFAULT_CHANNELS, G, "bf16")
    for g in range(G):
        eng.load_state_dict(states[g], group=g)
    x = torch.from_numpy(generate_planes(0, G * T)).reshape(G, T, 3, 19, 19).to(cuda_device)
    logits, value = eng.forward_grouped(x, want_value=True)
    single = Engine(cuda_device, 19, KERNELS, PolicyValueNet.DEFAULT_CHANNELS, 1, "bf16")
    for g in (0, 7, 15):
        single.load_state_dict(states[g])
        l1, v1 = single.forward(x[g])
        assert torch.equal(l1, logits[g]) and torch.equal(v1, value[g])
    rl, rv = TP.policy_value_forward(x[3, :32].cpu().double(), {k: v.double() for k, v in states[3].items()})
    assert (logits[3, :32].cpu().double() - rl).abs().max().item() < 0.12 * rl.std().item()
    # the training shape of the reference: many models, few tables each (G = 16 here, T = 4)
    # (4 boards per model take the direct stem, 512 the stem GEMM: same sums in another order)
    l4, _ = eng.forward_grouped(x[:, :4].contiguous())
    assert (l4 - logits[:, :4]).abs().max().item() < 0.05 * rl.std().item()
    assert eng.status() == 0 and single.status() == 0


def test_training_ensemble_128x4(cuda_device, monkeypatch):
    """The ensemble shape the reference trains against (connect6/history.py:276-303 with 128 stacked
    opponents and 4 tables each): every sampled group equals a single-model engine bit for bit (the single
    engine is told to take the direct stem too, which by default only many-model engines do)."""
    from connect6_b200.boards import generate_planes
    from connect6_b200.engine import Engine
    from connect6_b200.model import PolicyValueNet
    G, T = 128, 4
    states = [_state(2000 + g) for g in range(G)]
    eng = Engine(cuda_device, 19, KERNELS, PolicyValueNet.DEFAULT_CHANNELS, G, "bf16")
    for g in range(G):
        eng.load_state_dict(states[g], group=g)
    # with 4 boards per model the first layer runs straight from each model's own filter: the engine holds
    # about 1 MB per model (16-bit weights, the fp32 stem filter), not the 27 MB per model of the stem GEMM's
    # expanded operand
    assert eng.device_bytes < 150e6, eng.device_bytes
    x = torch.from_numpy(generate_planes(0, G * T)).reshape(G, T, 3, 19, 19).to(cuda_device)
    logits, value = eng.forward_grouped(x, want_value=True)
    assert eng.device_bytes < 260e6, eng.device_bytes           # + activation workspace for 512 boards
    monkeypatch.setenv("C6_STEM_DIRECT_GROUPS", "1")
    single = Engine(cuda_device, 19, KERNELS, PolicyValueNet.DEFAULT_CHANNELS, 1, "bf16")
    monkeypatch.delenv("C6_STEM_DIRECT_GROUPS")
    for g in (0, 63, 127):
        single.load_state_dict(states[g])
        l1, v1 = single.forward(x[g])
        assert torch.equal(l1, logits[g]) and torch.equal(v1, value[g])
        rl, rv = TP.policy_value_forward(x[g].cpu().double(), {k: v.double() for k, v in states[g].items()})
        assert (logits[g].cpu().double() - rl).abs().max().item() < 0.12 * rl.std().item()
        assert (value[g].cpu().double() - rv).abs().max().item() < 3e-2
    assert eng.status() == 0 and single.status() == 0


@pytest.mark.parametrize("precision", ["bf16", "f16"])
def test_direct_stem_against_gemm_stem_and_oracle(cuda_device, precision, monkeypatch):
    """Calls of at most 32 boards per weight set may take the direct stem (implicit GEMM from the filter;
    the default for engines with several weight sets, forced here for a single model), larger ones the
    Toeplitz stem GEMM.  Both against the oracle's first layer and against each other, with per-board
    orientation and a third plane that is not constant; the expanded operand of the stem GEMM is only
    allocated once a call needs it."""
    from connect6_b200.boards import generate_planes
    from connect6_b200.engine import Engine
    from connect6_b200.model import PolicyValueNet
    state = _state(42)
    chans = PolicyValueNet.DEFAULT_CHANNELS
    monkeypatch.setenv("C6_STEM_DIRECT_GROUPS", "1")
    direct = Engine(cuda_device, 19, KERNELS, chans, 1, precision)
    direct.load_state_dict(state)
    monkeypatch.delenv("C6_STEM_DIRECT_GROUPS")
    monkeypatch.setenv("C6_STEM_DIRECT_MAX", "0")
    gemm = Engine(cuda_device, 19, KERNELS, chans, 1, precision)
    gemm.load_state_dict(state)
    monkeypatch.delenv("C6_STEM_DIRECT_MAX")
    x = torch.from_numpy(generate_planes(300, 29))
    x[5:9, 2] += 0.25 * torch.randn(4, 19, 19).round()             # third plane not constant on some boards
    orient = torch.from_numpy((np.arange(29) % 8).astype(np.uint8)).to(cuda_device)
    tol = 1e-2 if precision == "bf16" else 2e-3
    for od in (None, orient):
        xv = x.numpy().copy()
        if od is not None:
            for b in range(29):
                xv[b] = O.transform_boards(x.numpy()[b], *O.symmetry_for_phase(b % 8))
        w, bias = state["convs.0.weight"].double(), state["convs.0.bias"].double()
        want = torch.nn.functional.silu(torch.nn.functional.conv2d(torch.from_numpy(xv).double(), w, bias, padding=11))
        a = direct.layer_output(x.to(cuda_device), 0, od).cpu().double()
        b = gemm.layer_output(x.to(cuda_device), 0, od).cpu().double()
        scale = want.abs().max().item()
        assert (a - want).abs().max().item() / scale < tol
        assert (b - want).abs().max().item() / scale < tol
        assert (a - b).abs().max().item() / scale < tol
    rl, rv = TP.policy_value_forward(x.double(), {k: v.double() for k, v in state.items()})
    for eng in (direct, gemm):
        logits, value = eng.forward(x.to(cuda_device))
        assert (logits.cpu().double() - rl).abs().max().item() < 0.12 * rl.std().item()
        assert (value.cpu().double() - rv).abs().max().item() < 3e-2
    # a 33-board pass is the stem GEMM in both engines: bit-identical, and it is what allocates the operand
    before = direct.device_bytes
    x33 = torch.from_numpy(generate_planes(0, 33)).to(cuda_device)
    l1, v1 = direct.forward(x33)
    l2, v2 = gemm.forward(x33)
    assert torch.equal(l1, l2) and torch.equal(v1, v2)
    assert direct.device_bytes - before > 20e6
    # raw int8 board input with a gather index through the direct stem equals the plane-fed step
    from connect6_b200.selfplay import canonical_network_input
    rng = np.random.default_rng(2)
    boards = torch.from_numpy(rng.choice([-1, 0, 0, 1], size=(40, 19, 19)).astype(np.int8)).to(cuda_device)
    player = torch.from_numpy(rng.choice([-1, 1], size=40).astype(np.int8)).to(cuda_device)
    stones = torch.from_numpy(rng.choice([1, 2], size=40).astype(np.int8)).to(cuda_device)
    index = torch.from_numpy(rng.permutation(40)[:17].astype(np.int64)).to(cuda_device)
    planes = canonical_network_input(boards, player, stones)[index]
    want = direct.forward_step(planes, seed=4, offset=1, want_logits=True)
    got = direct.forward_step_boards(boards, player, stones, index, seed=4, offset=1, want_logits=True)
    for w_, g_ in zip(want, got):
        assert torch.equal(w_, g_)
    assert direct.status() == 0 and gemm.status() == 0


@pytest.mark.parametrize("channels,kernels", [((96, 32), (23, 3)), ((160, 64, 32), (23, 3, 3)), ((256, 32), (23, 1))])
def test_stem_widths_against_oracle(cuda_device, channels, kernels):
    """Stem widths that change the tile shape of the Toeplitz GEMM (2 cells x 96 channels, 1 cell x 160,
    1 cell x 256 per tile; the epilogue warps then own 6, 5 and 8 pieces each), both with a constant
    third plane (short product) and with a varying one (full product)."""
    from connect6_b200.boards import generate_planes
    from connect6_b200.engine import Engine
    from connect6_b200.model import PolicyValueNet
    torch.manual_seed(11)
    m = PolicyValueNet(19, list(kernels), list(channels))
    with torch.no_grad():
        for p in m.parameters():
            if p.ndim == 1:
                p.uniform_(-0.2, 0.2)
    state = {k: v.detach().clone() for k, v in m.state_dict().items()}
    eng = Engine(cuda_device, 19, kernels, channels, 1, "bf16")
    eng.load_state_dict(state)
    x = torch.from_numpy(generate_planes(40, 130))
    xv = x.clone()
    xv[:, 2] += 0.125 * torch.randn(130, 19, 19).round()            # third plane no longer constant
    for inp in (x, xv):
        w, b = state["convs.0.weight"].double(), state["convs.0.bias"].double()
        want = torch.nn.functional.silu(torch.nn.functional.conv2d(inp.double(), w, b, padding=kernels[0] // 2))
        got = eng.layer_output(inp.to(cuda_device), 0).cpu().double()
        assert got.shape == want.shape
        err = (got - want).abs().max().item() / want.abs().max().item()
        assert err < 1e-2, f"stem {channels[0]} channels: relative error {err}"
        rl, rv = TP.policy_value_forward(inp.double(), {k: v.double() for k, v in state.items()})
        logits, value = eng.forward(inp.to(cuda_device))
        assert (logits.cpu().double() - rl).abs().max().item() < max(3e-2, 0.12 * rl.std().item())
        assert (value.cpu().double() - rv).abs().max().item() < 3e-2
    assert eng.status() == 0


def _sharded_rank(rank: int, world: int, port: int, total: int, out_dir: str, n_gpus: int) -> None:
    """One rank of the sharded D4 inference: its contiguous range of the global board index, results to disk."""
    import os
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    sys.path.insert(0, str(root))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank % n_gpus))
    from connect6_b200 import shard
    from connect6_b200.boards import generate_planes
    from connect6_b200.engine import Engine
    from connect6_b200.model import PolicyValueNet
    # ranks on distinct GPUs talk NCCL; two ranks sharing the one GPU of a small box reduce over gloo
    shard.init_from_env(backend="nccl" if n_gpus >= world else "gloo")
    dev = torch.device("cuda", rank % n_gpus)
    torch.cuda.set_device(dev)
    torch.manual_seed(42)
    state = {k: v.detach().clone() for k, v in PolicyValueNet(19).state_dict().items()}
    eng = Engine(dev, 19, KERNELS, PolicyValueNet.DEFAULT_CHANNELS, 1, "bf16")
    eng.load_state_dict(state)
    lo, hi = shard.shard_range(total, rank, world)
    x = torch.from_numpy(generate_planes(lo, hi - lo)).to(dev)
    orient = torch.from_numpy((np.arange(lo, hi) % 8).astype(np.uint8)).to(dev)
    logits, value = eng.forward(x, orient, mask=True, inverse_map=True)
    action, logprob, _, _ = eng.forward_step(x, seed=0xC6, offset=5, board_index0=lo, orient=orient, inverse_map=True)
    stats = torch.zeros(9, dtype=torch.int64, device=dev if n_gpus >= world else "cpu")
    stats[0] = hi - lo
    stats[4] = int(action.sum())
    shard.reduce_rollout_stats(stats)
    assert eng.status() == 0
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), logits=logits.cpu().numpy(), value=value.cpu().numpy(),
             action=action.cpu().numpy(), logprob=logprob.cpu().numpy(), stats=stats.cpu().numpy(), lo=lo, hi=hi)
    import torch.distributed as dist
    dist.destroy_process_group()


def test_two_rank_sharded_d4_inference_equals_one_rank(cuda_device, tmp_path):
    """BASELINE config 4's sharding rule on two ranks (two GPUs where the box has them, else both ranks on
    the one GPU): boards are cut by global index, orientation and random stream are keyed by that index,
    so the concatenated shards equal the unsharded run bit for bit; the statistics all-reduce sums."""
    import socket
    import torch.multiprocessing as mp
    from connect6_b200.boards import generate_planes
    from connect6_b200.engine import Engine
    from connect6_b200.model import PolicyValueNet
    total, world = 5001, 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_sharded_rank, args=(world, port, total, str(tmp_path), torch.cuda.device_count()), nprocs=world, join=True)
    torch.manual_seed(42)
    state = {k: v.detach().clone() for k, v in PolicyValueNet(19).state_dict().items()}
    eng = Engine(cuda_device, 19, KERNELS, PolicyValueNet.DEFAULT_CHANNELS, 1, "bf16")
    eng.load_state_dict(state)
    x = torch.from_numpy(generate_planes(0, total)).to(cuda_device)
    orient = torch.from_numpy((np.arange(total) % 8).astype(np.uint8)).to(cuda_device)
    logits, value = eng.forward(x, orient, mask=True, inverse_map=True)
    action, logprob, _, _ = eng.forward_step(x, seed=0xC6, offset=5, board_index0=0, orient=orient, inverse_map=True)
    parts = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    assert parts[0]["lo"] == 0 and parts[0]["hi"] == parts[1]["lo"] and parts[1]["hi"] == total
    for key, whole in (("logits", logits), ("value", value), ("action", action), ("logprob", logprob)):
        got = np.concatenate([p[key] for p in parts])
        assert np.array_equal(got, whole.cpu().numpy()), key
    for p in parts:
        assert p["stats"][0] == total and p["stats"][4] == int(action.sum())
