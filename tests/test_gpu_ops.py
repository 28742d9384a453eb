"""GPU tests of the sampling step and the small standalone operators (all through the C ABI)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import c6_oracle as O
from conftest import load_golden

pytestmark = pytest.mark.gpu


def _default_model(dev, precision="bf16"):
    from connect6_b200.model import PolicyValueNet
    torch.manual_seed(42)
    return PolicyValueNet(19, engine_precision=precision).to(dev).eval()


def _check_draws(masked: np.ndarray, legal: np.ndarray, actions: np.ndarray, logprob: np.ndarray, u: np.ndarray,
                 temperature: float):
    """Actions must be legal, log-probs must equal the oracle's log-softmax at the drawn action, and
    the draw must be the inverse-CDF pick for the board's Philox uniform (up to fp32 rounding of the
    running sum at a bin edge)."""
    B = masked.shape[0]
    assert legal[np.arange(B), actions].all()
    logp = O.masked_log_softmax(masked, legal, temperature)
    np.testing.assert_allclose(logprob, logp[np.arange(B), actions], atol=2e-4)
    want = O.sample_inverse_cdf(logp, u)
    cdf = np.cumsum(np.exp(logp), axis=1)
    edge = np.minimum(np.abs(cdf[np.arange(B), np.minimum(actions, want)] - u), 1.0)
    assert np.all((actions == want) | (edge < 1e-5)), "draw differs from the inverse-CDF pick away from a bin edge"


def test_selfplay_step_draws(cuda_device):
    from connect6_b200.boards import generate_planes
    m = _default_model(cuda_device)
    B, first, seed, offset = 512, 123456, 77, 5
    x = torch.from_numpy(generate_planes(first, B))
    xd = x.to(cuda_device)
    a, lp, v, masked = m.selfplay_step(xd, temperature=1.0, seed=seed, offset=offset, board_index0=first,
                                       want_logits=True)
    legal = O.legal_from_planes(x.numpy())
    u = O.board_uniform(seed, offset, first + np.arange(B)).astype(np.float64)
    _check_draws(masked.cpu().numpy(), legal, a.cpu().numpy(), lp.cpu().numpy(), u, 1.0)
    # determinism, and invariance under sharding: halves with their own board_index0 give the same draws
    a2, lp2, v2, _ = m.selfplay_step(xd, temperature=1.0, seed=seed, offset=offset, board_index0=first)
    assert torch.equal(a, a2) and torch.equal(lp, lp2) and torch.equal(v, v2)
    h = B // 2
    lo = m.selfplay_step(xd[:h], seed=seed, offset=offset, board_index0=first)
    hi = m.selfplay_step(xd[h:], seed=seed, offset=offset, board_index0=first + h)
    assert torch.equal(torch.cat([lo[0], hi[0]]), a) and torch.equal(torch.cat([lo[1], hi[1]]), lp)
    # another offset gives another stream
    a3 = m.selfplay_step(xd, seed=seed, offset=offset + 1, board_index0=first)[0]
    assert (a3 != a).float().mean().item() > 0.5
    # value equals the plain forward's value
    assert torch.equal(v, m.engine_for(cuda_device).forward(xd)[1])
    assert m.engine_for(cuda_device).status() == 0


def test_selfplay_step_with_orientation(cuda_device):
    from connect6_b200.boards import generate_planes
    m = _default_model(cuda_device)
    B = 128
    x = torch.from_numpy(generate_planes(999, B))
    orient = torch.from_numpy((np.arange(B) % 8).astype(np.uint8)).to(cuda_device)
    a, lp, v, masked = m.selfplay_step(x.to(cuda_device), seed=3, offset=9, orient=orient, inverse_map=True,
                                       want_logits=True)
    legal = O.legal_from_planes(x.numpy())          # canonical frame: actions index the caller's own board
    u = O.board_uniform(3, 9, np.arange(B)).astype(np.float64)
    _check_draws(masked.cpu().numpy(), legal, a.cpu().numpy(), lp.cpu().numpy(), u, 1.0)


@pytest.mark.parametrize("temperature", [1.0, 0.5, 2.0])
def test_sample_actions_matches_reference_distribution(cuda_device, temperature):
    """_sample_actions on the golden logits: log-probs equal the reference Categorical's."""
    from connect6_b200.selfplay import _sample_actions, _sample_actions_only
    g = load_golden("masking.npz")
    rows = 5 if temperature < 1 else 6
    logits = torch.from_numpy(g["logits"][:rows]).to(cuda_device)
    legal = torch.from_numpy(g["legal"][:rows]).to(cuda_device)
    a, lp = _sample_actions(logits, legal, temperature, seed=1, offset=0)
    ref = g[f"logp_T{temperature}"]
    an = a.cpu().numpy()
    np.testing.assert_allclose(lp.cpu().numpy(), ref[np.arange(rows), an], atol=2e-5, rtol=1e-5)
    lg = g["legal"][:rows]
    ok = lg[np.arange(rows), an] | ~lg.any(axis=1)        # an all-occupied board is uniform over all cells
    assert ok.all()
    assert an[4] == 17                                     # the single legal move
    assert torch.equal(_sample_actions_only(logits, legal, temperature, seed=1, offset=0), a)


def test_sample_frequencies(cuda_device):
    """Empirical frequencies of many draws from one distribution match softmax (chi-square)."""
    from connect6_b200.selfplay import _sample_actions_only
    rng = np.random.default_rng(0)
    A, N = 12, 200_000
    row = rng.normal(size=A).astype(np.float32)
    legal_row = np.ones(A, bool)
    legal_row[[2, 7]] = False
    logits = torch.from_numpy(np.tile(row, (N, 1))).to(cuda_device)
    legal = torch.from_numpy(np.tile(legal_row, (N, 1))).to(cuda_device)
    a = _sample_actions_only(logits, legal, 1.0, seed=9, offset=4).cpu().numpy()
    counts = np.bincount(a, minlength=A)
    p = np.exp(O.masked_log_softmax(row[None], legal_row[None], 1.0))[0]
    assert counts[[2, 7]].sum() == 0
    chi2 = (((counts - N * p) ** 2) / (N * p))[legal_row].sum()
    assert chi2 < 40.0, f"chi-square {chi2} with 9 degrees of freedom"


def test_mask_logits_bit_exact(cuda_device):
    from connect6_b200.model import mask_logits
    g = load_golden("masking.npz")
    out = mask_logits(torch.from_numpy(g["logits"]).to(cuda_device), torch.from_numpy(g["legal"]).to(cuda_device))
    assert np.array_equal(out.cpu().numpy(), g["masked"])
    bf = mask_logits(torch.from_numpy(g["logits"]).to(cuda_device).bfloat16(),
                     torch.from_numpy(g["legal"]).to(cuda_device))
    assert np.array_equal(bf.float().cpu().numpy(), g["masked_bf16"])


def test_d4_maps_bit_exact(cuda_device):
    from connect6_b200.selfplay import (_inverse_transform_actions, _symmetry_for_phase, _transform_actions,
                                        _transform_boards, transform_actions_per_board)
    g = load_golden("d4_tables.npz")
    for n in (7, 19):
        a = torch.arange(n * n, device=cuda_device)
        board = torch.arange(n * n, dtype=torch.int32).reshape(1, n, n)
        for p in range(8):
            k, flip = _symmetry_for_phase(p)
            assert [k, int(flip)] == list(g["phases"][p])
            assert np.array_equal(_transform_actions(a, n, k, flip).cpu().numpy(), g[f"fwd{n}"][p])
            assert np.array_equal(_inverse_transform_actions(a, n, k, flip).cpu().numpy(), g[f"inv{n}"][p])
            b8 = (board % 100).to(torch.int8).to(cuda_device)
            view = _transform_boards(b8, k, flip).cpu().numpy().reshape(-1)
            assert np.array_equal(view, (g[f"view{n}"][p] % 100).astype(np.int8))
    # per-board phases, round trip
    n, B = 19, 4096
    rng = np.random.default_rng(1)
    acts = torch.from_numpy(rng.integers(0, n * n, B)).to(cuda_device)
    ph = torch.from_numpy(rng.integers(0, 8, B).astype(np.uint8)).to(cuda_device)
    fwd = transform_actions_per_board(acts, n, ph)
    assert np.array_equal(fwd.cpu().numpy(), g["fwd19"][ph.cpu().numpy(), acts.cpu().numpy()])
    assert torch.equal(transform_actions_per_board(fwd, n, ph, inverse=True), acts)


def test_network_input_bit_exact(cuda_device):
    from connect6_b200.selfplay import canonical_network_input
    g = load_golden("network_input.npz")
    out = canonical_network_input(torch.from_numpy(g["boards"]).to(cuda_device),
                                  torch.from_numpy(g["player"]).to(cuda_device),
                                  torch.from_numpy(g["stones_left"]).to(cuda_device))
    assert out.dtype == torch.float32 and np.array_equal(out.cpu().numpy(), g["planes"])


def test_grouped_default_architecture(cuda_device):
    """G = 4 stacked default-architecture models, T = 96 boards each, bf16: every group matches its own
    fp64 oracle; logits AND values per group."""
    import torch_port as TP
    from connect6_b200.boards import generate_planes
    from connect6_b200.engine import Engine
    from connect6_b200.model import PolicyValueNet
    G, T = 4, 96
    states = []
    for g in range(G):
        torch.manual_seed(1000 + g)
        states.append({k: v.detach().clone() for k, v in PolicyValueNet(19).state_dict().items()})
    eng = Engine(cuda_device, 19, PolicyValueNet.DEFAULT_KERNELS, PolicyValueNet.DEFAULT_CHANNELS, G, "bf16")
    for g in range(G):
        eng.load_state_dict(states[g], group=g)
    x = torch.from_numpy(generate_planes(50_000, G * T)).reshape(G, T, 3, 19, 19)
    logits, value = eng.forward_grouped(x.to(cuda_device), want_value=True)
    for g in range(G):
        rl, rv = TP.policy_value_forward(x[g].double(), {k: v.double() for k, v in states[g].items()})
        dl = (logits[g].cpu().double() - rl).abs().max().item()
        assert dl < 3e-2 and dl < 0.12 * rl.std().item(), f"group {g}: {dl}"
        assert (value[g].cpu().double() - rv).abs().max().item() < 3e-2
    # another T re-bases the groups inside the workspace: results must not depend on history
    l40, _ = eng.forward_grouped(x[:, :40].contiguous().to(cuda_device))
    assert torch.equal(l40, logits[:, :40])
    # 5 boards per model take the direct stem (same sums, another order): equal within a fraction of the bf16 noise
    l5, _ = eng.forward_grouped(x[:, :5].contiguous().to(cuda_device))
    assert (l5 - logits[:, :5]).abs().max().item() < 0.05 * logits.std().item()
    l5b, _ = eng.forward_grouped(x[:, :5].contiguous().to(cuda_device))
    assert torch.equal(l5, l5b)
    l3, _ = eng.forward_grouped(x.to(cuda_device))
    assert torch.equal(l3, logits)
    assert eng.status() == 0


def test_host_step_pipeline_matches_direct_steps(cuda_device):
    """Pinned host planes in, pinned host results out, uploads overlapped: same results as direct calls."""
    from connect6_b200.boards import generate_planes
    from connect6_b200.hostpipe import HostStepPipeline
    m = _default_model(cuda_device)
    B = 96
    batches = [torch.from_numpy(generate_planes(1000 * i, B)).pin_memory() for i in range(4)]
    pipe = HostStepPipeline(m, B, cuda_device)
    pipe.submit(batches[0])
    for i in range(4):
        if i + 1 < 4:
            pipe.submit(batches[i + 1])
        a, lp, v = pipe.step(seed=5, offset=i, board_index0=1000 * i)
        da, dlp, dv, _ = m.selfplay_step(batches[i].to(cuda_device), seed=5, offset=i, board_index0=1000 * i)
        assert torch.equal(a, da.cpu()) and torch.equal(lp, dlp.cpu()) and torch.equal(v, dv.cpu())
    with pytest.raises(RuntimeError):
        pipe.step()
    pipe.submit(batches[0][:10])             # a smaller batch reuses the buffers
    a, lp, v = pipe.step(seed=5, offset=0, board_index0=0)
    assert a.shape == (10,)


def test_bounded_wait_expiry_is_reported_not_hung(cuda_device):
    """Failure detection without a fault: a wait that nothing satisfies runs out after its limit, the
    kernel returns, the status word says so, and the engine keeps working after the status is cleared."""
    from connect6_b200.boards import generate_planes
    m = _default_model(cuda_device)
    eng = m.engine_for(cuda_device)
    x = torch.from_numpy(generate_planes(0, 16)).to(cuda_device)
    before = eng.forward(x)
    assert eng.status() == 0
    eng.expire_wait_selftest()
    # first waiter: its limit ran out (bit 0); second waiter: left on the abort flag the first raised (bit 1)
    with pytest.raises(RuntimeError, match="0x3: a bounded wait"):
        eng.status()
    eng.clear_status()
    assert eng.status() == 0
    after = eng.forward(x)
    assert torch.equal(before[0], after[0]) and torch.equal(before[1], after[1])


@pytest.mark.parametrize("precision", ["bf16", "fp32"])
def test_step_from_raw_boards_equals_planes_path(cuda_device, precision):
    """int8 environment state (+ gather index, + orientation) gives exactly what the plane-fed step gives."""
    from connect6_b200.selfplay import canonical_network_input
    m = _default_model(cuda_device, precision)
    rng = np.random.default_rng(4)
    E, B = 300, 128
    boards = torch.from_numpy(rng.choice([-1, 0, 0, 0, 1], size=(E, 19, 19)).astype(np.int8)).to(cuda_device)
    player = torch.from_numpy(rng.choice([-1, 1], size=E).astype(np.int8)).to(cuda_device)
    stones = torch.from_numpy(rng.choice([1, 2], size=E).astype(np.int8)).to(cuda_device)
    index = torch.from_numpy(rng.permutation(E)[:B].astype(np.int64)).to(cuda_device)
    orient = torch.from_numpy((np.arange(B) % 8).astype(np.uint8)).to(cuda_device)
    planes = canonical_network_input(boards, player, stones)[index]
    for kw in (dict(), dict(orient=orient, inverse_map=True)):
        want = m.selfplay_step(planes, seed=21, offset=2, board_index0=50, want_logits=True, **kw)
        got = m.selfplay_step_from_boards(boards, player, stones, index, seed=21, offset=2, board_index0=50,
                                          want_logits=True, **kw)
        for w, g in zip(want, got):
            assert torch.equal(w, g)
    whole = m.selfplay_step_from_boards(boards, player, stones, seed=1, offset=1)
    ref = m.selfplay_step(canonical_network_input(boards, player, stones), seed=1, offset=1)
    assert torch.equal(whole[0], ref[0]) and torch.equal(whole[2], ref[2])


def test_fp32_engines_of_different_sizes_share_the_kernel(cuda_device):
    """Two fp32-mode engines in one process (e.g. two architectures in an evaluation run): creating the
    small one must not shrink the dynamic shared memory the default network's 23x23 stem needs."""
    from connect6_b200 import _lib as L
    from connect6_b200.boards import generate_planes
    from connect6_b200.engine import Engine
    from connect6_b200.model import PolicyValueNet
    big = _default_model(cuda_device, "fp32")
    x = torch.from_numpy(generate_planes(0, 4)).to(cuda_device)
    with torch.inference_mode():
        before = big(x)
    torch.manual_seed(1)
    small = PolicyValueNet(5, [3, 3], [8, 8], engine_precision="fp32").to(cuda_device).eval()
    with torch.inference_mode():
        small(torch.zeros(2, 3, 5, 5, device=cuda_device))
        after = big(x)
    assert torch.equal(before[0], after[0]) and torch.equal(before[1], after[1])
    # the entry point that works out of the library's fixed scratch launches the same kernel
    eng = big.engine_for(cuda_device)
    logits = torch.empty((4, 361), device=cuda_device)
    value = torch.empty((4,), device=cuda_device)
    with torch.cuda.device(cuda_device):
        rc = L.load().c6_forward_noalloc(eng._h, x.data_ptr(), L.C6_X_F32, 4, None, logits.data_ptr(), value.data_ptr(), 0,
                                         torch.cuda.current_stream(cuda_device).cuda_stream)
    assert rc == L.C6_OK, L.last_error(eng._h)
    assert torch.allclose(logits, before[0], atol=1e-6, rtol=0)
    assert eng.status() == 0


def test_engine_rejects_misshapen_inputs_and_flags_stale_indices(cuda_device):
    """The kernels index their inputs unchecked, so shapes are validated on the host; the values of a
    gather index stay on the device, where an entry outside the environments is skipped (that board is
    evaluated as empty) and reported through the status word."""
    m = _default_model(cuda_device)
    eng = m.engine_for(cuda_device)
    dev = cuda_device
    for bad in (torch.zeros(2, 3, 19, 18, device=dev), torch.zeros(2, 4, 19, 19, device=dev), torch.zeros(3, 19, 19, device=dev)):
        with pytest.raises(ValueError):
            eng.forward(bad)
        with pytest.raises(ValueError):
            eng.forward_step(bad)
    boards = torch.zeros(6, 19, 19, dtype=torch.int8, device=dev)
    player = torch.ones(6, dtype=torch.int8, device=dev)
    stones = torch.ones(6, dtype=torch.int8, device=dev)
    with pytest.raises(ValueError):
        eng.forward_step_boards(boards[:, :18], player, stones)
    with pytest.raises(ValueError):
        eng.forward_step_boards(boards, player[:5], stones)
    with pytest.raises(ValueError):
        eng.forward_step_boards(boards, player, stones[:2])
    with pytest.raises(ValueError):
        eng.forward_step_boards(boards, player, stones, torch.zeros(2, 2, dtype=torch.int64, device=dev))
    boards[2, 3, 4] = 1
    good = eng.forward_step_boards(boards, player, stones, torch.tensor([2, 0, 5], device=dev), seed=9, want_logits=True)
    assert eng.status() == 0
    stale = eng.forward_step_boards(boards, player, stones, torch.tensor([2, 6, -1], device=dev), seed=9, want_logits=True)
    with pytest.raises(RuntimeError, match="gather index"):
        eng.status()
    eng.clear_status()
    assert torch.equal(stale[3][0], good[3][0])                 # the valid entry is unaffected
    zero = eng.forward(torch.zeros(1, 3, 19, 19, device=dev))[0][0]
    assert torch.equal(stale[3][1], zero) and torch.equal(stale[3][2], zero)   # skipped entries: all-zero planes
    assert eng.status() == 0


def test_default_sampler_stream_follows_torch_seed(cuda_device):
    """The drop-in samplers called with the reference's signature draw from a stream keyed by
    torch.initial_seed(): reseeding reproduces a run, another seed gives other draws."""
    from connect6_b200 import selfplay as S
    logits = torch.zeros(512, 361, device=cuda_device)
    legal = torch.ones(512, 361, dtype=torch.bool, device=cuda_device)

    def draw(seed):
        torch.manual_seed(seed)
        S.set_seed(None)
        return [S._sample_actions(logits, legal, 1.0)[0] for _ in range(2)]

    a, b, c = draw(7), draw(7), draw(8)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    assert not torch.equal(a[0], a[1])                          # the call counter advances the stream
    assert not torch.equal(a[0], c[0])
    S.set_seed(123, board_index0=0)
    d = S._sample_actions_only(logits, legal, 1.0)
    S.set_seed(123, board_index0=512)
    e = S._sample_actions_only(logits, legal, 1.0)
    assert not torch.equal(d, e)
    S.set_seed(None)
