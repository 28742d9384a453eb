"""The oracle is pinned before it is trusted: every function is compared with fixtures that the
unmodified reference produced (tests/golden/make_golden.py) and with the relational identities
the reference's own tests assert."""
from __future__ import annotations

import hashlib

import numpy as np
import pytest
import torch

import c6_oracle as O
import torch_port as TP
from conftest import load_golden, params_from


def _state_hash(state: dict) -> str:
    h = hashlib.sha256()
    for k in sorted(state):
        h.update(k.encode())
        h.update(np.ascontiguousarray(state[k], dtype=np.float32).tobytes())
    return h.hexdigest()


def test_small_net_matches_reference_output():
    g = load_golden("small_net.npz")
    params = params_from(g)
    logits, value = O.policy_value_forward(g["x"], params)
    np.testing.assert_allclose(logits, g["logits"], atol=2e-5, rtol=1e-5)
    np.testing.assert_allclose(value, g["value"], atol=1e-6)
    tl, tv = TP.policy_value_forward(torch.from_numpy(g["x"]), {k: torch.from_numpy(v) for k, v in params.items()})
    np.testing.assert_allclose(tl.numpy(), g["logits"], atol=2e-5, rtol=1e-5)
    np.testing.assert_allclose(tv.numpy(), g["value"], atol=1e-6)


def test_default_net_seed42_matches_reference():
    """Weights come from this package's drop-in module with the reference's seed; their hash must
    equal the hash of the reference module's weights, then the oracle must reproduce the
    reference's logits and values on generated boards 0..5."""
    from connect6_b200.boards import generate_planes
    from connect6_b200.model import PolicyValueNet
    g = load_golden("default_net_seed42.npz")
    if str(g["torch_version"]) != torch.__version__:
        pytest.skip("fixture was generated with another torch version (RNG streams may differ)")
    torch.manual_seed(42)
    net = PolicyValueNet(board_size=19)
    state = {k: v.detach().numpy() for k, v in net.state_dict().items()}
    assert _state_hash(state) == str(g["weights_sha256"])
    x = generate_planes(0, 6)
    tl, tv = TP.policy_value_forward(torch.from_numpy(x), {k: torch.from_numpy(v) for k, v in state.items()})
    np.testing.assert_allclose(tl.numpy(), g["logits"], atol=1e-6)
    np.testing.assert_allclose(tv.numpy(), g["value"], atol=1e-6)
    logits, value = O.policy_value_forward(x[:2], state)   # numpy oracle: two boards keep it quick
    np.testing.assert_allclose(logits, g["logits"][:2], atol=1e-6)
    np.testing.assert_allclose(value, g["value"][:2], atol=1e-6)


def test_forward_rejects_bad_shapes_like_the_reference():
    g = load_golden("small_net.npz")
    with pytest.raises(ValueError):
        O.policy_value_forward(np.zeros((2, 4, 7, 7), np.float32), params_from(g))
    with pytest.raises(ValueError):
        O.policy_value_forward(np.zeros((3, 7, 7), np.float32), params_from(g))


def test_grouped_matches_reference_and_individual_models():
    g = load_golden("grouped_small.npz")
    plist = [params_from(g, f"w{i}::") for i in range(3)]
    logits, value = O.grouped_policy_value_forward(g["x"], plist)
    np.testing.assert_allclose(logits, g["logits"], atol=1e-5, rtol=1e-5)   # reference test's tolerance
    np.testing.assert_allclose(value, g["value"], atol=1e-6)
    np.testing.assert_allclose(O.grouped_policy_forward(g["x"], plist), logits, atol=0)
    with pytest.raises(ValueError):
        O.grouped_policy_forward(g["x"][:2], plist)


def test_d4_tables_bit_exact():
    g = load_golden("d4_tables.npz")
    for p in range(10):
        assert list(map(int, O.symmetry_for_phase(p))) == list(g["phases"][p])
    for n in (7, 19):
        a = np.arange(n * n)
        board = np.arange(n * n, dtype=np.int32).reshape(1, n, n)
        for p in range(8):
            k, flip = O.symmetry_for_phase(p)
            assert np.array_equal(O.transform_actions(a, n, k, flip), g[f"fwd{n}"][p])
            assert np.array_equal(O.inverse_transform_actions(a, n, k, flip), g[f"inv{n}"][p])
            view = O.transform_boards(board, k, flip).reshape(-1)
            assert np.array_equal(view, g[f"view{n}"][p])
            # identities the engine relies on
            assert np.array_equal(view, board.reshape(-1)[g[f"inv{n}"][p]])
            assert np.array_equal(g[f"inv{n}"][p][g[f"fwd{n}"][p]], a)
        assert np.array_equal(O.d4_forward_table(n), g[f"fwd{n}"])


def test_masking_and_log_softmax_match_reference():
    g = load_golden("masking.npz")
    masked = O.mask_logits(g["logits"], g["legal"])
    assert np.array_equal(masked, g["masked"])                      # bit-exact
    bf16_min = float(torch.finfo(torch.bfloat16).min)
    assert np.array_equal(O.mask_logits(O.bf16_round(g["logits"]), g["legal"], fill=bf16_min), g["masked_bf16"])
    for T, rows in ((1.0, 6), (0.5, 5), (2.0, 6)):
        ref = g[f"logp_T{T}"]
        got = O.masked_log_softmax(g["logits"][:rows], g["legal"][:rows], T)
        legal = g["legal"][:rows]
        np.testing.assert_allclose(got[legal], ref[legal], atol=2e-5, rtol=1e-6)
        assert np.all(np.exp(got[~legal & legal.any(axis=1, keepdims=True)]) == 0.0)
    # all-occupied board: the reference's normalised logits are 0 everywhere (log(361) is absorbed
    # by the -3.4e38 fill) while its probabilities stay uniform
    degenerate = O.masked_log_softmax(g["logits"][5:6], g["legal"][5:6], 1.0)
    assert np.array_equal(degenerate, g["logp_T1.0"][5:6]) and np.all(degenerate == 0.0)
    picks = O.sample_inverse_cdf(degenerate.repeat(4, 0), np.array([0.0, 0.25, 0.5, 0.999]))
    assert list(picks) == [0, 90, 180, 360]
    # log-prob of the reference's own sampled actions
    lp = O.masked_log_softmax(g["logits"][:4], g["legal"][:4], 1.0)
    acts = g["sampled_actions"]
    np.testing.assert_allclose(lp[np.arange(4), acts], g["sampled_logprob"], atol=2e-5)
    assert g["legal"][np.arange(4), acts].all()
    tp = TP.masked_log_softmax(torch.from_numpy(g["logits"]), torch.from_numpy(g["legal"]), 1.0).numpy()
    np.testing.assert_allclose(tp[g["legal"]], g["logp_T1.0"][g["legal"]], atol=1e-6)


def test_network_input_matches_reference():
    g = load_golden("network_input.npz")
    planes = O.canonical_network_input(g["boards"], g["player"], g["stones_left"])
    assert planes.dtype == np.float32 and np.array_equal(planes, g["planes"])
    legal = O.legal_from_planes(planes)
    assert np.array_equal(legal, (g["boards"] == 0).reshape(5, -1))


def test_philox_known_answers():
    """Known-answer vectors of Philox4x32-10 from the Random123 distribution (kat_vectors)."""
    kat = [
        ((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
        ((0xffffffff,) * 4, (0xffffffff,) * 2, (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
        ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0),
         (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1)),
    ]
    for ctr, key, want in kat:
        got = O.philox4x32_10(np.array(ctr, np.uint32), np.array(key, np.uint32))
        assert tuple(int(v) for v in got) == want
    u = O.board_uniform(1234, 7, np.arange(1000))
    assert u.dtype == np.float32 and (u >= 0).all() and (u < 1).all() and abs(u.mean() - 0.5) < 0.05


def test_inverse_cdf_draw():
    logp = np.log(np.array([[0.1, 0.0, 0.6, 0.3]]) + 1e-300)
    for u, want in ((0.0, 0), (0.0999, 0), (0.1001, 2), (0.6999, 2), (0.7001, 3), (0.99999, 3)):
        assert int(O.sample_inverse_cdf(logp, np.array([u]))[0]) == want


def test_oriented_forward_consistency():
    """logits_canon[a] == logits_view[fwd(a)] and the view of the input is what the net sees."""
    g = load_golden("small_net.npz")
    params = params_from(g)
    x = g["x"]
    orient = np.array([0, 3, 5, 6, 7], dtype=np.uint8)
    logits, value, logits_view = O.oriented_forward(x, orient, params)
    table = O.d4_forward_table(7)
    for b in range(5):
        k, flip = O.symmetry_for_phase(int(orient[b]))
        lv, vv = O.policy_value_forward(O.transform_boards(x[b:b + 1], k, flip), params)
        np.testing.assert_allclose(lv[0], logits_view[b], atol=1e-12)
        np.testing.assert_allclose(logits[b], lv[0][table[orient[b]]], atol=1e-12)
        np.testing.assert_allclose(value[b], vv[0], atol=1e-12)


def test_bf16_emulation_is_close_to_fp32():
    g = load_golden("small_net.npz")
    params = params_from(g)
    l_bf, v_bf = O.policy_value_forward_bf16_emulated(g["x"], params)
    assert np.abs(l_bf - g["logits"]).max() < 3e-2 * max(1.0, np.abs(g["logits"]).max())
    assert np.abs(v_bf - g["value"]).max() < 3e-2
    r = O.bf16_round(np.array([1.0, 1.00390625, 1.0 + 2 ** -9, 3.14159], np.float32))
    assert np.array_equal(r, torch.tensor([1.0, 1.00390625, 1.0 + 2 ** -9, 3.14159]).bfloat16().float().numpy())


def test_layer_backward_oracle_matches_reference_autograd():
    """The backward oracle against gradients recorded from loss.backward() through the reference's own network
    (a hook on one backbone layer: its input, the gradient at its output, the gradients it produced)."""
    import torch
    import torch_port as TP
    g = load_golden("layer_backward.npz")
    t = lambda k: torch.from_numpy(g[k])
    dx, dw, db = TP.layer_backward(t("x_in").double(), t("weight").double(), t("bias").double(), t("dy").double())
    for got, want in ((dx, g["dx"]), (dw, g["dw"]), (db, g["db"])):
        scale = np.abs(want).max()
        assert np.abs(got.numpy() - want).max() < 2e-6 * scale + 1e-12


def test_stack_backward_oracle_matches_reference_autograd():
    """The oracle for a run of layers (oracle/torch_port.py:stack_backward), driven by the head gradients that the
    recorded loss implies, against every backbone gradient recorded from loss.backward() through the reference's
    own network (tests/golden/network_backward.npz)."""
    import torch
    import torch_port as TP
    g = load_golden("network_backward.npz")
    params = {k[3:]: torch.from_numpy(g[k]).double() for k in g if k.startswith("w::")}
    x = torch.from_numpy(g["x"]).double()
    target = torch.from_numpy(g["target"])
    # stem forward, then the 3x3 layers as one stack; heads and loss differentiated by hand-written torch ops
    w0, b0 = params["convs.0.weight"], params["convs.0.bias"]
    a0 = torch.nn.functional.silu(torch.nn.functional.conv2d(x, w0, b0, padding=w0.shape[-1] // 2))
    L = len(g["kernels"])
    ws = [params[f"convs.{i}.weight"] for i in range(1, L)]
    bs = [params[f"convs.{i}.bias"] for i in range(1, L)]
    feats, _, _, _ = TP.stack_backward(a0, ws, bs, torch.zeros(a0.shape[0], ws[-1].shape[0], 9, 9, dtype=torch.float64))
    f = feats.clone().requires_grad_(True)
    logits = torch.nn.functional.conv2d(f, params["policy_output.weight"], params["policy_output.bias"]).flatten(1)
    value = torch.tanh(torch.nn.functional.conv2d(f, params["value_output.weight"], params["value_output.bias"]).mean(dim=(-2, -1))).squeeze(1)
    loss = torch.nn.functional.cross_entropy(logits, target) + 0.5 * (value - 0.25).pow(2).mean()
    assert abs(float(loss) - float(g["loss"])) < 1e-5
    loss.backward()
    _, da0, dws, dbs = TP.stack_backward(a0, ws, bs, f.grad)
    for i in range(1, L):
        for got, key in ((dws[i - 1], f"g::convs.{i}.weight"), (dbs[i - 1], f"g::convs.{i}.bias")):
            want = g[key]
            assert np.abs(got.numpy() - want).max() < 5e-6 * np.abs(want).max() + 1e-12, key


def test_ppo_loss_oracle_matches_reference_statements():
    """oracle/torch_port.py:ppo_loss against the reference's own loss statements (compiled out of connect6/train.py by
    tests/golden/make_golden.py and run on random network outputs): every loss component, both statistics and the
    gradients that loss.backward() hands to logits and values."""
    import torch
    import torch_port as TP
    g = load_golden("ppo_loss.npz")
    for case in range(int(g["ncases"])):
        p = f"c{case}_"
        t = lambda k: torch.from_numpy(g[p + k])
        temperature, clip_coef, value_coef, entropy_coef = (float(v) for v in g[p + "coefs"])
        r = TP.ppo_loss(t("logits"), t("legal"), t("actions"), t("old_logprob"), t("advantages"), t("returns"), t("values"),
                        temperature, clip_coef, value_coef, entropy_coef)
        got = np.array([float(r[k]) for k in ("loss", "policy_loss", "value_loss", "entropy", "approx_kl", "clipfrac")])
        assert np.abs(got - g[p + "stats"]).max() < 1e-6
        assert np.abs(r["dlogits"].numpy() - g[p + "dlogits"]).max() < 1e-8
        assert np.abs(r["dvalues"].numpy() - g[p + "dvalues"]).max() < 1e-8
