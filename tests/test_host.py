"""CPU tests: host-side logic of the drop-ins, the board generator and the C-ABI library surface."""
from __future__ import annotations

import ctypes as C
import re

import numpy as np
import pytest
import torch

from conftest import ROOT


def test_library_exports_every_declared_symbol(engine_lib):
    """Every function declared in include/*.h is exported and bound; no compute calls."""
    from connect6_b200 import _lib
    headers = sorted((ROOT / "include").glob("*.h"))
    assert [h.name for h in headers] == ["c6_debug.h", "c6_engine.h", "c6_env.h", "c6_train.h"]
    header = "\n".join(h.read_text() for h in headers)
    declared = set(re.findall(r"\b(c6_[a-z_0-9]+)\s*\(", header))
    assert declared, "no declarations parsed"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    for name in declared:
        assert hasattr(engine_lib, name)
    assert engine_lib.c6_version() >= 10000
    assert _lib.last_error(None) == "" or isinstance(_lib.last_error(None), str)


def test_create_rejects_bad_descriptors_without_a_gpu(engine_lib):
    from connect6_b200 import _lib
    h = C.c_void_p()
    d = _lib.C6Desc()
    d.board_size, d.n_layers, d.groups, d.precision = 19, 2, 1, 0
    d.kernels[0], d.kernels[1], d.channels[0], d.channels[1] = 4, 3, 8, 8       # even kernel
    assert engine_lib.c6_create(C.byref(d), C.byref(h)) == _lib.C6_ERR_ARG
    assert "odd" in _lib.last_error(None)
    d.kernels[0] = 3
    d.n_layers = 0
    assert engine_lib.c6_create(C.byref(d), C.byref(h)) == _lib.C6_ERR_ARG
    d.n_layers = 2
    d.channels[1] = 0
    assert engine_lib.c6_create(C.byref(d), C.byref(h)) == _lib.C6_ERR_ARG
    d.channels[1] = 8
    d.groups = 0
    assert engine_lib.c6_create(C.byref(d), C.byref(h)) == _lib.C6_ERR_ARG
    assert engine_lib.c6_create(None, C.byref(h)) == _lib.C6_ERR_ARG
    if not torch.cuda.is_available():
        d.groups = 1
        assert engine_lib.c6_create(C.byref(d), C.byref(h)) == _lib.C6_ERR_CUDA   # no device: loud, no fallback
        assert "no CPU path" in _lib.last_error(None)


def test_model_surface_matches_reference():
    from connect6_b200.model import PolicyValueNet, build_model
    m = PolicyValueNet(board_size=19)
    assert m.receptive_field == 37 and m.action_size == 361 and m.input_channels == 3
    assert m.kernels == (23, 3, 3, 3, 3, 3, 3, 3) and m.channels == (32, 32, 64, 64, 64, 96, 96, 96)
    sd = m.state_dict()
    assert len(sd) == 20 and sum(v.numel() for v in sd.values()) == 374_082
    assert tuple(sd["convs.0.weight"].shape) == (32, 3, 23, 23)
    assert tuple(sd["policy_output.weight"].shape) == (1, 96, 1, 1) and tuple(sd["value_output.bias"].shape) == (1,)
    cfg = {"architecture_version": 4, "kernels": [23, 3, 3, 3, 3, 3, 3, 3],
           "channels": [32, 32, 64, 64, 64, 96, 96, 96], "compile": False, "compile_mode": "default"}
    b = build_model(cfg, 19)
    assert [c.kernel_size[0] for c in b.convs] == cfg["kernels"]
    assert [c.out_channels for c in b.convs] == cfg["channels"]
    assert b.convs[0].in_channels == 3 and b.policy_output.in_channels == 96 and b.policy_output.out_channels == 1
    for bad in (dict(kernels=[3, 3], channels=[8]), dict(kernels=[], channels=[]), dict(kernels=[4], channels=[8]),
                dict(kernels=[3], channels=[0])):
        with pytest.raises(ValueError):
            PolicyValueNet(19, **bad)


def test_inference_has_no_cpu_path_but_training_forward_works():
    from connect6_b200.model import PolicyValueNet
    m = PolicyValueNet(7, [3, 3], [8, 8])
    x = torch.zeros(2, 3, 7, 7)
    with pytest.raises(ValueError):
        m(torch.zeros(2, 3, 7, 6))
    with torch.inference_mode():
        with pytest.raises(RuntimeError):
            m(x)
    logits, value = m(x)                      # grad enabled: the torch modules own the parameters
    assert logits.shape == (2, 49) and value.shape == (2,) and logits.requires_grad
    (logits.sum() + value.sum()).backward()
    assert m.convs[0].weight.grad is not None
    import copy
    c = copy.deepcopy(m)
    assert c._engines == {} and torch.equal(c.convs[1].weight, m.convs[1].weight)


def test_mask_logits_on_cpu_tensors_follows_dtype_min():
    from connect6_b200.model import mask_logits
    logits = torch.tensor([[1.0, 2.0, 3.0]])
    legal = torch.tensor([[True, False, True]])
    assert mask_logits(logits, legal)[0, 1].item() == torch.finfo(torch.float32).min
    assert mask_logits(logits.bfloat16(), legal)[0, 1].item() == torch.finfo(torch.bfloat16).min


def test_selfplay_helpers_refuse_cpu_tensors():
    from connect6_b200 import selfplay as S
    assert [S._symmetry_for_phase(i) for i in range(9)] == [(0, False), (1, False), (2, False), (3, False),
                                                            (0, True), (1, True), (2, True), (3, True), (0, False)]
    with pytest.raises(RuntimeError):
        S._sample_actions(torch.zeros(1, 9), torch.ones(1, 9, dtype=torch.bool), 1.0)
    with pytest.raises(RuntimeError):
        S._transform_actions(torch.zeros(3, dtype=torch.int64), 3, 1, False)


def test_history_ensemble_validation_without_gpu():
    from pathlib import Path
    from connect6_b200.history import HistoricalCheckpoint, HistoricalPolicyEnsemble
    with pytest.raises(ValueError):
        HistoricalPolicyEnsemble([], torch.device("cpu"))
    cfg = {"kernels": [3], "channels": [8]}
    cp = HistoricalCheckpoint(Path("model_update_00000001.pt"), 1, {}, cfg, {"board_size": 5})
    cp2 = HistoricalCheckpoint(Path("model_update_00000002.pt"), 2, {}, cfg, {"board_size": 7})
    with pytest.raises(ValueError):
        HistoricalPolicyEnsemble([cp, cp2], torch.device("cpu"))
    with pytest.raises(ValueError):
        HistoricalPolicyEnsemble([cp, HistoricalCheckpoint(Path("x"), 3, {}, {"kernels": [5], "channels": [8]},
                                                          {"board_size": 5})], torch.device("cpu"))
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError):          # valid checkpoints, but no device: loud failure
            HistoricalPolicyEnsemble([cp], torch.device("cpu"))


def test_board_generator_properties():
    from connect6_b200.boards import generate_planes, shard_range
    p = generate_planes(0, 4096)
    assert p.shape == (4096, 3, 19, 19) and p.dtype == np.float32
    assert set(np.unique(p)) <= {0.0, 1.0}
    mine, opp = p[:, 0].sum(axis=(1, 2)), p[:, 1].sum(axis=(1, 2))
    assert (p[:, 0] * p[:, 1]).sum() == 0                       # disjoint stones
    assert np.abs(mine - opp).max() <= 2
    total = mine + opp
    assert total.min() == 0 and total.max() == 120 and abs(total.mean() - 60) < 3
    assert ((p[:, 2].reshape(4096, -1).min(1)) == (p[:, 2].reshape(4096, -1).max(1))).all()   # constant plane
    assert 0.45 < p[:, 2, 0, 0].mean() < 0.55
    # keyed by global index: any sharding yields the same boards
    parts = [generate_planes(*(lambda lo, hi: (lo, hi - lo))(*shard_range(4096, r, 8))) for r in range(8)]
    assert np.array_equal(np.concatenate(parts), p)
    assert np.array_equal(generate_planes(1000, 10), p[1000:1010])
    wide = generate_planes(0, 512, max_stones=200)
    assert (wide[:, 0] + wide[:, 1]).sum(axis=(1, 2)).max() > 150
    cover = [shard_range(65536, r, 8) for r in range(8)]
    assert cover[0][0] == 0 and cover[-1][1] == 65536 and all(cover[i][1] == cover[i + 1][0] for i in range(7))


def test_training_workspace_sizes_are_host_arithmetic(engine_lib):
    """c6_conv_layer_backward_workspace_bytes / c6_backbone_workspace_bytes plan on the host only: positive for the
    shapes the operators support, 0 for the others, and growing with the batch."""
    import ctypes as C
    lib = engine_lib
    lib.c6_conv_layer_backward_workspace_bytes.restype = C.c_int64
    lib.c6_backbone_workspace_bytes.restype = C.c_int64
    one = lambda n, k, ci, co, B: lib.c6_conv_layer_backward_workspace_bytes(n, k, ci, co, C.c_int64(B))
    assert one(19, 3, 64, 96, 256) > 0 and one(19, 3, 64, 96, 512) > one(19, 3, 64, 96, 256)
    assert one(19, 5, 64, 96, 256) == 0 and one(19, 3, 192, 96, 256) == 0 and one(40, 3, 64, 96, 256) == 0
    def stack(n, channels, stem, B):
        arr = (C.c_int32 * len(channels))(*channels)
        return lib.c6_backbone_workspace_bytes(n, len(channels) - 1, arr, stem, C.c_int64(B))
    default = [3, 32, 32, 64, 64, 64, 96, 96, 96]
    assert stack(19, default, 23, 256) > 0 and stack(19, default, 23, 8192) > 30 * stack(19, default, 23, 256) // 2
    assert stack(19, default[1:], 0, 256) > 0                 # the 3x3 layers alone
    assert stack(19, default, 0, 256) > 0                     # 3 -> 32 as a 3x3 layer is a legal stack too
    assert stack(19, default, 22, 256) == 0                   # even stem
    assert stack(19, [5] + default[1:], 23, 256) == 0         # a stem reads 3 planes
    assert stack(19, [3, 32], 23, 256) == 0                   # a stem alone
    assert stack(19, [3, 96, 32], 23, 256) == 0               # stem wider than 64 channels
    assert stack(19, [32, 192], 0, 256) == 0                  # 3x3 layer wider than 128
    assert stack(19, default, 23, 0) == 0
