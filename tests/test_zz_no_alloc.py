"""GPU test of c6_forward_noalloc, the forward entry point that never allocates device memory.

It exists for callers that cannot afford (or are not allowed) to enter the CUDA allocator while
they run -- c6_forward may grow its workspace with cudaMalloc, this one works out of a fixed
2.5 MiB array inside the library.  The test calls it through the C ABI twice in a row with
different inputs (the array keeps the previous call's contents) and compares each result with
c6_forward on the same engine.  The file name sorts last so that a run stopping at the first
failure has already executed every other test.
The first call is also compared directly with the CPU oracle of the reference's forward.
"""
from __future__ import annotations

import ctypes as C

import pytest
import torch

import torch_port as TP

pytestmark = pytest.mark.gpu

TOL = 1e-6   # both entry points launch the same fp32 kernels; the engine's fp32 tolerance is 1e-3


def _call_noalloc(lib, L, eng, x, logits, value, flags=0, orient=None):
    return lib.c6_forward_noalloc(eng._h, x.data_ptr(), L.C6_X_F32, x.shape[0],
                                  None if orient is None else orient.data_ptr(), logits.data_ptr(), value.data_ptr(),
                                  flags, torch.cuda.current_stream(x.device).cuda_stream)


def test_forward_noalloc_matches_forward_twice_in_a_row(cuda_device):
    from connect6_b200 import _lib as L
    from connect6_b200.boards import generate_planes
    from connect6_b200.engine import Engine
    from connect6_b200.model import PolicyValueNet

    lib = L.load()
    torch.manual_seed(42)
    state = {k: v.detach().clone() for k, v in PolicyValueNet(19).state_dict().items()}
    eng = Engine(cuda_device, 19, PolicyValueNet.DEFAULT_KERNELS, PolicyValueNet.DEFAULT_CHANNELS, 1, "fp32")
    eng.load_state_dict(state)

    with torch.cuda.device(cuda_device):
        for first, boards in ((0, 9), (4000, 5)):                      # second call: other boards, smaller batch
            x = torch.from_numpy(generate_planes(first, boards)).to(cuda_device)
            want_logits, want_value = eng.forward(x, mask=True)
            logits = torch.full((boards, 361), float("nan"), device=cuda_device)
            value = torch.full((boards,), float("nan"), device=cuda_device)
            rc = _call_noalloc(lib, L, eng, x, logits, value, flags=L.C6_FLAG_MASK_LOGITS)
            assert rc == L.C6_OK, L.last_error(eng._h)
            torch.cuda.synchronize(cuda_device)
            assert torch.allclose(logits, want_logits, atol=TOL, rtol=0)
            assert torch.allclose(value, want_value, atol=TOL, rtol=0)
            if first == 0:   # and against the oracle itself (connect6/model.py:96-111 on CPU, fp64), legal cells only
                ref_l, ref_v = TP.policy_value_forward(x.cpu().double(), {k: v.double() for k, v in state.items()})
                legal = ((x[:, 0] == 0) & (x[:, 1] == 0)).flatten(1).cpu()
                assert (logits.cpu().double() - ref_l)[legal].abs().max().item() < 1e-5
                assert (value.cpu().double() - ref_v).abs().max().item() < 1e-5

        # per-board orientation goes through the same scratch
        x = torch.from_numpy(generate_planes(77, 8)).to(cuda_device)
        orient = torch.arange(8, dtype=torch.uint8, device=cuda_device)
        want_logits, want_value = eng.forward(x, orient, mask=True, inverse_map=True)
        logits = torch.empty((8, 361), device=cuda_device)
        value = torch.empty((8,), device=cuda_device)
        rc = _call_noalloc(lib, L, eng, x, logits, value, flags=L.C6_FLAG_MASK_LOGITS | L.C6_FLAG_INVERSE_MAP,
                           orient=orient)
        assert rc == L.C6_OK, L.last_error(eng._h)
        torch.cuda.synchronize(cuda_device)
        assert torch.allclose(logits, want_logits, atol=TOL, rtol=0) and torch.allclose(value, want_value, atol=TOL)

        # beyond the fixed scratch: rejected with a clear message, nothing launched
        big = torch.zeros((10, 3, 19, 19), device=cuda_device)
        out_l = torch.empty((10, 361), device=cuda_device)
        out_v = torch.empty((10,), device=cuda_device)
        launches = eng.launch_count
        assert _call_noalloc(lib, L, eng, big, out_l, out_v) == L.C6_ERR_ARG
        assert "scratch" in L.last_error(eng._h) and eng.launch_count == launches

        # only fp32-mode engines with one weight set are served
        bf16 = Engine(cuda_device, 19, PolicyValueNet.DEFAULT_KERNELS, PolicyValueNet.DEFAULT_CHANNELS, 1, "bf16")
        bf16.load_state_dict(state)
        assert _call_noalloc(lib, L, bf16, x, logits, value) == L.C6_ERR_UNSUPPORTED
    assert eng.status() == 0
