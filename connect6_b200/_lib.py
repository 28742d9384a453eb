"""ctypes binding of the engine's C ABI (include/c6_engine.h, include/c6_env.h, include/c6_train.h, include/c6_debug.h).

The library is loaded from the package directory (connect6_b200/libc6engine.so).  There is no
fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libc6engine.so"

C6_MAX_LAYERS = 16
C6_OK, C6_ERR_ARG, C6_ERR_CUDA, C6_ERR_UNSUPPORTED, C6_ERR_WEIGHTS, C6_ERR_DEVICE = range(6)
C6_PREC_BF16, C6_PREC_FP32, C6_PREC_F16 = 0, 1, 2
C6_STATUS_WAIT_MASK, C6_STATUS_BAD_INDEX, C6_STATUS_F16_RANGE = 63, 64, 128
C6_X_F32, C6_X_BF16 = 0, 1
C6_HEAD_POLICY, C6_HEAD_VALUE = 100, 101
C6_FLAG_MASK_LOGITS, C6_FLAG_INVERSE_MAP = 1, 2
C6_KIND_PACK, C6_KIND_STEM, C6_KIND_FINISH, C6_KIND_OTHER, C6_KIND_CONV0 = 0, 1, 2, 3, 8
C6_KIND_COUNT = 8 + C6_MAX_LAYERS


class C6Desc(C.Structure):
    _fields_ = [
        ("device", C.c_int32),
        ("board_size", C.c_int32),
        ("n_layers", C.c_int32),
        ("kernels", C.c_int32 * C6_MAX_LAYERS),
        ("channels", C.c_int32 * C6_MAX_LAYERS),
        ("groups", C.c_int32),
        ("precision", C.c_int32),
        ("max_chunk", C.c_int32),
    ]


class C6EnvState(C.Structure):
    """include/c6_env.h: the state tensors of VectorConnect6 as device pointers."""
    _fields_ = [
        ("boards", C.c_void_p), ("current_player", C.c_void_p), ("stones_left", C.c_void_p),
        ("empty_count", C.c_void_p), ("move_count", C.c_void_p),
        ("num_envs", C.c_int64), ("board_size", C.c_int32), ("win_length", C.c_int32),
    ]


class C6CollectorState(C.Structure):
    """include/c6_env.h: the rollout collector's per-environment bookkeeping tensors."""
    _fields_ = [
        ("current_episode_ids", C.c_void_p), ("current_segment_lengths", C.c_void_p),
        ("historical_mask", C.c_void_p), ("historical_current_colors", C.c_void_p),
        ("episode_results", C.c_void_p), ("episode_terminal_moves", C.c_void_p),
        ("episode_capacity", C.c_int64), ("next_episode_id", C.c_void_p),
    ]


C6_ENV_FAULT_OCCUPIED, C6_ENV_FAULT_ACTION, C6_ENV_FAULT_EPISODE, C6_ENV_FAULT_COUNT = 0, 1, 2, 4
C6_STAT_COUNT, C6_STAT_DONE_COUNT = 10, 9

_vp, _i, _i64, _u64, _f = C.c_void_p, C.c_int, C.c_int64, C.c_uint64, C.c_float

# name -> (restype, argtypes); mirrors include/*.h declaration by declaration
SIGNATURES = {
    "c6_version": (_i, []),
    "c6_create": (_i, [C.POINTER(C6Desc), C.POINTER(_vp)]),
    "c6_set_weights": (_i, [_vp, _i, _i, _vp, _vp, _vp]),
    "c6_reserve": (_i, [_vp, _i64]),
    "c6_forward": (_i, [_vp, _vp, _i, _i64, _vp, _vp, _vp, _i, _vp]),
    "c6_forward_noalloc": (_i, [_vp, _vp, _i, _i64, _vp, _vp, _vp, _i, _vp]),
    "c6_forward_step": (_i, [_vp, _vp, _i, _i64, _vp, _i, _f, _u64, _u64, _i64, _vp, _vp, _vp, _vp, _vp]),
    "c6_forward_step_boards": (_i, [_vp, _vp, _vp, _vp, _i64, _vp, _i64, _vp, _i, _f, _u64, _u64, _i64, _vp, _vp, _vp, _vp, _vp]),
    "c6_forward_grouped": (_i, [_vp, _vp, _i, _i64, _vp, _vp, _i, _vp]),
    "c6_sample_actions": (_i, [_vp, _vp, _i64, C.c_int32, _f, _u64, _u64, _i64, _vp, _vp, _vp]),
    "c6_mask_logits": (_i, [_vp, _vp, _i64, _f, _vp, _vp]),
    "c6_transform_actions": (_i, [_vp, _i64, C.c_int32, _vp, C.c_int32, C.c_int32, _vp, _vp]),
    "c6_transform_boards": (_i, [_vp, _i64, C.c_int32, _vp, C.c_int32, _vp, _vp]),
    "c6_network_input": (_i, [_vp, _vp, _vp, _i64, C.c_int32, _vp, _vp]),
    "c6_debug_layer_output": (_i, [_vp, _vp, _i, _i64, _vp, _i, _vp, _vp]),
    "c6_profile_enable": (_i, [_vp, _i]),
    "c6_profile_read": (_i, [_vp, C.POINTER(C.c_float), C.POINTER(_i64), _i]),
    "c6_debug_wait_cycles": (_i, [_vp, C.POINTER(_i64), _i]),
    "c6_debug_cta_times": (_i, [_vp, C.POINTER(_i64), _i]),
    "c6_clear_status": (_i, [_vp]),
    "c6_debug_expire_wait": (_i, [_vp, _vp]),
    "c6_status": (_i, [_vp, C.POINTER(_i)]),
    "c6_launch_count": (_i64, [_vp]),
    "c6_device_bytes": (_i64, [_vp]),
    "c6_last_error": (C.c_char_p, [_vp]),
    "c6_destroy": (_i, [_vp]),
    "c6_conv_layer_backward_workspace_bytes": (_i64, [C.c_int32, C.c_int32, C.c_int32, C.c_int32, _i64]),
    "c6_conv_layer_backward": (_i, [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _i64, _vp, _vp, _vp, _vp, _vp, _vp,
                                    _vp, _vp, _i64, _vp]),
    "c6_backbone_workspace_bytes": (_i64, [C.c_int32, C.c_int32, C.POINTER(C.c_int32), C.c_int32, _i64]),
    "c6_backbone_forward": (_i, [C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_int32), C.c_int32, _i64, _vp, C.POINTER(_vp),
                                 C.POINTER(_vp), _vp, _vp, _i64, _vp]),
    "c6_backbone_forward_boards": (_i, [C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_int32), C.c_int32, _i64, _vp, _vp, _vp, _i64, _vp,
                                        C.POINTER(_vp), C.POINTER(_vp), _vp, _vp, _i64, _vp]),
    "c6_backbone_backward": (_i, [C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_int32), C.c_int32, _i64, _vp, _vp,
                                  C.POINTER(_vp), C.POINTER(_vp), _vp, _i64, _vp]),
    "c6_backbone_heads_forward": (_i, [C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_int32), C.c_int32, _i64, _vp, _vp, _vp, _vp,
                                       _vp, _vp, _vp, _i64, _vp]),
    "c6_backbone_heads_backward": (_i, [C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_int32), C.c_int32, _i64, _vp, _vp, _vp, _vp,
                                        _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp]),
    "c6_ppo_loss": (_i, [C.c_int32, _i64, C.c_int32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, C.c_float, C.c_float, C.c_float, C.c_float,
                         _vp, _vp, _vp, _vp, _i64, _vp]),
    "c6_clip_adamw_step": (_i, [C.c_int32, C.c_int32, C.POINTER(_i64), C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp),
                                C.c_float, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float, _i64, _vp, _vp, _vp, _i64, _vp]),
    "c6_train_last_error": (C.c_char_p, []),
    "c6_env_step": (_i, [C.POINTER(C6EnvState), _vp, C.c_int32, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "c6_env_reset": (_i, [C.POINTER(C6EnvState), _vp, _i64, _vp]),
    "c6_env_legal_mask": (_i, [C.POINTER(C6EnvState), _vp, _vp]),
    "c6_env_collect_workspace_bytes": (_i64, [_i64]),
    "c6_env_collect_done": (_i, [C.POINTER(C6EnvState), C.POINTER(C6CollectorState), _vp, _vp, _vp, _vp, _vp, _vp,
                                 _vp, _vp]),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library once and attach the prototypes."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m connect6_b200.build` "
                "(the engine has no other execution path)"
            )
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def last_error(handle=None) -> str:
    msg = load().c6_last_error(handle)
    return msg.decode("utf-8", "replace") if msg else ""


def check(rc: int, handle=None, what: str = "") -> None:
    if rc == C6_OK:
        return
    msg = last_error(handle)
    names = {1: "bad argument", 2: "CUDA error", 3: "unsupported", 4: "weights missing", 5: "device status"}
    text = f"{what or 'c6 call'} failed ({names.get(rc, rc)}): {msg}"
    if rc in (C6_ERR_ARG, C6_ERR_UNSUPPORTED):
        raise ValueError(text)
    raise RuntimeError(text)


def ptr(t) -> int | None:
    """Device pointer of a torch tensor (None passes a null pointer)."""
    return None if t is None else t.data_ptr()
