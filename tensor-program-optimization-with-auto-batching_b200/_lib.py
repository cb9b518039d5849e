"""ctypes binding of ``libmlora.so`` (declared in ``include/mlora.h``).

The library is loaded on first use.  There is no fallback: if it is missing
or fails to load, every operator raises ``MloraLibraryError``.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libmlora.so")

_i32, _i64, _f32, _vp, _sz = C.c_int32, C.c_int64, C.c_float, C.c_void_p, C.c_size_t

CHAIN_MAX_PHASES = 6


class ChainPhase(C.Structure):
    """``mlora_chain_phase`` of include/mlora.h."""
    _fields_ = [("d_x", _vp), ("ldx", _i64), ("d_Wp", _vp), ("d_y", _vp), ("ldy", _i64), ("in_", _i32), ("out", _i32),
                ("flags", _i32), ("eps", _f32), ("d_res", _vp), ("d_delta", _vp), ("d_norm_w", _vp), ("d_A_all", _vp),
                ("d_u", _vp), ("d_Bp", _vp), ("r_max", _i32), ("n_mod", _i32), ("mod_offsets", _i32 * 5)]


# name -> (restype, argtypes); must list every symbol declared in include/mlora.h
PROTOTYPES = {
    "mlora_version": (C.c_int, []),
    "mlora_last_error": (C.c_char_p, []),
    "mlora_launch_count": (C.c_uint64, []),
    "mlora_bucket_sort_workspace": (_sz, [_i32, _i32, _i32]),
    "mlora_bucket_sort": (C.c_int, [_vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "mlora_lora_shrink": (C.c_int, [_vp, _i64, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _vp]),
    "mlora_linear_workspace": (_sz, [_i32, _i32, _i32]),
    "mlora_packed_lora_b_bytes": (_sz, [_i32, _i32, _i32]),
    "mlora_pack_lora_b": (C.c_int, [_vp, _i32, _i32, _i32, _vp, _vp]),
    "mlora_packed_weight_bytes": (_sz, [_i32, _i32]),
    "mlora_pack_weight": (C.c_int, [_vp, _i32, _i32, _vp, _vp]),
    "mlora_linear_workspace_flags": (_sz, [_i32, _i32, _i32, _i32]),
    "mlora_linear_plan": (C.c_int, [_i32, _i32, _i32, C.POINTER(_i32)]),
    "mlora_linear": (C.c_int, [_vp, _i64, _vp, _vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32,
                               C.POINTER(_i32), _i32, _vp, _sz, _vp]),
    "mlora_linear_norm": (C.c_int, [_vp, _i64, _vp, _vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32,
                                    C.POINTER(_i32), _i32, _vp, _sz, _vp, _i64, _vp, _vp, _vp, _i32, C.c_float, _i32, _vp]),
    "mlora_lora_linear": (C.c_int, [_vp, _i64, _vp, _vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32,
                                    _i32, C.POINTER(_i32), _i32, _vp, _sz, _vp]),
    "mlora_decode_chain": (C.c_int, [C.POINTER(ChainPhase), _i32, _i32, _vp, _vp, _vp, _i32, _vp, _sz, _vp]),
    "mlora_residual_rmsnorm": (C.c_int, [_vp, _vp, _vp, _f32, _vp, _i32, _i32, _vp]),
    "mlora_residual_rmsnorm_shrink": (C.c_int, [_vp, _vp, _vp, _vp, _f32, _vp, _i32, _i32, _vp, _vp, _i32, _i32, _vp, _vp]),
    "mlora_embed": (C.c_int, [_vp, _vp, _i32, _i32, _i32, _vp, _vp, _vp]),
    "mlora_argmax": (C.c_int, [_vp, _i64, _i32, _i32, _vp, _vp]),
    "mlora_kv_append_rope": (C.c_int, [_vp, _i64, _vp, _vp, _vp, _i32, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _f32, _vp]),
    "mlora_paged_attention_workspace": (_sz, [_i32, _i32, _i32, _i32]),
    "mlora_paged_attention": (C.c_int, [_vp, _i64, _vp, _vp, _vp, _i32, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _f32,
                                        _i32, _vp, _i64, _i32, _vp, _sz, _vp]),
    "mlora_prefill_attention": (C.c_int, [_vp, _i64, _vp, _vp, _i32, _vp, _i32, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp,
                                          _i64, _vp, _vp]),
    "mlora_paged_attention_splits": (C.c_uint32, [_i32, _i32, _i32]),
    "mlora_paged_attention_shrink_workspace": (_sz, [_i32, _i32, _i32]),
    "mlora_paged_attention_shrink": (C.c_int, [_vp, _i64, _vp, _vp, _vp, _i32, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _f32,
                                               _i32, _vp, _i64, _vp, _vp, _vp, _i32, _i32, _vp, _vp, _sz, _vp]),
    "mlora_paged_attention_static_max_bytes": (_sz, []),
    "mlora_paged_attention_static": (C.c_int, [_vp, _i64, _vp, _vp, _vp, _i32, _vp, _vp, _i32, _i32, _i32, _i32, _i32,
                                               _f32, _i32, _vp, _i64, _i32, _vp]),
    "mlora_kv_begin_decode": (C.c_int, [_vp, _vp, _vp, _i32, _vp]),
    "mlora_tp_arena_bytes": (_sz, [_i32, _i32]),
    "mlora_tp_create": (C.c_int, [_i32, _i32, _i32, _i32, C.POINTER(_vp)]),
    "mlora_tp_export": (C.c_int, [_vp, _vp]),
    "mlora_tp_connect": (C.c_int, [_vp, _i32, _vp]),
    "mlora_tp_set_spin_limit": (C.c_int, [_vp, C.c_uint32]),
    "mlora_tp_status": (C.c_int, [_vp, C.POINTER(_i32)]),
    "mlora_tp_reset": (C.c_int, [_vp]),
    "mlora_tp_destroy": (C.c_int, [_vp]),
    "mlora_tp_allreduce_rmsnorm": (C.c_int, [_vp, _vp, _vp, _vp, _f32, _vp, _i32, _i32, _vp]),
    "mlora_decode_step_begin": (C.c_int, [_vp, _vp, _vp, _vp, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "mlora_decode_step_end": (C.c_int, [_vp, _vp, _i32, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _vp, _vp]),
}


class MloraLibraryError(RuntimeError):
    pass


class MloraError(RuntimeError):
    pass


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise MloraLibraryError(
                f"{LIB_PATH} is missing: build it with `python {os.path.join(HERE, 'build.py')}` "
                "(there is no CPU or PyTorch fallback for these operators)")
        try:
            handle = C.CDLL(LIB_PATH)
        except OSError as e:  # pragma: no cover
            raise MloraLibraryError(f"cannot load {LIB_PATH}: {e}") from e
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(rc: int, what: str):
    if rc != 0:
        msg = lib().mlora_last_error().decode(errors="replace")
        raise MloraError(f"{what} failed with code {rc}: {msg}")
