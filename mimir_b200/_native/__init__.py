"""ctypes binding of ``libmimir_b200.so`` (plain C ABI, see ``csrc/*.cu``).

The library is built in-tree by :mod:`mimir_b200._native.build`.  On a machine
with a GPU a missing library is an error, never a silent fallback: callers use
:func:`lib` and get an exception that names the build command.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "libmimir_b200.so"
_lib = None


class NativeUnavailable(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """Returns the loaded native library, building nothing: raises if absent."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise NativeUnavailable(
                f"{LIB_PATH} is missing; run `python -m mimir_b200._native.build`")
        _lib = ctypes.CDLL(str(LIB_PATH), mode=os.RTLD_LOCAL | os.RTLD_NOW)
        _declare(_lib)
    return _lib


def available() -> bool:
    try:
        lib()
        return True
    except (NativeUnavailable, OSError):
        return False


c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_float = ctypes.c_float
c_ll = ctypes.c_longlong


def _declare(l: ctypes.CDLL) -> None:
    def sig(name, res, *args):
        fn = getattr(l, name, None)
        if fn is not None:
            fn.restype = res
            fn.argtypes = list(args)

    sig("mimir_version", c_int)
    sig("mimir_set_device", c_int, c_int)
    sig("mimir_error_word", ctypes.c_uint, c_int)
    sig("mimir_launch_count", c_ll)
    sig("mimir_launch_count_add", None, c_ll)
    sig("mimir_last_error", ctypes.c_char_p)
    sig("mimir_sm_count", c_int)
    sig("mimir_gemm_workspace_bytes", c_ll, c_int, c_int)
    sig("mimir_gemm_bf16", c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
        c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_float, c_void_p, c_ll,
        c_int, c_int, c_void_p)
    P, I, F, L = c_void_p, c_int, c_float, c_ll
    sig("mimir_layernorm_fwd", I, P, P, P, P, P, P, I, I, F, P)
    sig("mimir_rmsnorm_fwd", I, P, P, P, P, I, I, F, P)
    sig("mimir_norm_bwd_blocks", I)
    sig("mimir_layernorm_bwd", I, P, P, P, P, P, P, P, P, P, P, I, I, I, P)
    sig("mimir_rmsnorm_bwd", I, P, P, P, P, P, P, P, P, I, I, I, P)
    sig("mimir_colsum", I, P, I, I, I, P, P, I, P)
    sig("mimir_cross_entropy", I, P, P, P, P, P, I, I, I, F, F, P)
    sig("mimir_softmax_rows", I, P, P, I, I, I, P)
    sig("mimir_embedding_fwd", I, P, P, P, P, I, I, I, I, P)
    sig("mimir_embedding_bwd", I, P, P, P, P, I, I, I, I, I, P)
    sig("mimir_act_fwd", I, P, P, L, I, P)
    sig("mimir_act_bwd", I, P, P, P, L, I, P)
    sig("mimir_swiglu_fwd", I, P, P, I, I, P)
    sig("mimir_swiglu_bwd", I, P, P, P, I, I, P)
    sig("mimir_swiglu2_fwd", I, P, P, P, L, P)
    sig("mimir_swiglu2_bwd", I, P, P, P, P, P, L, P)
    sig("mimir_rope", I, P, P, P, I, I, I, I, I, I, I, P)
    sig("mimir_cast_f32_bf16", I, P, P, L, F, P)
    sig("mimir_cast_bf16_f32", I, P, P, L, F, P)
    sig("mimir_axpby", I, P, P, P, L, F, F, P)
    sig("mimir_sumsq", I, P, L, I, P, P)
    sig("mimir_philox_uniform", I, P, L, ctypes.c_ulonglong, P)
    sig("mimir_philox_dropout", I, P, P, L, ctypes.c_ulonglong, F, P)
    sig("mimir_attention_fwd", I, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, I, F, P)
    sig("mimir_attention_bwd", I, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, I,
        I, I, I, F, P)
    PP = ctypes.POINTER(c_void_p)
    sig("mimir_peer_alloc", I, L, PP)
    sig("mimir_peer_free", I, P)
    sig("mimir_ipc_export", I, P, ctypes.c_char_p)
    sig("mimir_ipc_open", I, ctypes.c_char_p, PP)
    sig("mimir_ipc_close", I, P)
    sig("mimir_set_peer_wait_ms", None, L)
    sig("mimir_dp_bucket", I, PP, PP, PP, P, P, P, P, P, P, L, L, L, L, F, F, F, F, I, I, I, I, I, P)
    sig("mimir_dp_step_begin", I, P, P, I, P, I, P)
    sig("mimir_peer_wait_probe", I, P, ctypes.c_uint, L, P, P)
    sig("mimir_adamw_flat", I, P, P, P, I, P, P, L, L, F, F, F, F, F, I, F, P, F, P, P)


def last_error() -> str:
    return lib().mimir_last_error().decode()


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what}: {last_error()}")
