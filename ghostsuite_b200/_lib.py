"""ctypes binding of libghost_b200.so.

The shared object is the product; this module only declares prototypes and turns status codes into
the exception types GhostSuite raises (ValueError for bad arguments, RuntimeError otherwise).
There is no fallback: if the library is missing or the device is not sm_100 every op raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libghost_b200.so")

GHOST_OK = 0
GHOST_ERR_INVALID = -1
GHOST_ERR_CUDA = -2
GHOST_ERR_DEVICE = -3
GHOST_ERR_KERNEL_TIMEOUT = -4
GHOST_ERR_INDEX = -5

_vp, _i, _ll, _f = C.c_void_p, C.c_int, C.c_longlong, C.c_float


class SmallJob(C.Structure):
    """``ghost_small_job`` of include/ghost_b200.h."""
    _fields_ = [("X", _vp), ("M", _vp), ("sum_out", _vp), ("n_train", _i), ("n_val", _i), ("F", _i),
                ("sum_is_f32", _i), ("dot_scale", _f), ("sum_scale", _f),
                ("Xv", _vp), ("v_rank_pitch", _ll), ("v_per_rank", _i)]


# name -> (restype, argtypes); mirrors include/ghost_b200.h one to one
PROTOTYPES = {
    "ghost_version": (C.c_char_p, []),
    "ghost_last_error": (C.c_char_p, []),
    "ghost_device_check": (_i, []),
    "ghost_sm_count": (_i, []),
    "ghost_launch_count": (_ll, []),
    "ghost_poll_kernel_error": (_i, [_i]),
    "ghost_cast_split_bf16": (_i, [_vp, _i, _ll, _ll, _i, _ll, _vp, _ll, _i, _i, _i, _i, _i, _i, _vp]),
    "ghost_gram_dot_bf16": (_i, [_vp, _vp, _vp, _vp, _i, _i, _ll, _i, _i, _ll, _ll, _ll, _ll, _i, _f, _vp, _vp]),
    "ghost_set_gram_pair_mode": (_i, [_i]),
    "ghost_set_persample_pair_mode": (_i, [_i]),
    "ghost_set_wgrad_pair_mode": (_i, [_i]),
    "ghost_wgrad_workspace_bytes": (_ll, [_i, _i]),
    "ghost_wgrad_bf16": (_i, [_vp, _vp, _ll, _i, _i, _ll, _ll, _f, _i, _vp, _i, _vp, _ll, _vp]),
    "ghost_persample_workspace_bytes": (_ll, [_i, _i, _i, _i, _i]),
    "ghost_set_persample_budget_bytes": (_i, [_ll]),
    "ghost_persample_dot_bf16": (_i, [_vp, _vp, _i, _i, _ll, _i, _i, _ll, _ll, _f, _vp, _i, _vp, _i, _f, _i, _i, _vp, _vp, _ll, _vp]),
    "ghost_persample_tiles_bytes": (_ll, [_i, _i, _i]),
    "ghost_persample_tiles_bf16": (_i, [_vp, _vp, _i, _ll, _i, _i, _ll, _ll, _i, _i, _i, _vp, _vp, _ll, _vp]),
    "ghost_tile_dot_bf16": (_i, [_vp, _i, _i, _vp, _i, _i, _i, _f, _vp, _vp, _i, _f, _i, _vp]),
    "ghost_colsum": (_i, [_vp, _i, _i, _ll, _i, _ll, _vp, _vp]),
    "ghost_layernorm_workspace_bytes": (_ll, [_i, _ll, _i]),
    "ghost_layernorm_persample": (_i, [_vp, _vp, _i, _i, _ll, _i, _f, _vp, _vp, _vp, _ll, _vp]),
    "ghost_rmsnorm_persample": (_i, [_vp, _vp, _i, _i, _ll, _i, _f, _vp, _vp, _vp, _ll, _vp]),
    "ghost_small_gram_f32": (_i, [_vp, _i, _i, _i, _f, _vp, _vp]),
    "ghost_rows_sum": (_i, [_vp, _i, _i, _f, _vp, _i, _i, _vp]),
    "ghost_small_reduce_batch": (_i, [C.POINTER(SmallJob), _i, _vp]),
    "ghost_embedding_dot_workspace_bytes": (_ll, [_i, _ll, _i]),
    "ghost_embedding_dot_workspace_bytes_for": (_ll, [_i, _ll, _i, _i]),
    "ghost_embedding_dot": (_i, [_vp, _vp, _i, _i, _i, _ll, _i, _i, _f, _vp, _vp, _ll, _vp]),
    "ghost_embedding_dot_noalloc": (_i, [_vp, _vp, _i, _i, _i, _ll, _i, _i, _f, _vp, _vp]),
    "ghost_embedding_wgrad_workspace_bytes": (_ll, [_i, _ll, _i]),
    "ghost_embedding_wgrad": (_i, [_vp, _vp, _i, _i, _ll, _i, _i, _f, _f, _i, _vp, _vp, _ll, _vp]),
    "ghost_gradproj_dense_bf16": (_i, [_vp, _vp, _i, _ll, _i, _i, _ll, _ll, _vp, _vp, _i, _i, _ll, _ll, _f, _vp, _ll, _vp]),
    "ghost_gradproj_embedding": (_i, [_vp, _vp, _i, _i, _ll, _i, _ll, _vp, _ll, _i, _i, _vp, _ll, _i, _i, _i, _f,
                                      _i, _vp, _ll, _i, _vp]),
    "ghost_projection_similarity": (_i, [_vp, _vp, _i, _i, _i, _ll, _ll, _ll, _f, _vp, _ll, _vp]),
    "ghost_workload_ce_forward": (_i, [_vp, _i, _ll, _i, _i, _ll, _vp, _ll, _vp, _vp, _vp, _vp, _vp]),
    "ghost_workload_ce_rescale": (_i, [_vp, _i, _ll, _i, _vp, _vp]),
    "ghost_workload_ce_backward": (_i, [_vp, _i, _ll, _i, _i, _ll, _vp, _ll, _vp, _vp, _vp, _ll, _vp]),
}

_lib = None


class GhostKernelError(RuntimeError):
    """A CUDA call failed or a kernel gave up a bounded wait."""


def load() -> C.CDLL:
    """Load the shared object (once).  Raises RuntimeError with build instructions if absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m ghostsuite_b200.build` "
            "(needs nvcc with sm_100a support). There is no CPU or PyTorch fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)   # AttributeError here means header and library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error() -> str:
    return load().ghost_last_error().decode("utf-8", "replace")


def check(status: int) -> None:
    """Translate a status code into GhostSuite's exception types."""
    if status == GHOST_OK:
        return
    msg = last_error()
    if status == GHOST_ERR_INVALID:
        raise ValueError(msg)
    if status == GHOST_ERR_INDEX:
        raise IndexError(msg)
    if status == GHOST_ERR_DEVICE:
        raise RuntimeError(f"ghostsuite_b200 needs a B200 (sm_100) GPU: {msg}")
    raise GhostKernelError(msg)


def launch_count() -> int:
    return int(load().ghost_launch_count())


def poll_kernel_error(clear: bool = True) -> None:
    check(load().ghost_poll_kernel_error(1 if clear else 0))
