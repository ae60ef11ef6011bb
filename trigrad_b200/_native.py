"""ctypes binding of ``libtrigrad_b200.so`` (the C ABI declared in ``include/trigrad_b200.h``).

There is no fallback: if the shared library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# TRIGRAD_B200_LIB names another build of the same ABI (comparing two builds of the kernels in one session)
LIB_PATH = os.environ.get("TRIGRAD_B200_LIB") or os.path.join(HERE, "libtrigrad_b200.so")

TG_OK, TG_ERR_BAD_ARG, TG_ERR_WORKSPACE, TG_ERR_CAPACITY, TG_ERR_DEVICE_FLAG, TG_ERR_CUDA = range(6)
TG_ACCUMULATE_PACKED = 2   # accumulate mode of the backward entry points: the sums stay in the scratch
TG_FORWARD_CULL_TILES = 1  # flag of the forward entry points: list a (triangle, tile) pair only if it can cover a pixel
TG_INPUT_PACKED = 2        # flag of the forward entry points: faces [T,4] int32 and colours [V,4] (r, g, b, opacity)
GEO_WORDS = 16
ATTR_WORDS = 24

_vp, _i, _u32, _f, _sz = C.c_void_p, C.c_int, C.c_uint32, C.c_float, C.c_size_t

# name -> (restype, argtypes); one entry per symbol declared in include/trigrad_b200.h
SIGNATURES = {
    "tg_version": (_i, []),
    "tg_status_string": (C.c_char_p, [_i]),
    "tg_last_error": (C.c_char_p, []),
    "tg_launch_count": (C.c_ulonglong, []),
    "tg_preprocess": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "tg_scan_scratch_bytes": (_sz, [_i]),
    "tg_scan": (_i, [_vp, _vp, _i, _vp, _sz, _vp, _vp]),
    "tg_scan_static": (_i, [_vp, _vp, _i, _vp, _vp]),
    "tg_selftest_bounded_wait": (_i, [_vp, _sz, _vp, _u32, _vp]),
    "tg_emit_keys": (_i, [_vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _u32, _vp]),
    "tg_sort_scratch_bytes": (_sz, [_u32]),
    "tg_sort_pairs": (_i, [_vp, _vp, _vp, _vp, _u32, _i, _i, _vp, _sz, _vp, C.POINTER(_i), _vp]),
    "tg_tile_ranges": (_i, [_vp, _u32, _i, _vp, _vp]),
    "tg_tile_sort_scratch_bytes": (_sz, [_i]),
    "tg_sort_tile_lists": (_i, [_vp, _vp, _i, _vp, _vp, _sz, _vp]),
    "tg_selection_planes": (_i, [_i, _i]),
    "tg_blend_forward": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "tg_backward_scratch_bytes": (_sz, [_i]),
    "tg_blend_backward": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                               _vp, _vp, _i, _vp, _sz, _vp]),
    "tg_blend_backward_corrected": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                         _vp, _vp, _i, _vp, _sz, _vp]),
    "tg_blend_backward_l2": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _f, _f, _vp, _vp, _vp, _vp, _vp, _vp,
                                  _vp, _vp, _vp, _i, _vp, _sz, _vp]),
    "tg_blend_backward_l2_u8": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _f, _f, _vp, _vp, _vp, _vp, _vp, _vp,
                                     _vp, _vp, _vp, _i, _vp, _sz, _vp]),
    "tg_blend_step_l2": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _vp, _f, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                              _vp, _i, _vp, _sz, _vp]),
    "tg_forward_workspace_bytes": (_sz, [_i, _i, _u32]),
    "tg_render_forward": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                               _u32, _vp, _vp, _sz, _vp, _vp, C.c_uint, _vp]),
    "tg_unpack_gradients": (_i, [_vp, _sz, _i, _f, _vp, _vp, _vp, _vp, _i, _vp]),
    "tg_pack_inputs": (_i, [_vp, _vp, _vp, _i, _i, _vp, _vp, _vp]),
    "tg_unpack_gradients_rgba": (_i, [_vp, _sz, _i, _f, _vp, _vp, _vp, _i, _vp]),
    "tg_project": (_i, [_vp, _i, _vp, _vp, _vp]),
    "tg_project_backward": (_i, [_vp, _i, _vp, _vp, _vp, _i, _vp]),
    "tg_project_clip": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "tg_project_clip_backward": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "tg_unpack_project_backward": (_i, [_vp, _sz, _i, _vp, _vp, _f, _vp, _vp, _vp, _vp, _vp]),
    "tg_render_step_l2": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _vp, _f, _f, _vp, _vp, _vp, _vp, _vp, _vp,
                               _vp, _vp, _u32, _vp, _vp, _vp, _vp, _i, _vp, _sz, _vp, _sz, _vp, _vp, C.c_uint, _vp]),
}

_lib = None


class NativeError(RuntimeError):
    def __init__(self, stage: str, status: int, detail: str):
        super().__init__(f"trigrad_b200 {stage} failed: status {status} ({detail})")
        self.stage = stage
        self.status = status


def lib() -> C.CDLL:
    """Load the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build the CUDA library first (python -m trigrad_b200.build). "
                "trigrad_b200 has no CPU or PyTorch fallback.")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(stage: str, status: int) -> None:
    if status != TG_OK:
        L = lib()
        detail = L.tg_last_error().decode() or L.tg_status_string(status).decode()
        raise NativeError(stage, status, detail)
