"""ctypes binding of libgq_b200.so (the C ABI in include/gq_b200.h).

The library is the only compute path: if it is missing this module raises on first use — there is
no PyTorch, Triton or CPU fallback.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libgq_b200.so")

ERRORS = {-1: "unsupported GGML type", -2: "bad shape (K not a multiple of 256, negative size, or M over the limit)",
          -3: "bad argument (null or misaligned pointer, inconsistent sizes)", -4: "workspace too small",
          -5: "CUDA runtime error", -6: "size beyond a fixed maximum"}
DESC_WORDS = 8
MAX_GEMV_ROWS = 64

_lib = None
_vp, _i64, _i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int

# every symbol include/gq_b200.h declares: name -> (restype, argtypes)
SIGNATURES = {
    "gq_bytes_per_256": (_i32, [_i32]),
    "gq_packed_bytes": (_i64, [_i32, _i64, _i64]),
    "gq_slab_map": (_i32, [_i32, _vp]),
    "gq_repack": (_i32, [_i32, _vp, _i64, _i64, _i64, _vp, _vp]),
    "gq_unrepack": (_i32, [_i32, _vp, _i64, _i64, _vp, _i64, _vp]),
    "gq_dequant": (_i32, [_i32, _vp, _i64, _i64, _vp, _i32, _i64, _vp]),
    "gq_desc_rows": (_i64, [_i32, _vp, _i32]),
    "gq_build_descs": (_i64, [_i32, _vp, _vp, _i64, _i32, _vp]),
    "gq_split_for": (_i32, [_i64, _i64, _i64, _i32, _i32]),
    "gq_run_info": (_i32, [_i32, _vp]),
    "gq_workspace_bytes": (_i64, [_i64, _i64, _i64, _i32]),
    "gq_gemv_grouped": (_i32, [_vp, _i64, _i64, _i64, _vp, _vp, _i64, _i32, _i32, _vp, _i64, _i64, _vp, _i64, _vp]),
    "gq_gemv_grouped_phases": (_i32, [_vp, _i64, _i64, _i64, _vp, _vp, _i64, _i32, _i32, _vp, _i64, _i64, _vp, _i64, _vp, _i32]),
    "gq_gemv_grouped_prefetch": (_i32, [_vp, _i64, _i64, _i64, _vp, _vp, _i64, _i32, _i32, _vp, _i64, _i64, _vp, _i64, _vp, _vp, _i64]),
    "gq_gemv_grouped_pre": (_i32, [_vp, _i64, _i64, _i64, _i32, _vp, _vp, _vp, _i64, ctypes.c_float, _vp, _vp, _i64, _i32, _i32, _vp, _i64, _i64, _vp,
                                   _i64, _vp]),
    "gq_static_workspace_limit": (_i64, []),
    "gq_gemv_grouped_static": (_i32, [_vp, _i64, _i64, _i64, _vp, _vp, _i64, _i32, _i32, _vp, _i64, _i64, _vp]),
    "gq_allreduce_buffer_bytes": (_i64, [_i32, _i64]),
    "gq_allreduce_push": (_i32, [_vp, _vp, _i64, _i32, _i32, _vp, _i64, _vp]),
    "gq_fused_allreduce_buffer_bytes": (_i64, [_i32, _i64, _i64]),
    "gq_gemv_grouped_allreduce": (_i32, [_vp, _i64, _i64, _i64, _vp, _vp, _i64, _i32, _i32, _vp, _i64, _i64, _vp, _i64, _i32, _i32, _vp,
                                         _i64, _i64, _vp]),
    "gq_gemv_grouped_allreduce_silu_mul": (_i32, [_vp, _i64, _i64, _i64, _vp, _vp, _i64, _i32, _i32, _vp, _i64, _i64, _vp, _i64, _i32, _i32, _vp,
                                                  _i64, _i64, _vp]),
    "gq_prefill_workspace_bytes": (_i64, [_i64, _i64, _i64, _i64]),
    "gq_gemm_prefill": (_i32, [_vp, _i64, _i64, _i64, _vp, _vp, _i64, _i32, _vp, _i64, _i64, _vp, _i64, _vp]),
    "gq_read_status": (_i32, [_vp, _i64, _vp]),
    "gq_device_status": (_i32, [_i32, _vp]),
    "gq_set_peer_wait_limit_ns": (_i32, [_i64]),
    "gq_last_cuda_error": (ctypes.c_char_p, []),
    "gq_launch_count": (_i64, []),
}


class GqError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise GqError(f"{LIB_PATH} is missing: build it with `python -m hyperqwen_rtx4080s32_b200.build` "
                          "(there is no fallback path)")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def check(rc: int, what: str) -> int:
    if rc < 0:
        detail = ERRORS.get(int(rc), "unknown error")
        if rc == -5:
            detail += ": " + lib().gq_last_cuda_error().decode()
        raise GqError(f"{what} failed ({rc}): {detail}")
    return rc
