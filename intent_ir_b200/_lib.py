"""ctypes binding of ``libintentir_b200.so`` (declared in ``include/intentir_b200.h``).

The library is the only execution path.  If it is missing there is no fallback: loading
raises :class:`B200LibraryError` with the build command.
"""

from __future__ import annotations

import ctypes as C
import os
from typing import Optional

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libintentir_b200.so")

OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_CUDA, ERR_BUFFER, ERR_DEVICE_WAIT = 0, -1, -2, -3, -4, -5
F32, BF16, F16, I32, I64, BOOL, U8, I8, I16, F64 = range(10)
REDUCE_SUM, REDUCE_MAX, REDUCE_ANY = 0, 1, 2
ACT_NONE, ACT_RELU = 0, 1
GEMM_ALLOW_TF32 = 1
GEMM_CTA_PAIRS = 2
GEMM_ONE_CTA = 4
GEMM_NARROW_TAIL = 8

DTYPE_CODE = {"f32": F32, "bf16": BF16, "f16": F16, "i32": I32, "i64": I64, "bool": BOOL, "i1": BOOL,
              "u8": U8, "i8": I8, "i16": I16, "f64": F64}
DTYPE_BYTES = {F32: 4, BF16: 2, F16: 2, I32: 4, I64: 8, BOOL: 1, U8: 1, I8: 1, I16: 2, F64: 8}


class B200LibraryError(ImportError):
    pass


_vp, _i, _i64, _f, _sz, _cp = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t, C.c_char_p

# name -> (restype, argtypes); every symbol include/intentir_b200.h declares
SIGNATURES = {
    "ib200_last_error": (_cp, []),
    "ib200_version": (_i, []),
    "ib200_plan_json": (_i, [_cp, _cp, _cp, _sz]),
    "ib200_plan_create": (_i, [_cp, _cp, C.POINTER(_vp)]),
    "ib200_plan_destroy": (None, [_vp]),
    "ib200_plan_describe": (_i, [_vp, _cp, _sz]),
    "ib200_plan_num_args": (_i, [_vp]),
    "ib200_plan_workspace_bytes": (_sz, [_vp]),
    "ib200_plan_num_launches": (_i, [_vp]),
    "ib200_plan_launch": (_i, [_vp, C.POINTER(_vp), _i, _vp, _sz, _vp]),
    "ib200_plan_launch_noalloc": (_i, [_vp, C.POINTER(_vp), _i, _vp]),
    "ib200_noalloc_workspace_limit": (_sz, []),
    "ib200_plan_check_status": (_i, [_vp, _vp, _vp]),
    "ib200_plan_check_status_noalloc": (_i, [_vp, _vp]),
    "ib200_noalloc_debug_poke_status": (_i, [_vp, C.c_int32, _vp]),
    "ib200_reduce": (_i, [_vp, _vp, _i, _i, _i, _i64, _i64, _i64, _f, _vp]),
    "ib200_reduce_scratch_bytes": (C.c_size_t, [_i64, _i64, _i64]),
    "ib200_reduce_ws": (_i, [_vp, _vp, _i, _i, _i, _i64, _i64, _i64, _f, _vp, C.c_size_t, _vp]),
    "ib200_reduce_any_f32": (_i, [_vp, _vp, _i64, _i64, _vp]),
    "ib200_softmax": (_i, [_vp, _vp, _vp, _vp, _i, _i64, _i64, _vp]),
    "ib200_softmax_io": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i64, _i64, _vp]),
    "ib200_softmax_masked": (_i, [_vp, _vp, _i64, _f, _vp, _vp, _vp, _i64, _i64, _vp]),
    "ib200_norm_rows": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i64, _i64, _i64, _i64, _f, _vp]),
    "ib200_layernorm": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i64, _i64, _f, _vp]),
    "ib200_groupnorm": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i64, _i64, _i64, _i64, _f, _vp]),
    "ib200_softmax_ws": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i64, _i64, _vp, _sz, _vp]),
    "ib200_softmax_scratch_bytes": (_sz, [_i, _i64, _i64]),
    "ib200_norm_rows_ws": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i64, _i64, _i64, _i64, _f, _vp, _sz, _vp]),
    "ib200_norm_scratch_bytes": (_sz, [_i, _i64, _i64]),
    "ib200_gemm_bias_act": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i64, _i64, _i64, _i, _i, _vp, _vp]),
    "ib200_gemm_bias_act_ws": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i64, _i64, _i64, _i, _i, _i, _vp, _sz, _vp, _vp]),
    "ib200_gemm_scratch_bytes": (_sz, [_i, _i, _i64, _i64, _i64, _i, _i]),
    "ib200_check_status": (_i, [_vp, _vp]),
    "ib200_transpose2d": (_i, [_vp, _vp, _i, _i64, _i64, _vp]),
}

_lib: Optional[C.CDLL] = None


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise B200LibraryError(
            f"{LIB_PATH} is missing. Build it with `python -m intent_ir_b200.build` (needs nvcc); "
            "there is no fallback execution path."
        )
    try:
        lib = C.CDLL(LIB_PATH)
    except OSError as e:
        raise B200LibraryError(f"cannot load {LIB_PATH}: {e}") from e
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise B200LibraryError(f"{LIB_PATH} does not export {name}; rebuild it") from e
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def last_error() -> str:
    msg = load().ib200_last_error()
    return msg.decode("utf-8", "replace") if msg else ""
