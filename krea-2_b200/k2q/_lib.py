"""ctypes binding of ``libk2q.so`` (declarations mirror ``include/k2q.h``).

There is no CPU fallback: if the library is missing or a call fails, a ``RuntimeError`` carrying
the C error string is raised.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libk2q.so"

K2Q_OK, K2Q_EINVAL, K2Q_EARCH, K2Q_ECUDA, K2Q_ETIMEOUT = 0, -1, -2, -3, -4
K2Q_BF16, K2Q_F32 = 0, 1
ACT_NONE, ACT_GELU_TANH = 0, 1


class Epilogue(C.Structure):
    """``struct k2q_epilogue`` of include/k2q.h."""
    _fields_ = [
        ("sx", C.c_void_p),
        ("bias", C.c_void_p),
        ("u", C.c_void_p),
        ("Bm", C.c_void_p),
        ("ldu", C.c_int64),
        ("ldb", C.c_int64),
        ("rank", C.c_int32),
        ("lora_scale", C.c_float),
        ("act", C.c_int32),
    ]


class Linear(C.Structure):
    """``struct k2q_linear`` of include/k2q.h: a quantised base as the host pipeline takes it."""
    _fields_ = [
        ("bits", C.c_int32),
        ("pad_", C.c_int32),
        ("codes", C.c_void_p),
        ("scale", C.c_void_p),
        ("bias", C.c_void_p),
        ("N", C.c_int64),
        ("K", C.c_int64),
    ]


_i64, _i32, _p, _f = C.c_int64, C.c_int32, C.c_void_p, C.c_float

# name -> (restype, argtypes); every symbol include/k2q.h declares
SIGNATURES = {
    "k2q_version": (C.c_int, []),
    "k2q_last_error": (C.c_char_p, []),
    "k2q_status_bytes": (_i64, []),
    "k2q_check_status": (C.c_int, [_p, _p]),
    "k2q_quant_weight_i8": (C.c_int, [_p, C.c_int, _i64, _i64, _i64, _p, _p, _p]),
    "k2q_quant_weight_i4": (C.c_int, [_p, C.c_int, _i64, _i64, _i64, _p, _p, _p]),
    "k2q_fwht_quant_act_i8": (C.c_int, [_p, C.c_int, _i64, _i64, _i64, _p, _p, _p]),
    "k2q_swiglu_fwht_quant": (C.c_int, [_p, _i64, _p, _i64, _i64, _i64, _p, _p, _p]),
    "k2q_gate_fwht_quant": (C.c_int, [_p, _i64, _p, _i64, _i64, _i64, _p, _p, _p]),
    "k2q_norm_mod_fwht_quant": (C.c_int, [_p, _i64, _i64, _i64, _p, _p, _p, _i64, _f, _p, _p, _p]),
    "k2q_quant_rows_i8": (C.c_int, [_p, C.c_int, _i64, _i64, _i64, _p, _p, _p, _p]),
    "k2q_fwht_rows": (C.c_int, [_p, C.c_int, _i64, _i64, _i64, _p, C.c_int, _i64, _p]),
    "k2q_gemm_w8a8": (C.c_int, [_p, _p, _p, _i64, _i64, _i64, C.POINTER(Epilogue), _p, _i64, _p, _p]),
    "k2q_gemm_w4a8": (C.c_int, [_p, _p, _p, _i64, _i64, _i64, C.POINTER(Epilogue), _p, _i64, _p, _p]),
    "k2q_qknorm_rope": (C.c_int, [_p, _i64, C.c_int, _p, _p, _i64, C.c_int, _p, _i64, _p, _p, C.c_float, _p]),
    "k2q_norm_mod_fwd": (C.c_int, [_p, _i64, _i64, _i64, _p, _p, _p, _i64, C.c_float, _p, _i64, _p, _p]),
    "k2q_norm_mod_bwd": (C.c_int, [_p, _i64, _p, _i64, _p, _i64, _i64, _p, _p, _i64, _p, _i64, _p]),
    "k2q_qknorm_rope_fwd": (C.c_int, [_p, _i64, C.c_int, _p, _p, _i64, _p, _i64, C.c_int, _p, _p, _i64, _i64, _p, _p,
                                      C.c_float, _p]),
    "k2q_qknorm_rope_bwd": (C.c_int, [_p, _i64, C.c_int, _p, _p, _i64, _i64, _i64, _p, _i64,
                                      _p, _i64, C.c_int, _p, _p, _i64, _i64, _i64, _p, _i64,
                                      _i64, _i64, _p, _p, C.c_float, _p]),
    "k2q_swiglu_fwd": (C.c_int, [_p, _i64, _p, _i64, _i64, _i64, _p, _i64, _p]),
    "k2q_swiglu_bwd": (C.c_int, [_p, _i64, _p, _i64, _p, _i64, _i64, _i64, _p, _i64, _p, _i64, _p]),
    "k2q_sigmoid_gate_fwd": (C.c_int, [_p, _i64, _p, _i64, _i64, _i64, _p, _i64, _p]),
    "k2q_sigmoid_gate_bwd": (C.c_int, [_p, _i64, _p, _i64, _p, _i64, _i64, _i64, _p, _i64, _p, _i64, _p]),
    "k2q_gate_residual": (C.c_int, [_p, _i64, _p, _i64, _p, _i64, _i64, _i64, _p, _i64, _p]),
    "k2q_requant_i4_to_i8": (C.c_int, [_p, _p, _i64, _i64, _p, _i64, _p, _p]),
    "k2q_gemm_dx_w8": (C.c_int, [_p, _p, _i64, _i64, _i64, C.POINTER(Epilogue), _p, _i64, _p, _p]),
    "k2q_transpose_i8": (C.c_int, [_p, _i64, _i64, _p, _p]),
    "k2q_lora_down": (C.c_int, [_p, _i64, _i64, _i64, _p, _i64, _i64, _i32, _f, _p, _i64, _p]),
    "k2q_lora_tn_workspace_bytes": (_i64, [_i64, _i32, _i64]),
    "k2q_lora_tn_static_max_bytes": (_i64, []),
    "k2q_lora_tn_static": (C.c_int, [_p, _i64, _p, _i64, _i64, _i32, _i64, _f, _p, _i64, _p]),
    "k2q_measure_i8_peak": (C.c_int, [C.c_int, _p, C.POINTER(C.c_double), _p]),
    "k2q_lora_tn": (C.c_int, [_p, _i64, _p, _i64, _i64, _i32, _i64, _f, _p, _i64, _p, _i64, _p]),
    "k2q_sumsq_workspace_bytes": (_i64, []),
    "k2q_sumsq_f32": (C.c_int, [_p, _i64, _p, C.c_int, _p, _i64, _p]),
    "k2q_adamw_clip_f32": (C.c_int, [_p, _p, _p, _p, _i64, _f, _f, _f, _f, _f, _i64, _f, _p, C.c_int, _p]),
    "k2q_selftest_wait_expiry": (C.c_int, [_p, C.c_int, _p]),
    "k2q_fwht_quant_act_i8_stream_ok": (C.c_int, [C.c_int, _i64, _i64, _i64]),
    "k2q_fwht_quant_act_i8_stream": (C.c_int, [_p, _i64, _i64, _p, _p, _p, _p]),
    "k2q_mlp_gelu_host_workspace_bytes": (_i64, [_i64, _i64, _i64, _i64, _i64]),
    "k2q_mlp_gelu_host": (C.c_int, [_p, _i64, C.POINTER(Linear), C.POINTER(Linear), _p, C.POINTER(_i64), C.c_int,
                                    _p, _i64, _p, _p, _p, _p]),
}

_lib = None


def load() -> C.CDLL:
    """Loads the library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m k2q.build` "
                "(or __graft_entry__.build()); there is no CPU fallback")
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def last_error() -> str:
    return load().k2q_last_error().decode("utf-8", "replace")


def check(rc: int, what: str) -> None:
    if rc == K2Q_OK:
        return
    msg = f"{what} failed ({rc}): {last_error()}"
    if rc == K2Q_EINVAL:
        raise ValueError(msg)
    raise RuntimeError(msg)
