"""ctypes binding of libcamel_tensor_b200.so (declared in include/camel_tensor_b200.h).

The library must have been built (``python -m camel_b200.build``); there is no fallback of
any kind: a missing library raises at import of this module, a missing GPU raises at the
first compute call (status CT_ERR_NO_DEVICE).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import os

# CAMEL_TENSOR_LIB: another build of the same library (e.g. one compiled with tracing)
LIB_PATH = Path(os.environ.get("CAMEL_TENSOR_LIB") or Path(__file__).resolve().parent / "libcamel_tensor_b200.so")

# ct_status
OK, ERR_INVALID, ERR_CUDA, ERR_DIV_ZERO, ERR_LOG_DOMAIN, ERR_TIMEOUT, ERR_NO_DEVICE, ERR_TOO_LARGE = range(8)
# ct_dtype
F32, I64, BOOL = 0, 1, 2
# ct_binary_op / ct_compare_op
ADD, SUB, MUL, DIV, POW = range(5)
LT, LE, GT, GE, EQ = range(5)
# ct_activation
ACT_NONE, ACT_RELU, ACT_SOFTMAX = 0, 1, 2
# ct_precision
PREC_3XTF32, PREC_BF16 = 0, 1

_vp, _i64, _u64, _int, _dbl, _sz = C.c_void_p, C.c_int64, C.c_uint64, C.c_int, C.c_double, C.c_size_t

# name -> (restype, argtypes); every symbol of the header, checked by the CPU tests.
PROTOTYPES = {
    "ct_last_error": (C.c_char_p, []),
    "ct_version": (C.c_char_p, []),
    "ct_device_count": (_int, [C.POINTER(_int)]),
    "ct_set_device": (_int, [_int]),
    "ct_get_device": (_int, [C.POINTER(_int)]),
    "ct_set_stream": (_int, [_vp]),
    "ct_sync": (_int, []),
    "ct_check": (_int, []),
    "ct_inject_status": (_int, [_int, C.c_uint32]),
    "ct_measure_mma_peak": (_int, [_int, _int, _int, C.POINTER(_dbl), C.POINTER(_dbl)]),
    "ct_measure_mma_rate_shifted": (_int, [_int, _int, _int, _int, _int, _int, C.POINTER(_dbl), C.POINTER(_dbl)]),
    "ct_measure_mma_rate": (_int, [_int, _int, _int, _int, _int, C.POINTER(_dbl), C.POINTER(_dbl)]),
    "ct_measure_mma_clocks": (_int, [_int, _int, _int, C.POINTER(_dbl), C.POINTER(_dbl)]),
    "ct_launch_count": (_u64, []),
    "ct_profile_enable": (_int, [_int]),
    "ct_profile_read": (_int, [C.c_char_p, C.POINTER(_dbl), C.POINTER(_u64)]),
    "ct_set_precision": (_int, [_int]),
    "ct_get_precision": (_int, []),
    "ct_graph_begin": (_int, []),
    "ct_graph_end": (_int, [C.POINTER(_vp)]),
    "ct_graph_launch": (_int, [_vp]),
    "ct_graph_destroy": (_int, [_vp]),
    "ct_alloc":(_int, [C.POINTER(_vp), _sz]),
    "ct_free": (_int, [_vp]),
    "ct_h2d": (_int, [_vp, _vp, _sz]),
    "ct_d2h": (_int, [_vp, _vp, _sz]),
    "ct_d2h_checked": (_int, [_vp, _vp, _sz]),
    "ct_d2d": (_int, [_vp, _vp, _sz]),
    "ct_host_alloc": (_int, [C.POINTER(_vp), _sz]),
    "ct_host_free": (_int, [_vp]),
    "ct_h2d_async": (_int, [_vp, _vp, _sz]),
    "ct_d2h_async": (_int, [_vp, _vp, _sz]),
    "ct_stream_create": (_int, [C.POINTER(_vp)]),
    "ct_stream_destroy": (_int, [_vp]),
    "ct_event_create": (_int, [C.POINTER(_vp)]),
    "ct_event_destroy": (_int, [_vp]),
    "ct_event_record": (_int, [_vp]),
    "ct_stream_wait_event": (_int, [_vp]),
    "ct_event_sync": (_int, [_vp]),
    "ct_event_elapsed_ms": (_int, [_vp, _vp, C.POINTER(C.c_float)]),
    "ct_result_dtype": (_int, [_int, _int, _int]),
    "ct_binary": (_int, [_int, _int, _vp, _int, _vp, _u64, _vp]),
    "ct_binary_scalar": (_int, [_int, _int, _vp, _dbl, _int, _int, _u64, _vp]),
    "ct_compare": (_int, [_int, _int, _vp, _int, _vp, _u64, _vp]),
    "ct_compare_scalar": (_int, [_int, _int, _vp, _dbl, _int, _u64, _vp]),
    "ct_exp": (_int, [_vp, _u64, _vp]),
    "ct_log": (_int, [_vp, _u64, _vp]),
    "ct_relu": (_int, [_vp, _u64, _vp]),
    "ct_sum": (_int, [_int, _vp, _u64, C.POINTER(_dbl)]),
    "ct_sum_axis": (_int, [_int, _vp, _i64, _i64, _i64, _vp]),
    "ct_max_axis": (_int, [_int, _vp, _i64, _i64, _i64, _vp]),
    "ct_argmax_axis": (_int, [_int, _vp, _i64, _i64, _i64, _vp]),
    "ct_softmax_rows": (_int, [_vp, _i64, _i64, _vp]),
    "ct_transpose": (_int, [_int, _vp, _i64, _i64, _vp]),
    "ct_concat": (_int, [_int, _vp, _vp, _u64, _u64, _u64, _u64, _vp]),
    "ct_fill": (_int, [_int, _dbl, _u64, _vp]),
    "ct_eye": (_int, [_i64, _vp]),
    "ct_arange": (_int, [_i64, _i64, _i64, _vp]),
    "ct_matmul": (_int, [_int, _vp, _int, _vp, _i64, _i64, _i64, _vp]),
    "ct_matmul_tn": (_int, [_vp, _vp, _i64, _i64, _i64, _vp]),
    "ct_scaled_sub": (_int, [_vp, _vp, _dbl, _u64, _vp]),
    "ct_dense": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _int, _vp, _vp]),
    "ct_weights_pack": (_int, [_vp, _i64, _i64, C.POINTER(_vp)]),
    "ct_weights_free": (_int, [_vp]),
    "ct_rows_pack": (_int, [_vp, _i64, _i64, C.POINTER(_vp)]),
    "ct_rows_free": (_int, [_vp]),
    "ct_matmul_packed_rows": (_int, [_vp, _i64, _i64, _vp, _vp]),
    "ct_matmul_packed_bands": (_int, [_vp, _vp, _int, C.POINTER(_i64), C.POINTER(_vp), _vp, C.POINTER(C.c_uint32)]),
    "ct_stream_wait_value": (_int, [_vp, C.c_uint32]),
    "ct_dense_packed": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp, _vp]),
    "ct_conv2d": (_int, [_vp, _vp, _vp] + [_i64] * 9 + [_int, _vp]),
    "ct_conv2d_maxpool2": (_int, [_vp, _vp, _vp] + [_i64] * 9 + [_int, _vp]),
    "ct_maxpool2d": (_int, [_vp, _i64, _i64, _i64, _i64, _i64, _vp]),
    "ct_matmul_f32_static": (_int, [_vp, _vp, _i64, _i64, _i64, _vp, _vp]),
    "ct_matmul_host":(_int, [_vp, _vp, _i64, _i64, _i64, _vp]),
    "ct_binary_host": (_int, [_int, _vp, _vp, _u64, _vp]),
}


class CamelTensorError(RuntimeError):
    """Raised for every non-zero ct_status; ``status`` holds the code."""

    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m camel_b200.build` "
            "(there is no CPU or PyTorch fallback)"
        )
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def check(status: int) -> None:
    if status != OK:
        raise CamelTensorError(status, lib.ct_last_error().decode())
