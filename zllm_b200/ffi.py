"""ctypes binding of ``libzq_b200.so`` (the C ABI declared in ``include/zq_b200.h``).

The CUDA library is the product; this module only loads it and gives the entry points their prototypes.
There is no fallback of any kind: if the library is missing or fails to load, importing raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libzq_b200.so")

Q4_0, Q8_0, Q4_K, Q5_K, Q6_K, IQ4_NL = 2, 8, 12, 13, 14, 20
Q5_0, Q5_1, Q3_K, IQ4_XS = 6, 7, 11, 23
F32, F16, BF16 = 0, 1, 2
JOB_ROW_PARALLEL = 1
ROUTE_SOFTMAX, ROUTE_SIGMOID_BIAS, ROUTE_SQRT_SOFTPLUS_BIAS = 0, 1, 2
MOE_NO_ROUTE = 0xFFFFFFFF  # ZQ_MOE_NO_ROUTE: an expert id that means "no route in this place"
DIST_HANDLE_BYTES = 80
BLOCK = {Q4_0: (32, 18), Q8_0: (32, 34), Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210), IQ4_NL: (32, 18), Q5_0: (32, 22), Q5_1: (32, 24), Q3_K: (256, 110), IQ4_XS: (256, 136)}


class ZqError(C.Structure):
    _fields_ = [("message", C.c_char * 512)]


class ZqFailure(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"zq_b200 error {code}: {message}")
        self.code = code
        self.message = message


_vp, _sz, _u32, _i, _f = C.c_void_p, C.c_size_t, C.c_uint32, C.c_int, C.c_float


class ZqLinearJob(C.Structure):
    """``zq_linear_job``: one projection of a ``zq_linear_batch`` call."""

    _fields_ = [("w", C.c_void_p), ("w_up", C.c_void_p), ("dev_x", C.c_void_p), ("m", C.c_size_t), ("dev_y", C.c_void_p), ("dev_residual", C.c_void_p), ("flags", C.c_uint32)]


class ZqLinearHostJob(C.Structure):
    """``zq_linear_host_job``: one host-buffer projection of a ``zq_linear_host_batch`` call."""

    _fields_ = [("w", C.c_void_p), ("host_x", C.c_void_p), ("m", C.c_size_t), ("host_y", C.c_void_p)]


_err = C.POINTER(ZqError)

PROTOTYPES = {
    "zq_ctx_create": (_i, [_i, C.POINTER(_vp), _err]),
    "zq_ctx_destroy": (None, [_vp]),
    "zq_ctx_set_stream": (_i, [_vp, _vp, _err]),
    "zq_ctx_use_own_stream": (_i, [_vp, _err]),
    "zq_ctx_sync": (_i, [_vp, _err]),
    "zq_ctx_set_option": (_i, [_vp, C.c_char_p, _i, _err]),
    "zq_ctx_sm_count": (_i, [_vp]),
    "zq_ctx_launch_count": (C.c_uint64, [_vp]),
    "zq_weight_prepare": (_i, [_vp, _u32, _vp, _sz, _sz, _sz, C.POINTER(_vp), _err]),
    "zq_weight_prepare_device": (_i, [_vp, _u32, _vp, _sz, _sz, _sz, C.POINTER(_vp), _err]),
    "zq_weight_release": (None, [_vp]),
    "zq_weight_rows": (_sz, [_vp]),
    "zq_weight_cols": (_sz, [_vp]),
    "zq_weight_type": (_u32, [_vp]),
    "zq_weight_gguf_bytes": (_sz, [_vp]),
    "zq_dequantize_f32": (_i, [_vp, _vp, _vp, _err]),
    "zq_gather_rows": (_i, [_vp, _vp, _vp, _sz, _vp, _i, _err]),
    "zq_quantize": (_i, [_vp, _u32, _vp, _sz, _sz, _vp, _sz, _err]),
    "zq_linear": (_i, [_vp, _vp, _vp, _i, _sz, _vp, _i, _vp, _err]),
    "zq_linear_batch": (_i, [_vp, C.POINTER(ZqLinearJob), _sz, _i, _i, _err]),
    "zq_linear_row_parallel": (_i, [_vp, _vp, _vp, _i, _sz, _vp, _i, _vp, _err]),
    "zq_dist_export": (_i, [_vp, _sz, _vp, _err]),
    "zq_dist_init": (_i, [_vp, _i, _i, _vp, _err]),
    "zq_dist_set_wait_ms": (_i, [_vp, C.c_uint, _err]),
    "zq_dist_rank": (_i, [_vp]),
    "zq_dist_world": (_i, [_vp]),
    "zq_dist_shutdown": (None, [_vp]),
    "zq_linear_multi": (_i, [_vp, C.POINTER(_vp), _sz, _vp, _i, _sz, C.POINTER(_vp), _i, _err]),
    "zq_rmsnorm_linear": (_i, [_vp, C.POINTER(_vp), _sz, _vp, _i, _sz, _vp, C.c_float, C.c_float, C.POINTER(_vp), _i, _err]),
    "zq_rope_qk": (_i, [_vp, _vp, _sz, _vp, _sz, _i, _sz, _sz, _sz, _i, _i, _sz, _vp, _vp, _sz, _err]),
    "zq_gated_silu": (_i, [_vp, _vp, _vp, _vp, _i, _sz, _vp, _i, _err]),
    "zq_gated_mlp": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _sz, _vp, _i, _vp, _err]),
    "zq_linear_noalloc": (_i, [_vp, _vp, _vp, _i, _sz, _vp, _i, _err]),
    "zq_linear_host": (_i, [_vp, _vp, _vp, _i, _sz, _vp, _i, _err]),
    "zq_linear_host_batch": (_i, [_vp, _vp, _sz, _i, _i, _err]),
    "zq_batch_begin": (_i, [_vp, _err]),
    "zq_batch_finish": (_i, [_vp, _err]),
    "zq_moe_route_softmax_topk": (_i, [_vp, _vp, _i, _sz, _sz, _vp, _vp, _sz, _sz, _f, _i, _vp, _vp, _err]),
    "zq_moe_route_topk": (_i, [_vp, _i, _vp, _i, _sz, _sz, _vp, _vp, _sz, _sz, _f, _i, _vp, _vp, _err]),
    "zq_moe_gather_rows": (_i, [_vp, _vp, _i, _sz, _sz, _vp, _sz, _vp, _err]),
    "zq_moe_scatter_add_rows": (_i, [_vp, _vp, _i, _vp, _vp, _sz, _sz, _vp, _sz, _err]),
    "zq_moe_experts_create": (_i, [_vp, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp), _sz, C.POINTER(_vp), _err]),
    "zq_moe_experts_destroy": (None, [_vp]),
    "zq_gguf_open": (_i, [C.c_char_p, C.POINTER(_vp), _err]),
    "zq_gguf_close": (None, [_vp]),
    "zq_gguf_tensor_count": (_sz, [_vp]),
    "zq_gguf_tensor_name": (_i, [_vp, _sz, C.c_char_p, _sz, _err]),
    "zq_gguf_tensor_info": (_i, [_vp, C.c_char_p, C.POINTER(_u32), C.POINTER(_u32), C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), _err]),
    "zq_gguf_metadata_u64": (_i, [_vp, C.c_char_p, C.POINTER(C.c_uint64), _err]),
    "zq_gguf_metadata_f64": (_i, [_vp, C.c_char_p, C.POINTER(C.c_double), _err]),
    "zq_gguf_metadata_str": (_i, [_vp, C.c_char_p, C.c_char_p, _sz, _err]),
    "zq_gguf_load_matrix": (_i, [_vp, _vp, C.c_char_p, C.POINTER(_vp), _err]),
    "zq_gguf_load_matrix_slice": (_i, [_vp, _vp, C.c_char_p, _sz, C.POINTER(_vp), _err]),
    "zq_argmax_rows": (_i, [_vp, _vp, _i, _sz, _sz, _vp, _err]),
    "zq_lm_head_argmax": (_i, [_vp, _vp, _vp, _i, _sz, _vp, _err]),
    "zq_moe_ep_export": (_i, [_vp, _sz, _sz, _sz, _sz, _i, _vp, _err]),
    "zq_moe_ep_init": (_i, [_vp, _vp, _err]),
    "zq_moe_ep_shutdown": (None, [_vp]),
    "zq_moe_forward_ep": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _sz, _sz, _vp, _vp, _sz, _vp, _i, _vp, _err]),
    "zq_moe_forward": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _sz, _vp, _vp, _sz, _vp, _i, _vp, _err]),
}

_lib = None


def load() -> C.CDLL:
    """Load the CUDA library (built in-tree by ``zllm_b200.build``)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m zllm_b200.build` (there is no fallback path)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def call(name: str, *args):
    """Call an entry point that returns a status code and takes a trailing ``zq_error*``."""
    err = ZqError()
    rc = getattr(load(), name)(*args, C.byref(err))
    if rc != 0:
        raise ZqFailure(rc, err.message.decode("utf-8", "replace"))
    return rc
