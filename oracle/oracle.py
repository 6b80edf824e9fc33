"""ctypes binding of the CPU oracle (``oracle/zq_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline /
reference legs of ``bench.py``.  The product package never imports this module.

Parity pin: the oracle is checked against the reference's own known-answer unit tests
(``tests/test_oracle_kat.py``); the Rust reference itself cannot be built in this environment.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "build", "libzq_oracle.so")

Q4_0, Q8_0, Q4_K, Q5_K, Q6_K, IQ4_NL = 2, 8, 12, 13, 14, 20
Q5_0, Q5_1, Q3_K, IQ4_XS = 6, 7, 11, 23
BLOCK = {Q4_0: (32, 18), Q8_0: (32, 34), Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210), IQ4_NL: (32, 18), Q5_0: (32, 22), Q5_1: (32, 24), Q3_K: (256, 110), IQ4_XS: (256, 136)}
KVALUES_IQ4NL = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], dtype=np.int8)


def build(force: bool = False) -> str:
    """Compile the oracle with gcc (``make -C oracle``) unless the library is already up to date."""
    src = os.path.join(_HERE, "zq_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE] + (["-B"] if force else []), check=True, capture_output=True)
    return _LIB_PATH


class _Matrix(C.Structure):
    _fields_ = [("tensor_type", C.c_uint32), ("bytes", C.c_void_p), ("nbytes", C.c_size_t), ("rows", C.c_size_t), ("columns", C.c_size_t)]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.zqo_f16_to_f32.restype = C.c_float
        _lib.zqo_f16_to_f32.argtypes = [C.c_uint16]
        _lib.zqo_f32_to_f16.restype = C.c_uint16
        _lib.zqo_f32_to_f16.argtypes = [C.c_float]
    return _lib


def _u8(a) -> np.ndarray:
    return np.ascontiguousarray(np.frombuffer(a, dtype=np.uint8) if isinstance(a, (bytes, bytearray)) else a, dtype=np.uint8)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


class OracleError(ValueError):
    pass


def _check(rc: int, what: str):
    if rc != 0:
        raise OracleError(f"{what}: shape or byte-count mismatch (code {rc})")


def set_threads(n: int):
    lib().zqo_set_threads(C.c_int(n))


def threads() -> int:
    return lib().zqo_get_threads()


def row_bytes(tensor_type: int, columns: int) -> int:
    e, b = BLOCK[tensor_type]
    if columns % e:
        raise OracleError(f"columns={columns} not aligned to block {e}")
    return columns // e * b


def dequantize(tensor_type: int, data, elements: int) -> np.ndarray:
    data = _u8(data)
    out = np.empty(elements, dtype=np.float32)
    _check(lib().zqo_dequantize(C.c_uint32(tensor_type), _p(data), C.c_size_t(data.size), C.c_size_t(elements), _p(out)), "dequantize")
    return out


def encode_q4_k(values) -> np.ndarray:
    """Reference ``encode_q4_k`` over a flat f32 array whose length is a multiple of 256."""
    values = _f32(values).reshape(-1)
    if values.size % 256:
        raise OracleError("encode_q4_k needs a multiple of 256 values")
    out = np.empty(values.size // 256 * 144, dtype=np.uint8)
    fn = lib().zqo_encode_q4_k
    for block in range(values.size // 256):
        fn(C.c_void_p(values.ctypes.data + block * 1024), C.c_void_p(out.ctypes.data + block * 144))
    return out


def requantize_q4_k(tensor_type: int, data, elements: int) -> np.ndarray:
    data = _u8(data)
    out = np.empty(elements // 256 * 144, dtype=np.uint8)
    _check(lib().zqo_requantize_q4_k(C.c_uint32(tensor_type), _p(data), C.c_size_t(data.size), C.c_size_t(elements), _p(out)), "requantize_q4_k")
    return out


def matvec(tensor_type, data, rows, columns, x, out_len=None) -> np.ndarray:
    data, x = _u8(data), _f32(x).reshape(-1)
    out = np.zeros(rows if out_len is None else out_len, dtype=np.float32)
    _check(lib().zqo_matvec(C.c_uint32(tensor_type), _p(data), C.c_size_t(data.size), C.c_size_t(rows), C.c_size_t(columns), _p(x), C.c_size_t(x.size), _p(out), C.c_size_t(out.size)), "matvec")
    return out


def matvec_residual(tensor_type, data, rows, columns, x, residual) -> np.ndarray:
    data, x, residual = _u8(data), _f32(x).reshape(-1), _f32(residual).reshape(-1)
    out = np.zeros(rows, dtype=np.float32)
    _check(lib().zqo_matvec_residual(C.c_uint32(tensor_type), _p(data), C.c_size_t(data.size), C.c_size_t(rows), C.c_size_t(columns), _p(x), C.c_size_t(x.size), _p(out), C.c_size_t(out.size), _p(residual), C.c_size_t(residual.size)), "matvec_residual")
    return out


def gated_silu_matvec(tensor_type, gate, up, rows, columns, x) -> np.ndarray:
    gate, up, x = _u8(gate), _u8(up), _f32(x).reshape(-1)
    out = np.zeros(rows, dtype=np.float32)
    _check(lib().zqo_gated_silu_matvec(C.c_uint32(tensor_type), _p(gate), C.c_size_t(gate.size), _p(up), C.c_size_t(up.size), C.c_size_t(rows), C.c_size_t(columns), _p(x), C.c_size_t(x.size), _p(out), C.c_size_t(out.size)), "gated_silu_matvec")
    return out


def matmul(tensor_type, data, rows, columns, x) -> np.ndarray:
    """Y[M, rows] for X[M, columns] (reference layout ``out[token*rows + row]``)."""
    data, x = _u8(data), _f32(x)
    m = x.size // columns if columns else 0
    out = np.zeros((m, rows), dtype=np.float32)
    _check(lib().zqo_matmul(C.c_uint32(tensor_type), _p(data), C.c_size_t(data.size), C.c_size_t(rows), C.c_size_t(columns), C.c_size_t(m), _p(x), C.c_size_t(x.size), _p(out), C.c_size_t(out.size)), "matmul")
    return out


def gated_silu_matmul(tensor_type, gate, up, rows, columns, x) -> np.ndarray:
    gate, up, x = _u8(gate), _u8(up), _f32(x)
    m = x.size // columns
    out = np.zeros((m, rows), dtype=np.float32)
    _check(lib().zqo_gated_silu_matmul(C.c_uint32(tensor_type), _p(gate), C.c_size_t(gate.size), _p(up), C.c_size_t(up.size), C.c_size_t(rows), C.c_size_t(columns), C.c_size_t(m), _p(x), C.c_size_t(x.size), _p(out), C.c_size_t(out.size)), "gated_silu_matmul")
    return out


def linear(tensor_type, data, rows, columns, x) -> np.ndarray:
    """``CpuContext::linear``: matvec for one token row, matmul for several."""
    data, x = _u8(data), _f32(x).reshape(-1, columns)
    out = np.zeros((x.shape[0], rows), dtype=np.float32)
    _check(lib().zqo_linear(C.c_uint32(tensor_type), _p(data), C.c_size_t(data.size), C.c_size_t(rows), C.c_size_t(columns), C.c_size_t(x.shape[0]), _p(x), _p(out)), "linear")
    return out


def gated_linear(tensor_type, gate, up, rows, columns, x) -> np.ndarray:
    gate, up, x = _u8(gate), _u8(up), _f32(x).reshape(-1, columns)
    out = np.zeros((x.shape[0], rows), dtype=np.float32)
    _check(lib().zqo_gated_linear(C.c_uint32(tensor_type), _p(gate), C.c_size_t(gate.size), _p(up), C.c_size_t(up.size), C.c_size_t(rows), C.c_size_t(columns), C.c_size_t(x.shape[0]), _p(x), _p(out)), "gated_linear")
    return out


def silu_mul(gate, up) -> np.ndarray:
    gate, up = _f32(gate).reshape(-1), _f32(up).reshape(-1)
    out = np.empty_like(gate)
    lib().zqo_silu_mul(_p(gate), _p(up), _p(out), C.c_size_t(gate.size))
    return out


def rope(data, head_count, rotary_dim, position, cos, sin, layout=0, placement=0) -> np.ndarray:
    """attention::rope::apply_f32 (src/attention/rope.rs:120-165) on ``data`` [rows, columns]; returns a new array.
    layout 0 = split-half, 1 = interleaved; placement 0 = prefix, 1 = suffix."""
    out = np.array(data, dtype=np.float32, order="C", copy=True)
    rows, columns = out.shape
    cos, sin = _f32(cos).reshape(-1), _f32(sin).reshape(-1)
    if cos.size != sin.size:
        raise OracleError("rope: cos and sin tables differ in length")
    _check(lib().zqo_rope(_p(out), C.c_size_t(rows), C.c_size_t(columns), C.c_size_t(head_count), C.c_size_t(rotary_dim), C.c_size_t(position), _p(cos), _p(sin), C.c_size_t(cos.size), C.c_int(layout), C.c_int(placement)), "rope")
    return out


def route_softmax_logits(logits, top_k, scaling_factor=1.0, normalize_selected=True):
    logits = _f32(logits).reshape(-1)
    ids = np.zeros(top_k, dtype=np.uint32)
    w = np.zeros(top_k, dtype=np.float32)
    _check(lib().zqo_route_softmax_logits(_p(logits), C.c_size_t(logits.size), C.c_size_t(top_k), C.c_float(scaling_factor), C.c_int(int(normalize_selected)), _p(ids), _p(w)), "route_softmax_logits")
    return ids, w


def router_logits(x_row, router) -> np.ndarray:
    """kernel::cpu::moe::router_logits (src/kernel/cpu/moe.rs:38-55) for one token."""
    x_row, router = _f32(x_row).reshape(-1), _f32(router)
    out = np.zeros(router.shape[0], dtype=np.float32)
    lib().zqo_router_logits(_p(x_row), _p(router), C.c_size_t(x_row.size), C.c_size_t(router.shape[0]), _p(out))
    return out


def route_bias_corrected_logits(logits, bias, top_k, scaling_factor=1.0, kind=1):
    """route_sigmoid_bias_logits (kind 1) / route_sqrt_softplus_bias_logits (kind 2), src/moe/routing.rs:43-81, one row."""
    logits, bias = _f32(logits).reshape(-1), _f32(bias).reshape(-1)
    if logits.size != bias.size:
        raise OracleError("router: logits and bias differ in length")
    ids = np.zeros(top_k, dtype=np.uint32)
    w = np.zeros(top_k, dtype=np.float32)
    _check(lib().zqo_route_bias_corrected_logits(_p(logits), _p(bias), C.c_size_t(logits.size), C.c_size_t(top_k), C.c_float(scaling_factor), C.c_int(kind), _p(ids), _p(w)), "route_bias_corrected_logits")
    return ids, w


def moe_route_softmax(x, router, top_k, scaling_factor=1.0, normalize_selected=True):
    x, router = _f32(x), _f32(router)
    rows, hidden = x.shape
    experts = router.shape[0]
    ids = np.zeros((rows, top_k), dtype=np.uint32)
    w = np.zeros((rows, top_k), dtype=np.float32)
    _check(lib().zqo_moe_route_softmax(_p(x), C.c_size_t(rows), C.c_size_t(hidden), _p(router), C.c_size_t(experts), C.c_size_t(top_k), C.c_float(scaling_factor), C.c_int(int(normalize_selected)), _p(ids), _p(w)), "moe_route_softmax")
    return ids, w


def group_routing(expert_ids, weights, top_k, expert_count):
    """Token-major stable grouping; returns CSR ``(offsets[E+1], tokens[routes], route_weights[routes])``."""
    expert_ids = np.ascontiguousarray(expert_ids, dtype=np.uint32).reshape(-1)
    weights = _f32(weights).reshape(-1)
    if expert_ids.size != weights.size:
        raise OracleError("router shape mismatch")
    offsets = np.zeros(expert_count + 1, dtype=np.uint32)
    tokens = np.zeros(expert_ids.size, dtype=np.uint32)
    rw = np.zeros(expert_ids.size, dtype=np.float32)
    _check(lib().zqo_group_routing(_p(expert_ids), _p(weights), C.c_size_t(expert_ids.size), C.c_size_t(top_k), C.c_size_t(expert_count), _p(offsets), _p(tokens), _p(rw)), "group_routing")
    return offsets, tokens, rw


def _matrices(items):
    keep = []
    arr = (_Matrix * len(items))()
    for i, (t, data, rows, cols) in enumerate(items):
        data = _u8(data)
        keep.append(data)
        arr[i] = _Matrix(t, data.ctypes.data, data.size, rows, cols)
    return arr, keep


def moe_forward(gates, ups, downs, x, expert_ids, weights, shared=None, residual=None) -> np.ndarray:
    """Routed (+ shared, + residual) MoE layer.  ``gates/ups/downs``: lists of ``(type, bytes, rows, cols)``."""
    x = _f32(x)
    rows, hidden = x.shape
    expert_ids = np.ascontiguousarray(expert_ids, dtype=np.uint32)
    weights = _f32(weights)
    top_k = expert_ids.size // rows
    g, k1 = _matrices(gates)
    u, k2 = _matrices(ups)
    d, k3 = _matrices(downs)
    sg = su = sd = None
    keep = []
    if shared is not None:
        (sga, ka), (sua, kb), (sda, kc) = _matrices([shared[0]]), _matrices([shared[1]]), _matrices([shared[2]])
        keep += [sga, sua, sda, ka, kb, kc]
        sg, su, sd = C.byref(sga[0]), C.byref(sua[0]), C.byref(sda[0])
    res = _f32(residual) if residual is not None else None
    out = np.zeros((rows, hidden), dtype=np.float32)
    _check(lib().zqo_moe_forward(g, u, d, C.c_size_t(len(gates)), sg, su, sd, _p(x), C.c_size_t(rows), C.c_size_t(hidden), _p(expert_ids), _p(weights), C.c_size_t(top_k), _p(res) if res is not None else None, _p(out)), "moe_forward")
    return out


def f16_to_f32(bits: int) -> float:
    return float(lib().zqo_f16_to_f32(C.c_uint16(bits)))


def f32_to_f16(value: float) -> int:
    return int(lib().zqo_f32_to_f16(C.c_float(value)))
