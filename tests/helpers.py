"""Shared test-input generators (numpy).  Encoders for Q8_0 / Q4_0 / IQ4_NL are input generators only: the
reference has no encoder for these types and parity is defined on bytes -> values."""
from __future__ import annotations

import numpy as np

from oracle import oracle as orc

Q4_0, Q8_0, Q4_K, Q5_K, Q6_K, IQ4_NL = orc.Q4_0, orc.Q8_0, orc.Q4_K, orc.Q5_K, orc.Q6_K, orc.IQ4_NL
Q5_0, Q5_1, Q3_K, IQ4_XS = orc.Q5_0, orc.Q5_1, orc.Q3_K, orc.IQ4_XS
# byte offsets of the f16 scale fields of a block, per type
SCALE_OFFSETS = {Q4_0: (0,), Q8_0: (0,), IQ4_NL: (0,), Q4_K: (0, 2), Q5_K: (0, 2), Q6_K: (208,), Q5_0: (0,), Q5_1: (0, 2), Q3_K: (108,), IQ4_XS: (0,)}
F16_EDGE_SCALES = [0x0000, 0x0001, 0x03FF, 0x0400, 0x0401, 0x13FF, 0x17FF, 0x8401]


def f16_bytes(value: float) -> bytes:
    return np.float16(value).tobytes()


def reference_packed_blocks(tensor_type: int, rows: int) -> np.ndarray:
    """The deterministic generator of the reference's CPU tests (src/kernel/cpu/ggml_quant.rs:370-414),
    types 8, 12, 13, 14: eight Q8_0 blocks or one K-quant super-block per row."""
    block_bytes = {8: 34, 12: 144, 13: 176, 14: 210}[tensor_type]
    per_row = 8 if tensor_type == 8 else 1
    out = np.zeros(rows * per_row * block_bytes, dtype=np.uint8)
    for bi in range(rows * per_row):
        row = bi // per_row
        b = out[bi * block_bytes:(bi + 1) * block_bytes]
        if tensor_type == 8:
            b[:2] = np.frombuffer(f16_bytes(0.03125), dtype=np.uint8)
            idx = np.arange(32, dtype=np.int64)
            b[2:] = ((idx * 7 + ((row * 3) & 0xFF)) & 0xFF).astype(np.uint8)  # i8 wrapping arithmetic
        elif tensor_type == 14:
            idx = np.arange(192, dtype=np.int64)
            b[:192] = ((idx * 37 + row * 11) & 0xFF).astype(np.uint8)
            idx = np.arange(16, dtype=np.int64)
            b[192:208] = ((idx % 9) - 4).astype(np.int8).view(np.uint8)
            b[208:210] = np.frombuffer(f16_bytes(0.03125), dtype=np.uint8)
        else:
            b[:2] = np.frombuffer(f16_bytes(0.0625), dtype=np.uint8)
            b[2:4] = np.frombuffer(f16_bytes(0.03125), dtype=np.uint8)
            b[4:16] = 0x11
            idx = np.arange(block_bytes - 16, dtype=np.int64)
            b[16:] = ((idx * 29 + row * 7) & 0xFF).astype(np.uint8)
    return out


def _f16_round(a: np.ndarray) -> np.ndarray:
    return a.astype(np.float16).astype(np.float32)


def quantize_q8_0(values: np.ndarray) -> np.ndarray:
    v = np.ascontiguousarray(values, dtype=np.float32).reshape(-1, 32)
    d = _f16_round(np.abs(v).max(axis=1) / 127.0)
    inv = np.where(d > 0, 1.0 / np.where(d > 0, d, 1.0), 0.0).astype(np.float32)
    q = np.clip(np.rint(v * inv[:, None]), -127, 127).astype(np.int8)
    out = np.zeros((v.shape[0], 34), dtype=np.uint8)
    out[:, :2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def _nearest_code(scaled: np.ndarray, codebook: np.ndarray) -> np.ndarray:
    return np.abs(scaled[..., None] - codebook[None, None, :].astype(np.float32)).argmin(axis=-1).astype(np.uint8)


def _pack_nibbles(d: np.ndarray, codes: np.ndarray) -> np.ndarray:
    out = np.zeros((codes.shape[0], 18), dtype=np.uint8)
    out[:, :2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = codes[:, :16] | (codes[:, 16:] << 4)
    return out.reshape(-1)


def quantize_q4_0(values: np.ndarray) -> np.ndarray:
    v = np.ascontiguousarray(values, dtype=np.float32).reshape(-1, 32)
    idx = np.abs(v).argmax(axis=1)
    signed_max = v[np.arange(v.shape[0]), idx]
    d = _f16_round(signed_max / -8.0)
    inv = np.where(d != 0, 1.0 / np.where(d != 0, d, 1.0), 0.0).astype(np.float32)
    codes = _nearest_code(v * inv[:, None], np.arange(-8, 8))
    return _pack_nibbles(d, codes)


def quantize_iq4_nl(values: np.ndarray) -> np.ndarray:
    v = np.ascontiguousarray(values, dtype=np.float32).reshape(-1, 32)
    idx = np.abs(v).argmax(axis=1)
    signed_max = v[np.arange(v.shape[0]), idx]
    d = _f16_round(signed_max / -127.0)
    inv = np.where(d != 0, 1.0 / np.where(d != 0, d, 1.0), 0.0).astype(np.float32)
    codes = _nearest_code(v * inv[:, None], orc.KVALUES_IQ4NL)
    return _pack_nibbles(d, codes)


def quantize(tensor_type: int, values: np.ndarray) -> np.ndarray:
    if tensor_type == Q4_K:
        return orc.encode_q4_k(values)
    return {Q8_0: quantize_q8_0, Q4_0: quantize_q4_0, IQ4_NL: quantize_iq4_nl}[tensor_type](values)


def random_weight(tensor_type: int, rows: int, cols: int, seed: int, std: float = 0.02) -> np.ndarray:
    if tensor_type in (Q5_K, Q6_K, Q5_0, Q5_1, Q3_K, IQ4_XS):
        return random_kquant_weight(tensor_type, rows, cols, seed)
    rng = np.random.default_rng(seed)
    return quantize(tensor_type, rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(std))


def random_bytes_weight(tensor_type: int, rows: int, cols: int, seed: int) -> np.ndarray:
    """Uniformly random payload bytes with finite random f16 scales: exercises every code and scale pattern."""
    rng = np.random.default_rng(seed)
    e, b = orc.BLOCK[tensor_type]
    blocks = rows * cols // e
    out = rng.integers(0, 256, size=(blocks, b), dtype=np.uint8)
    for off in SCALE_OFFSETS[tensor_type]:
        bits = rng.integers(0, 0x7C00, size=blocks, dtype=np.uint16) | (rng.integers(0, 2, size=blocks, dtype=np.uint16) << 15)
        out[:, off:off + 2] = bits.view(np.uint8).reshape(-1, 2)
    return out.reshape(-1)


def random_kquant_weight(tensor_type: int, rows: int, cols: int, seed: int) -> np.ndarray:
    """Q5_K / Q6_K input generator (the reference has no encoder for them): uniformly random payload and scale-code
    bytes under small positive f16 super-block scales, so that every code occurs and the values stay in the range of
    real tensors."""
    rng = np.random.default_rng(seed)
    e, b = orc.BLOCK[tensor_type]
    blocks = rows * cols // e
    out = rng.integers(0, 256, size=(blocks, b), dtype=np.uint8)
    # super-block scales of K-quants multiply 6-bit sub-scales; block-32 scales multiply the codes directly
    lo, hi = ((2.0e-4, 6.0e-4) if tensor_type in (Q5_K, Q6_K, Q3_K, IQ4_XS) else (2.0e-3, 6.0e-3))
    for off in SCALE_OFFSETS[tensor_type]:
        d = rng.uniform(lo, hi, size=blocks).astype(np.float16)
        out[:, off:off + 2] = d.view(np.uint8).reshape(-1, 2)
    return out.reshape(-1)


def max_rel_error(actual: np.ndarray, expected: np.ndarray) -> float:
    """max_i |a_i - e_i| / max(|e_i|, rms(e)): the layer-output error metric (bound 2e-3)."""
    a = np.asarray(actual, dtype=np.float64).reshape(-1)
    e = np.asarray(expected, dtype=np.float64).reshape(-1)
    rms = np.sqrt(np.mean(e * e)) if e.size else 0.0
    denom = np.maximum(np.abs(e), max(rms, 1e-30))
    return float(np.max(np.abs(a - e) / denom)) if e.size else 0.0
