"""GPU parity of the codec: dequantised values bit-exact against the CPU oracle (through the C ABI)."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import helpers as H
from tests.gpu_util import ctx, dev, host

pytestmark = pytest.mark.gpu
TYPES = [H.Q4_0, H.Q8_0, H.Q4_K, H.Q5_K, H.Q6_K, H.IQ4_NL, H.Q5_0, H.Q5_1, H.Q3_K, H.IQ4_XS]


def _bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.mark.parametrize("tensor_type", TYPES)
@pytest.mark.parametrize("rows,cols", [(3, 256), (37, 1024), (130, 512), (5, 4096)])
def test_dequantize_is_bit_exact_on_random_bytes(tensor_type, rows, cols):
    data = H.random_bytes_weight(tensor_type, rows, cols, seed=rows * 7 + cols)
    w = ctx().prepare_weight(tensor_type, data, rows, cols)
    got = host(ctx().dequantize(w))
    want = orc.dequantize(tensor_type, data, rows * cols).reshape(rows, cols)
    assert np.array_equal(_bits(got), _bits(want))


@pytest.mark.parametrize("tensor_type", [H.Q4_0, H.Q8_0, H.IQ4_NL, H.Q5_0, H.Q5_1])
@pytest.mark.parametrize("cols", [32, 1056, 2560])
def test_dequantize_handles_rows_that_are_not_whole_units(tensor_type, cols):
    """Column counts of the reference's Q8_0 test (src/kernel/cuda/linear.rs:2209-2230): 32-aligned, not 256-aligned."""
    rows = 9
    data = H.random_bytes_weight(tensor_type, rows, cols, seed=cols)
    w = ctx().prepare_weight(tensor_type, data, rows, cols)
    got = host(ctx().dequantize(w))
    want = orc.dequantize(tensor_type, data, rows * cols).reshape(rows, cols)
    assert np.array_equal(_bits(got), _bits(want))


def test_q4_k_every_finite_f16_scale_pattern_decodes_bit_exactly():
    """All 63 488 finite f16 patterns as d and dmin, crossed with every 6-bit code and nibble through random payloads."""
    finite = np.array([b for b in range(65536) if (b & 0x7C00) != 0x7C00], dtype=np.uint16)
    rng = np.random.default_rng(1)
    blocks = finite.size
    data = rng.integers(0, 256, size=(blocks, 144), dtype=np.uint8)
    data[:, 0:2] = finite.view(np.uint8).reshape(-1, 2)
    data[:, 2:4] = rng.permutation(finite).view(np.uint8).reshape(-1, 2)
    rows, cols = blocks // 8, 2048
    data = data[: rows * 8].reshape(-1)
    w = ctx().prepare_weight(H.Q4_K, data, rows, cols)
    got = host(ctx().dequantize(w))
    want = orc.dequantize(H.Q4_K, data, rows * cols).reshape(rows, cols)
    assert np.array_equal(_bits(got), _bits(want))


@pytest.mark.parametrize("tensor_type", TYPES)
def test_f16_edge_scales(tensor_type):
    """Zero, smallest subnormal, subnormal edge, non-powers of two and a negative scale (src/kernel/rocm/hip/linear/gguf.rs:869)."""
    e, b = orc.BLOCK[tensor_type]
    rng = np.random.default_rng(2)
    n = len(H.F16_EDGE_SCALES)
    per_row = 256 // e
    data = rng.integers(0, 256, size=(n * per_row, b), dtype=np.uint8)
    for i, bits in enumerate(H.F16_EDGE_SCALES):
        for j in range(per_row):
            offs = H.SCALE_OFFSETS[tensor_type]
            data[i * per_row + j, offs[0]:offs[0] + 2] = np.frombuffer(np.uint16(bits).tobytes(), dtype=np.uint8)
            if len(offs) > 1:
                data[i * per_row + j, offs[1]:offs[1] + 2] = np.frombuffer(np.uint16(H.F16_EDGE_SCALES[(i + 3) % n]).tobytes(), dtype=np.uint8)
    data = data.reshape(-1)
    w = ctx().prepare_weight(tensor_type, data, n, 256)
    got = host(ctx().dequantize(w))
    want = orc.dequantize(tensor_type, data, n * 256).reshape(n, 256)
    assert np.array_equal(_bits(got), _bits(want))


def test_reference_known_answers_through_the_device_path():
    """src/weight/codec/ggml.rs:513-537, 593-597 decoded by the CUDA kernels."""
    block = np.zeros((8, 18), dtype=np.uint8)
    block[:, :2] = np.frombuffer(H.f16_bytes(0.5), dtype=np.uint8)
    block[0, 2] = 0x0F
    block[0, 3] = 0x98
    out = host(ctx().dequantize(ctx().prepare_weight(H.IQ4_NL, block.reshape(-1), 1, 256)))[0]
    assert out[0] == 0.5 * 113.0 and out[16] == 0.5 * -127.0 and out[1] == 0.5 and out[17] == 0.5 * 13.0
    q8 = np.zeros((8, 34), dtype=np.uint8)
    q8[0, :2] = [0x00, 0x40]
    q8[0, 2] = np.int8(-3).view(np.uint8)
    q8[0, 3] = 4
    out = host(ctx().dequantize(ctx().prepare_weight(H.Q8_0, q8.reshape(-1), 1, 256)))[0]
    assert list(out[:2]) == [-6.0, 8.0]
    q4 = np.zeros(144, dtype=np.uint8)
    q4[:2] = [0x00, 0x3C]
    q4[4] = 1
    q4[16] = 2
    out = host(ctx().dequantize(ctx().prepare_weight(H.Q4_K, q4, 1, 256)))[0]
    assert out[0] == 2.0
    q5 = np.zeros(176, dtype=np.uint8)  # src/weight/codec/ggml.rs:577-604, Q5_K and Q6_K cases
    q5[:2] = [0x00, 0x3C]
    q5[4] = 1
    q5[16] = 1
    q5[48] = 2
    assert host(ctx().dequantize(ctx().prepare_weight(H.Q5_K, q5, 1, 256)))[0][0] == 18.0
    q6 = np.zeros(210, dtype=np.uint8)
    q6[192] = 1
    q6[208:] = [0x00, 0x3C]
    assert host(ctx().dequantize(ctx().prepare_weight(H.Q6_K, q6, 1, 256)))[0][0] == -32.0


def test_reference_known_answers_of_the_operand_pass_types():
    """src/weight/codec/ggml.rs:483-511, 578-585, 616-625 (Q5_0, Q5_1, Q3_K, IQ4_XS) decoded by the CUDA kernels."""
    b = np.zeros((1, 22), dtype=np.uint8)
    b[0, :2] = np.frombuffer(H.f16_bytes(0.5), dtype=np.uint8)
    b[0, 2:6] = np.frombuffer(np.uint32(0xFFFF0000).tobytes(), dtype=np.uint8)
    for i in range(16):
        b[0, 6 + i] = i | ((15 - i) << 4)
    out = host(ctx().dequantize(ctx().prepare_weight(H.Q5_0, b.reshape(-1), 1, 32)))[0]
    assert all(out[i] == (i - 16.0) * 0.5 and out[16 + i] == (15 - i) * 0.5 for i in range(16))
    b = np.zeros((1, 24), dtype=np.uint8)
    b[0, :2] = np.frombuffer(H.f16_bytes(0.25), dtype=np.uint8)
    b[0, 2:4] = np.frombuffer(H.f16_bytes(-3.0), dtype=np.uint8)
    b[0, 4:8] = np.frombuffer(np.uint32(0xFFFF0000).tobytes(), dtype=np.uint8)
    for i in range(16):
        b[0, 8 + i] = i | (i << 4)
    out = host(ctx().dequantize(ctx().prepare_weight(H.Q5_1, b.reshape(-1), 1, 32)))[0]
    assert all(out[i] == i * 0.25 - 3.0 for i in range(32))
    q3 = np.zeros(110, dtype=np.uint8)
    q3[0], q3[32], q3[96], q3[104] = 1, 3, 1, 2
    q3[108:] = [0x00, 0x3C]
    assert host(ctx().dequantize(ctx().prepare_weight(H.Q3_K, q3, 1, 256)))[0][0] == 3.0
    xs = np.zeros(136, dtype=np.uint8)
    xs[:2] = [0x00, 0x3C]
    xs[2:4] = [2, 0]
    xs[4] = 1
    xs[8] = 0xF0
    out = host(ctx().dequantize(ctx().prepare_weight(H.IQ4_XS, xs, 1, 256)))[0]
    assert out[0] == -127.0 and out[16] == 113.0


@pytest.mark.parametrize("tensor_type", [H.Q5_0, H.Q5_1, H.Q3_K, H.IQ4_XS])
@pytest.mark.parametrize("m", [1, 5, 40])
def test_operand_pass_types_run_the_linear_layer(tensor_type, m):
    """Q5_0, Q5_1, Q3_K and IQ4_XS have no decode kernel: every projection is the f16 operand pass and the tensor-core GEMM
    (2e-3 against the CPU path, which decodes each block and takes an f32 dot product)."""
    rows, cols = 192, 1024
    data = H.random_weight(tensor_type, rows, cols, seed=40 + m)
    x = np.random.default_rng(m).standard_normal((m, cols)).astype(np.float32)
    xb = dev(x, torch.bfloat16)
    w = ctx().prepare_weight(tensor_type, data, rows, cols)
    got = host(ctx().linear(xb, w, out_dtype=torch.float32))
    want = orc.linear(tensor_type, data, rows, cols, xb.float().cpu().numpy())
    assert H.max_rel_error(got, want) <= 2e-3


@pytest.mark.parametrize("tensor_type", [H.Q8_0, H.IQ4_NL, H.Q4_K, H.Q5_K, H.Q6_K, H.Q5_0, H.IQ4_XS])
def test_gather_rows_equals_f16_of_dequant(tensor_type):
    """src/kernel/cuda/linear.rs:2156-2173: gathered rows == f16(dequant) exactly."""
    rows, cols = 50, 512
    data = H.random_weight(tensor_type, rows, cols, seed=5)
    w = ctx().prepare_weight(tensor_type, data, rows, cols)
    ids = np.array([49, 0, 7, 7, 23], dtype=np.int32)
    got = ctx().gather_rows(w, torch.from_numpy(ids), dtype=torch.float16)
    ctx().sync()
    want = orc.dequantize(tensor_type, data, rows * cols).reshape(rows, cols)[ids].astype(np.float16)
    assert np.array_equal(got.cpu().numpy().view(np.uint16), want.view(np.uint16))


def test_gather_rows_reports_bad_row_ids_without_faulting():
    from zllm_b200 import ffi

    rows, cols = 4, 256
    w = ctx().prepare_weight(H.Q8_0, H.random_weight(H.Q8_0, rows, cols, seed=6), rows, cols)
    ctx().gather_rows(w, torch.tensor([1, 99], dtype=torch.int32), dtype=torch.float32)
    with pytest.raises(ffi.ZqFailure):
        ctx().sync()
    ctx().sync()  # the status word is cleared once reported


def test_quantize_q4_k_matches_reference_encoder_bit_for_bit():
    """encode_q4_k (src/weight/codec/ggml.rs:188-227) on the device against the oracle restatement."""
    rng = np.random.default_rng(7)
    v = (rng.standard_normal((24, 1024)) * 0.02).astype(np.float32)
    v[0, :256] = 0.0            # all-zero block: d == dmin == 0 branch
    v[1, :32] = np.abs(v[1, :32])  # all-positive group: min clamps to 0
    got = ctx().quantize(H.Q4_K, dev(v))
    ctx().sync()
    want = orc.encode_q4_k(v)
    assert np.array_equal(got.cpu().numpy(), want)


@pytest.mark.parametrize("tensor_type", [H.Q8_0, H.Q4_0, H.IQ4_NL])
def test_block32_encoders_match_the_test_generators(tensor_type):
    rng = np.random.default_rng(8)
    v = (rng.standard_normal((16, 512)) * 0.02).astype(np.float32)
    got = ctx().quantize(tensor_type, dev(v))
    ctx().sync()
    got = got.cpu().numpy()
    want = H.quantize(tensor_type, v)
    back_got = orc.dequantize(tensor_type, got, v.size)
    back_want = orc.dequantize(tensor_type, want, v.size)
    # same algorithm; allow rare ties to resolve differently, but the reconstruction must be as good
    assert np.mean(got != want) < 1e-3
    assert abs(np.abs(back_got - v.ravel()).max() - np.abs(back_want - v.ravel()).max()) < 1e-4


def test_prepare_weight_rejects_wrong_sizes():
    """Byte-count and alignment mismatches are errors (src/kernel/cuda/linear.rs:1441-1444)."""
    from zllm_b200 import ffi

    with pytest.raises(ffi.ZqFailure):
        ctx().prepare_weight(H.Q4_K, np.zeros(143, dtype=np.uint8), 1, 256)
    with pytest.raises(ffi.ZqFailure):
        ctx().prepare_weight(H.Q4_K, np.zeros(144, dtype=np.uint8), 1, 255)
    with pytest.raises(ffi.ZqFailure):
        ctx().prepare_weight(10, np.zeros(84, dtype=np.uint8), 1, 256)  # Q2_K: not a type of this path
