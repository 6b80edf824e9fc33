"""GPU parity of the prefill GEMM (tcgen05 path, more than 16 activation rows) against the CPU oracle.

Tolerance: max_i |a_i - e_i| / max(|e_i|, rms(e)) <= 2e-3.  The tensor-core path rounds dequantised weights and
activations to f16 once (2^-12 relative each) and accumulates in f32; the oracle consumes the same activation
values the device consumes (bf16/f16 inputs are exact in f16).
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import helpers as H
from tests.gpu_util import ctx, dev, host

pytestmark = pytest.mark.gpu
BOUND = 2e-3


@pytest.fixture(autouse=True, params=["fused", "operand_pass"])
def gemm_variant(request):
    """Q4_K runs on the kernel that dequantises inside the GEMM and on the separate f16 operand pass + plain GEMM (what
    the other formats use); both must produce the same bits, so every case runs on both."""
    ctx().set_option("disable_fused_gemm", 1 if request.param == "operand_pass" else 0)
    ctx().set_option("force_fused_gemm", 1 if request.param == "fused" else 0)
    yield request.param
    ctx().set_option("disable_fused_gemm", 0)
    ctx().set_option("force_fused_gemm", 0)


def test_fused_and_operand_pass_kernels_agree_bit_for_bit(gemm_variant):
    if gemm_variant == "operand_pass":
        pytest.skip("compares a fused variant with the operand pass in one go")
    rows, cols, m = 300, 1024, 530
    data = H.random_weight(H.Q4_K, rows, cols, seed=77)
    x = dev(np.random.default_rng(78).standard_normal((m, cols)).astype(np.float32), torch.bfloat16)
    w = ctx().prepare_weight(H.Q4_K, data, rows, cols)
    a = host(ctx().linear(x, w, out_dtype=torch.float32)).copy()
    ctx().set_option("force_fused_gemm", 0)
    ctx().set_option("disable_fused_gemm", 1)
    b = host(ctx().linear(x, w, out_dtype=torch.float32))
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


@pytest.mark.parametrize("tensor_type", [H.Q4_K, H.Q4_0, H.Q8_0, H.IQ4_NL])
@pytest.mark.parametrize("m,rows,cols", [(17, 200, 1024), (64, 128, 256), (300, 384, 2048), (512, 130, 512)])
def test_prefill_linear_matches_cpu_matmul(tensor_type, m, rows, cols):
    data = H.random_weight(tensor_type, rows, cols, seed=3 * m + rows)
    x = np.random.default_rng(m).standard_normal((m, cols)).astype(np.float32)
    x16 = dev(x, torch.bfloat16)
    w = ctx().prepare_weight(tensor_type, data, rows, cols)
    got = host(ctx().linear(x16, w, out_dtype=torch.float32))
    want = orc.linear(tensor_type, data, rows, cols, x16.float().cpu().numpy())
    assert H.max_rel_error(got, want) <= BOUND


def test_prefill_reference_generator_case():
    """src/kernel/cuda/linear.rs:2176-2206 shape (M = 9 runs the decode kernel; M = 33 the tensor-core path) with
    the reference's own device gate 0.05 + 0.002*|e| as an outer bound."""
    rows, cols, m = 2, 256, 33
    packed = H.reference_packed_blocks(12, rows)
    idx = np.arange(m * cols, dtype=np.int64)
    x = (((idx * 17 % 101).astype(np.float32) - 50.0) / 64.0).reshape(m, cols)
    w = ctx().prepare_weight(12, packed, rows, cols)
    got = host(ctx().linear(dev(x, torch.float16), w, out_dtype=torch.float32))
    want = orc.linear(12, packed, rows, cols, x)
    assert np.all(np.abs(got - want) <= 0.05 + 0.002 * np.abs(want))
    assert H.max_rel_error(got, want) <= BOUND


@pytest.mark.parametrize("y_dtype", [torch.bfloat16, torch.float16])
def test_prefill_output_dtypes_and_residual(y_dtype):
    rows, cols, m = 256, 768, 100
    data = H.random_weight(H.Q4_K, rows, cols, seed=5)
    x = dev(np.random.default_rng(6).standard_normal((m, cols)).astype(np.float32), torch.bfloat16)
    r = dev(np.random.default_rng(7).standard_normal((m, rows)).astype(np.float32), y_dtype)
    w = ctx().prepare_weight(H.Q4_K, data, rows, cols)
    got = host(ctx().linear_add(x, w, r))
    want = orc.linear(H.Q4_K, data, rows, cols, x.float().cpu().numpy()) + r.float().cpu().numpy()
    tol = BOUND + (2 ** -8 if y_dtype == torch.bfloat16 else 2 ** -11)  # compute bound + rounding of the stored dtype
    assert H.max_rel_error(got, want) <= tol


@pytest.mark.parametrize("tensor_type", [H.Q4_K, H.Q4_0])
def test_prefill_gated_matches_cpu_path(tensor_type):
    """src/kernel/cuda/linear.rs:2317-2355 (gated Q4_K prefill, M = 9 there; 40 here to reach the tensor-core path)."""
    rows, cols, m = 320, 512, 40
    gate, up = H.random_weight(tensor_type, rows, cols, seed=8), H.random_weight(tensor_type, rows, cols, seed=9)
    x = dev(np.random.default_rng(10).standard_normal((m, cols)).astype(np.float32), torch.bfloat16)
    wg, wu = ctx().prepare_weight(tensor_type, gate, rows, cols), ctx().prepare_weight(tensor_type, up, rows, cols)
    got = host(ctx().gated_linear(x, wg, wu, out_dtype=torch.float32))
    want = orc.gated_linear(tensor_type, gate, up, rows, cols, x.float().cpu().numpy())
    assert H.max_rel_error(got, want) <= BOUND


def test_prefill_full_width_slice():
    """One 128-row x 256-token tile of the 5120 -> 17408 prefill shape at full K, checked on a seeded subsample."""
    rows, cols, m = 128, 5120, 256
    data = H.random_weight(H.Q4_K, rows, cols, seed=11)
    x = dev(np.random.default_rng(12).standard_normal((m, cols)).astype(np.float32), torch.bfloat16)
    w = ctx().prepare_weight(H.Q4_K, data, rows, cols)
    got = host(ctx().linear(x, w, out_dtype=torch.float32))
    sel = np.random.default_rng(13).choice(m, size=24, replace=False)
    want = orc.linear(H.Q4_K, data, rows, cols, x.float().cpu().numpy()[sel])
    assert H.max_rel_error(got[sel], want) <= BOUND
