"""Q5_K and Q6_K linear layers (src/weight/codec/ggml.rs:425-469; the reference's CUDA kernels for them:
src/kernel/cuda/linear.rs:1167-1234, 1967-2101) against the CPU oracle, through the C ABI.

Decode (up to 16 rows, plain and gated) runs the integer-MMA kernels: Q5_K with Q4_K's unpacker plus the high bit, Q6_K
on a re-laid 224-byte unit with one MMA per 16-weight scale group (16-bit integer activations: held to 3e-4 here).  More
rows, and every row count with the f16 switch set, run the f16 operand pass and the tensor-core GEMM (2e-3).
"""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import helpers as H
from tests.gpu_util import ctx, dev, host

pytestmark = pytest.mark.gpu
BOUND = 2e-3
TYPES = [H.Q5_K, H.Q6_K]


@pytest.mark.parametrize("tensor_type", TYPES)
@pytest.mark.parametrize("m,rows,cols", [(1, 200, 1024), (4, 128, 256), (7, 1031, 768), (8, 5, 5120), (16, 384, 2048), (40, 130, 512), (300, 256, 1536)])
@pytest.mark.parametrize("x_dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_linear_matches_cpu_path(tensor_type, m, rows, cols, x_dtype):
    if m > 8 and x_dtype != torch.bfloat16:
        pytest.skip("the tensor-core path is checked on activations that are exact in f16")
    data = H.random_weight(tensor_type, rows, cols, seed=5 * m + rows)
    x = dev(np.random.default_rng(m).standard_normal((m, cols)).astype(np.float32), x_dtype)
    w = ctx().prepare_weight(tensor_type, data, rows, cols)
    got = host(ctx().linear(x, w, out_dtype=torch.float32))
    want = orc.linear(tensor_type, data, rows, cols, x.float().cpu().numpy())
    tight = 3e-4 if m <= 16 else BOUND
    assert H.max_rel_error(got, want) <= tight


@pytest.mark.parametrize("tensor_type", TYPES)
@pytest.mark.parametrize("m", [1, 3, 8, 13])
def test_decode_kernels_agree_with_the_cpu_path(tensor_type, m):
    """Every decode route: the integer-MMA kernel of zq_linear, the work-list kernel (zq_linear_batch: plain, residual
    and gated jobs in one call), and, with the f16 switch set, the operand pass + GEMM."""
    Q5_K = tensor_type  # shorthand in this body: either of the two types
    rows, cols = 640, 2048
    gate, up, down = H.random_weight(Q5_K, rows, cols, seed=31), H.random_weight(Q5_K, rows, cols, seed=32), H.random_weight(Q5_K, 384, cols, seed=33)
    x_np = np.random.default_rng(34 + m).standard_normal((m, cols)).astype(np.float32)
    r_np = np.random.default_rng(35).standard_normal((m, 384)).astype(np.float32)
    x, r = dev(x_np), dev(r_np)
    wg, wu, wd = (ctx().prepare_weight(Q5_K, d, n, cols) for d, n in ((gate, rows), (up, rows), (down, 384)))
    want_plain = orc.linear(Q5_K, gate, rows, cols, x_np)
    want_res = orc.linear(Q5_K, down, 384, cols, x_np) + r_np
    want_gated = orc.gated_linear(Q5_K, gate, up, rows, cols, x_np)
    assert H.max_rel_error(host(ctx().linear(x, wg)), want_plain) <= 3e-4
    assert H.max_rel_error(host(ctx().gated_linear(x, wg, wu)), want_gated) <= 6e-4
    outs = ctx().linear_batch([(x, wg), (x, wd, r), (x, wg, wu, "gated")])
    assert H.max_rel_error(host(outs[0]), want_plain) <= 3e-4
    assert H.max_rel_error(host(outs[1]), want_res) <= 3e-4
    assert H.max_rel_error(host(outs[2]), want_gated) <= 6e-4
    ctx().set_option("force_f16_gemv", 1)
    try:
        assert H.max_rel_error(host(ctx().linear(x, wg)), want_plain) <= BOUND
    finally:
        ctx().set_option("force_f16_gemv", 0)


@pytest.mark.parametrize("tensor_type", TYPES)
def test_reference_generator_case(tensor_type):
    """The reference's deterministic blocks and inputs (src/kernel/cpu/ggml_quant.rs:370-414, 432), one row of
    activations, with the reference's device gate 0.05 + 0.002*|e| as an outer bound."""
    rows, cols = 3, 256
    packed = H.reference_packed_blocks(tensor_type, rows)
    idx = np.arange(cols, dtype=np.int64)
    x = (((idx * 17 % 101).astype(np.float32) - 50.0) / 64.0).reshape(1, cols)
    w = ctx().prepare_weight(tensor_type, packed, rows, cols)
    got = host(ctx().linear(dev(x, torch.float16), w, out_dtype=torch.float32))
    want = orc.linear(tensor_type, packed, rows, cols, x)
    assert np.all(np.abs(got - want) <= 0.05 + 0.002 * np.abs(want))
    assert H.max_rel_error(got, want) <= BOUND


@pytest.mark.parametrize("tensor_type", TYPES)
@pytest.mark.parametrize("m", [2, 48])
def test_linear_add_and_gated(tensor_type, m):
    rows, cols = 256, 512
    gate, up = H.random_weight(tensor_type, rows, cols, seed=21), H.random_weight(tensor_type, rows, cols, seed=22)
    x = dev(np.random.default_rng(23).standard_normal((m, cols)).astype(np.float32), torch.bfloat16)
    r = dev(np.random.default_rng(24).standard_normal((m, rows)).astype(np.float32), torch.float32)
    wg, wu = ctx().prepare_weight(tensor_type, gate, rows, cols), ctx().prepare_weight(tensor_type, up, rows, cols)
    xf = x.float().cpu().numpy()
    got = host(ctx().linear_add(x, wg, r))
    want = orc.linear(tensor_type, gate, rows, cols, xf) + r.cpu().numpy()
    assert H.max_rel_error(got, want) <= BOUND
    got = host(ctx().gated_linear(x, wg, wu, out_dtype=torch.float32))
    want = orc.gated_linear(tensor_type, gate, up, rows, cols, xf)
    assert H.max_rel_error(got, want) <= 2 * BOUND  # two f16-operand products multiplied: each factor is within BOUND


def test_no_decode_entry_and_no_encoder_for_these_types():
    from zllm_b200 import ffi

    data = H.random_weight(H.Q6_K, 128, 256, seed=1)
    w = ctx().prepare_weight(H.Q6_K, data, 128, 256)
    x = dev(np.ones((1, 256), dtype=np.float32), torch.float32)
    y = torch.empty((1, 128), dtype=torch.float32, device=x.device)
    with pytest.raises(ffi.ZqFailure):
        ffi.call("zq_linear_noalloc", ctx().handle, w.handle, C.c_void_p(x.data_ptr()), ffi.F32, 1, C.c_void_p(y.data_ptr()), ffi.F32)
    with pytest.raises(ffi.ZqFailure):
        ctx().quantize(H.Q5_K, dev(np.zeros((1, 256), dtype=np.float32), torch.float32))


@pytest.mark.parametrize("down_type", TYPES)
@pytest.mark.parametrize("m", [3, 48, 400])
def test_moe_experts_with_k_quant_down_projection(down_type, m):
    """Q4_K gate/up with a Q5_K or Q6_K down projection, the mix the reference's CUDA experts accept
    (src/backend/cuda/expert.rs:462-473), against the oracle's moe_forward.  The down projection runs on f16
    operands behind the f16-rounded activated intermediate, hence the composite bound of the MoE prefill test."""
    from zllm_b200.backend import MoeExperts, moe_forward

    n_exp, top_k, hidden, inter = 8, 2, 512, 256
    rng = np.random.default_rng(40 + m)
    gates = [H.random_weight(H.Q4_K, inter, hidden, seed=300 + 3 * e) for e in range(n_exp)]
    ups = [H.random_weight(H.Q4_K, inter, hidden, seed=301 + 3 * e) for e in range(n_exp)]
    downs = [H.random_weight(down_type, hidden, inter, seed=302 + 3 * e) for e in range(n_exp)]
    x = rng.standard_normal((m, hidden)).astype(np.float32)
    ids_np = np.stack([rng.permutation(n_exp)[:top_k] for _ in range(m)]).astype(np.uint32)
    w_np = rng.random((m, top_k)).astype(np.float32)
    w_np /= w_np.sum(axis=1, keepdims=True)
    c = ctx()
    table = MoeExperts(c, [c.prepare_weight(H.Q4_K, g, inter, hidden) for g in gates], [c.prepare_weight(H.Q4_K, u, inter, hidden) for u in ups],
                       [c.prepare_weight(down_type, d, hidden, inter) for d in downs])
    got = host(moe_forward(c, table, dev(x), torch.from_numpy(ids_np.astype(np.int32)).cuda(), dev(w_np)))
    want = orc.moe_forward([(H.Q4_K, g, inter, hidden) for g in gates], [(H.Q4_K, u, inter, hidden) for u in ups], [(down_type, d, hidden, inter) for d in downs], x, ids_np, w_np)
    # two chained f16-operand GEMMs; the uniformly random codes of the generator give the down weights a large common
    # offset, so single outputs out of ~2e5 reach 4.1e-3 while the relative L2 error stays under 1e-3
    assert H.max_rel_error(got, want) <= 2.5 * BOUND
    assert float(np.linalg.norm(got - want) / np.linalg.norm(want)) <= 1e-3
