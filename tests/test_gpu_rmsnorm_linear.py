"""RMSNorm followed by quantized projections (Backend::rmsnorm_linear / rmsnorm_dual_linear, src/backend/mod.rs:455-464;
norm formula src/kernel/cpu/rmsnorm.rs:7-41) against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import helpers as H
from tests.gpu_util import ctx, dev, host

pytestmark = pytest.mark.gpu


def _rmsnorm(x, w, eps, offset):
    """f32 restatement of rmsnorm_with_weight_offset: x * (1 / sqrt(mean(x^2) + eps)) * (w + offset)."""
    x = x.astype(np.float32)
    mean_sq = (np.sum(x.astype(np.float64) ** 2, axis=1) / x.shape[1]).astype(np.float32)
    inv = (np.float32(1.0) / np.sqrt(mean_sq + np.float32(eps))).astype(np.float32)
    weight = w if offset == 0.0 else (np.float32(offset) + w).astype(np.float32)
    return ((x * inv[:, None]).astype(np.float32) * weight[None, :]).astype(np.float32)


@pytest.mark.parametrize("tensor_type", [H.Q4_K, H.Q8_0, H.Q6_K])
@pytest.mark.parametrize("m", [1, 5, 40])
@pytest.mark.parametrize("offset", [0.0, 1.0])
def test_rmsnorm_linear_matches_cpu_path(tensor_type, m, offset):
    rows, cols, eps = 384, 1536, 1e-6
    rng = np.random.default_rng(17 * m + tensor_type)
    data = H.random_weight(tensor_type, rows, cols, seed=tensor_type + m)
    x = (rng.standard_normal((m, cols)) * 3.0).astype(np.float32)
    nw = (1.0 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
    w = ctx().prepare_weight(tensor_type, data, rows, cols)
    got = host(ctx().rmsnorm_linear(dev(x), dev(nw), eps, w, out_dtype=torch.float32, weight_offset=offset))
    want = orc.linear(tensor_type, data, rows, cols, _rmsnorm(x, nw, eps, offset))
    # decode kernels see f32 normalised rows; the tensor-core path rounds them to f16 (activations that are not exact
    # in f16 add 2^-12 per element to the weight rounding)
    assert H.max_rel_error(got, want) <= (3e-4 if m <= 16 else 2e-3)


def test_rmsnorm_dual_linear_shares_one_normalisation():
    rows, cols, m, eps = 256, 512, 3, 1e-5
    rng = np.random.default_rng(5)
    a, b = H.random_weight(H.Q4_K, rows, cols, seed=61), H.random_weight(H.Q4_0, 128, cols, seed=62)
    x = rng.standard_normal((m, cols)).astype(np.float32)
    nw = rng.standard_normal(cols).astype(np.float32)
    wa, wb = ctx().prepare_weight(H.Q4_K, a, rows, cols), ctx().prepare_weight(H.Q4_0, b, 128, cols)
    ya, yb = ctx().rmsnorm_dual_linear(dev(x, torch.bfloat16), dev(nw), eps, wa, wb, out_dtype=torch.float32)
    xn = _rmsnorm(dev(x, torch.bfloat16).float().cpu().numpy(), nw, eps, 0.0)
    assert H.max_rel_error(host(ya), orc.linear(H.Q4_K, a, rows, cols, xn)) <= 3e-4
    assert H.max_rel_error(host(yb), orc.linear(H.Q4_0, b, 128, cols, xn)) <= 3e-4


def test_rmsnorm_linear_rejects_bad_arguments():
    from zllm_b200 import ffi

    data = H.random_weight(H.Q4_K, 128, 256, seed=1)
    w = ctx().prepare_weight(H.Q4_K, data, 128, 256)
    x = dev(np.ones((2, 256), dtype=np.float32))
    with pytest.raises(ffi.ZqFailure):
        ctx().rmsnorm_linear(x, dev(np.ones(255, dtype=np.float32)), 1e-6, w)
    with pytest.raises(ffi.ZqFailure):
        ctx().rmsnorm_linear(x, dev(np.ones(256, dtype=np.float32)), -1.0, w)
