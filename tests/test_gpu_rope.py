"""GPU parity of the rotary embedding on q / k projection outputs (zq_rope_qk) against the CPU oracle: f32 rows bit for
bit (the products are rounded separately on both sides), half-precision rows to half an ulp of the storage type."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.gpu_util import ctx

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("suffix", [False, True])
@pytest.mark.parametrize("rows,heads,kv_heads,head_dim,rotary", [(1, 24, 8, 64, 64), (5, 4, 2, 32, 16), (300, 8, 8, 128, 64), (2, 3, 1, 10, 6)])
def test_rope_qk_matches_cpu_path_bit_for_bit(interleaved, suffix, rows, heads, kv_heads, head_dim, rotary):
    rng = np.random.default_rng(rows + heads)
    pos = 7
    q = rng.standard_normal((rows, heads * head_dim)).astype(np.float32)
    k = rng.standard_normal((rows, kv_heads * head_dim)).astype(np.float32)
    cos = rng.standard_normal((pos + rows, rotary // 2)).astype(np.float32)
    sin = rng.standard_normal((pos + rows, rotary // 2)).astype(np.float32)
    dq, dk = torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda()
    ctx().rope_prefix_qk(dq, dk, heads, kv_heads, rotary, pos, torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda(), interleaved=interleaved, suffix=suffix)
    ctx().sync()
    want_q = orc.rope(q, heads, rotary, pos, cos, sin, int(interleaved), int(suffix))
    want_k = orc.rope(k, kv_heads, rotary, pos, cos, sin, int(interleaved), int(suffix))
    assert np.array_equal(dq.cpu().numpy().view(np.uint32), want_q.view(np.uint32))
    assert np.array_equal(dk.cpu().numpy().view(np.uint32), want_k.view(np.uint32))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_rope_on_half_precision_rows(dtype):
    rng = np.random.default_rng(1)
    rows, heads, head_dim, rotary, pos = 4, 8, 64, 64, 0
    q = torch.from_numpy(rng.standard_normal((rows, heads * head_dim)).astype(np.float32)).to(dtype)
    ang = rng.uniform(0, 6.28, size=(rows, rotary // 2)).astype(np.float32)
    cos, sin = np.cos(ang), np.sin(ang)
    dq = q.cuda()
    ctx().rope_prefix_qk(dq, None, heads, 0, rotary, pos, torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda())
    ctx().sync()
    want = torch.from_numpy(orc.rope(q.float().numpy(), heads, rotary, pos, cos, sin)).to(dtype)
    assert torch.equal(dq.cpu(), want)  # computed in f32 from the stored values, rounded once


def test_rope_parameter_errors():
    from zllm_b200 import ffi

    q = torch.zeros((1, 4), device="cuda")
    t = torch.zeros(2, device="cuda")
    with pytest.raises(ffi.ZqFailure):
        ctx().rope_prefix_qk(q, None, 1, 0, 4, 1, t, t, suffix=True)  # the table is one row short (src/attention/rope.rs:179-182)
    with pytest.raises(ffi.ZqFailure):
        ctx().rope_prefix_qk(q, None, 1, 0, 3, 0, t, t)  # odd rotary dimension
    with pytest.raises(ffi.ZqFailure):
        ctx().rope_prefix_qk(q, None, 1, 0, 6, 0, torch.zeros(3, device="cuda"), torch.zeros(3, device="cuda"))  # rotary > head_dim
