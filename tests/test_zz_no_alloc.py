"""The allocation-free decode entry point, zq_linear_noalloc, against the regular zq_linear.

Some callers cannot allocate device memory where they run a layer (the host application owns the allocator, or
the call sits in a region where allocator calls are forbidden), so this entry keeps its scratch in a fixed
device array inside the library.  It must give the same result as zq_linear, call after call, although every
call reuses (and finds the leftovers of) the same scratch.  The file sorts last so that a failure here cannot
hide any other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from tests import helpers as H
from tests.gpu_util import ctx, dev, host

pytestmark = pytest.mark.gpu


def _noalloc(x, w, m):
    from zllm_b200 import ffi

    y = torch.empty((m, w.rows), dtype=torch.float32, device=x.device)
    ffi.call("zq_linear_noalloc", ctx().handle, w.handle, C.c_void_p(x.data_ptr()), ffi.F32, m, C.c_void_p(y.data_ptr()), ffi.F32)
    return y


@pytest.mark.parametrize("tensor_type,rows,cols,m", [(H.Q4_K, 128, 17408, 1), (H.Q4_K, 3840, 3840, 4), (H.Q8_0, 300, 2560, 8), (H.Q4_0, 200, 1024, 2)])
def test_noalloc_matches_regular_linear_on_consecutive_calls(tensor_type, rows, cols, m):
    """Shapes include a tile split over many CTAs (128 x 17408), which is what exercises the static scratch."""
    # the kernel that keeps split-tile partials in scratch is the per-item staging one; select it so that the
    # static scratch is really exercised (the cluster kernel reduces through shared memory and needs none)
    ctx().set_option("force_staged_gemv", 1)
    data = H.random_weight(tensor_type, rows, cols, seed=rows + m)
    w = ctx().prepare_weight(tensor_type, data, rows, cols)
    x1 = dev(np.random.default_rng(1).standard_normal((m, cols)).astype(np.float32))
    x2 = dev(np.random.default_rng(2).standard_normal((m, cols)).astype(np.float32))
    want1, want2 = host(ctx().linear(x1, w)).copy(), host(ctx().linear(x2, w)).copy()
    got1 = _noalloc(x1, w, m)   # two calls in a row, no synchronisation in between: the second one finds the
    got2 = _noalloc(x2, w, m)   # first one's leftovers in the shared scratch
    got1, got2 = host(got1), host(got2)
    ctx().set_option("force_staged_gemv", 0)
    assert H.max_rel_error(got1, want1) <= 2e-5 and H.max_rel_error(got2, want2) <= 2e-5
    assert np.array_equal(got1.view(np.uint32), want1.view(np.uint32))
    assert np.array_equal(got2.view(np.uint32), want2.view(np.uint32))


@pytest.mark.parametrize("m", [1, 4, 5, 8])
@pytest.mark.parametrize("tensor_type", [H.Q4_K, H.Q8_0, H.IQ4_NL])
def test_noalloc_with_default_options(tensor_type, m):
    """The kernels a caller gets without any option set: equal to zq_linear bit for bit for 1..4 rows, within the
    integer-MMA kernel's activation rounding for 5..8 rows (which zq_linear runs on that kernel and this entry on the
    f16-limb one); against the CPU oracle at the decode path's bound; and the device's free memory does not move."""
    from oracle import oracle as O

    rows, cols = 384, 4096
    data = H.random_weight(tensor_type, rows, cols, seed=11 * m)
    w = ctx().prepare_weight(tensor_type, data, rows, cols)
    x_host = np.random.default_rng(m).standard_normal((m, cols)).astype(np.float32)
    x = dev(x_host)
    want = host(ctx().linear(x, w)).copy()
    _noalloc(x, w, m)  # the first call on a device resolves the scratch address
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    got1 = _noalloc(x, w, m)
    got2 = _noalloc(x, w, m)
    torch.cuda.synchronize()
    # torch.empty for the two outputs is served from torch's cache or not; the library itself must take nothing:
    # the outputs are 2 * m * rows * 4 bytes, far below one allocator segment, so allow exactly torch's segment
    free_after, _ = torch.cuda.mem_get_info()
    assert free_before - free_after <= 2 * (2 << 20)
    got1, got2 = host(got1), host(got2)
    assert np.array_equal(got1.view(np.uint32), got2.view(np.uint32))
    if m <= 4:
        assert np.array_equal(got1.view(np.uint32), want.view(np.uint32))
    else:
        assert H.max_rel_error(got1, want) <= 3e-4
    ref = O.linear(tensor_type, data, rows, cols, x_host)
    assert H.max_rel_error(got1, ref) <= 3e-4  # the decode path's own bound (16-bit activation slices), inside the 2e-3 contract


def test_noalloc_rejects_sizes_beyond_its_limits():
    from zllm_b200 import ffi

    w = ctx().prepare_weight(H.Q4_K, H.random_weight(H.Q4_K, 64, 256, seed=3), 64, 256)
    x = dev(np.zeros((9, 256), dtype=np.float32))
    with pytest.raises(ffi.ZqFailure) as info:
        _noalloc(x, w, 9)
    assert "1..8" in str(info.value)
