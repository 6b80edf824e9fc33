"""GPU parity of the work-list decode kernel (``zq_linear_batch`` and the entries built on it) against the CPU
oracle, through the C ABI.

Tolerance: the contract is max_i |a_i - e_i| / max(|e_i|, rms(e)) <= 2e-3 (fp32 accumulation); the integer-MMA
arithmetic (activations as 16-bit integers per 256-column slice, exact integer weights) is held to 3e-4 on top.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import helpers as H
from tests.gpu_util import ctx, dev, host

pytestmark = pytest.mark.gpu

BOUND = 2e-3
TIGHT = 3e-4


def _check(got, want, tight=TIGHT):
    err = H.max_rel_error(got, want)
    assert err <= BOUND, f"max relative error {err} above the 2e-3 contract"
    assert err <= tight, f"max relative error {err} above the kernel's own {tight}"


def _weight(tensor_type, rows, cols, seed):
    data = H.random_weight(tensor_type, rows, cols, seed=seed)
    return data, ctx().prepare_weight(tensor_type, data, rows, cols)


def test_batch_of_mixed_jobs_matches_cpu_path():
    """Three weight types, every row-count class (1-4, 5-8, 9-16), ragged row counts, odd unit counts, a residual."""
    rng = np.random.default_rng(7)
    specs = [  # (type, rows, cols, m, with residual)
        (H.Q4_K, 200, 1024, 1, False), (H.Q4_K, 130, 768, 4, True), (H.Q4_K, 64, 2560, 3, False), (H.Q4_K, 384, 512, 8, False),
        (H.Q4_K, 257, 1280, 16, True), (H.Q4_0, 7, 96, 1, False), (H.Q4_0, 300, 1056, 2, True), (H.Q4_0, 128, 544, 12, False),
        (H.Q8_0, 64, 1056, 1, False), (H.Q8_0, 2, 32, 4, False), (H.Q8_0, 300, 2560, 6, True), (H.Q4_K, 1000, 256, 1, False),
    ]
    jobs, wants, keep = [], [], []
    for i, (tt, rows, cols, m, res) in enumerate(specs):
        data, w = _weight(tt, rows, cols, 100 + i)
        x = rng.standard_normal((m, cols)).astype(np.float32)
        want = orc.linear(tt, data, rows, cols, x)
        r = None
        if res:
            r = rng.standard_normal((m, rows)).astype(np.float32)
            want = want + r
        jobs.append((dev(x), w, dev(r)) if res else (dev(x), w))
        wants.append(want)
        keep.append(w)
    ys = ctx().linear_batch(jobs)
    for y, want in zip(ys, wants):
        _check(host(y), want)


@pytest.mark.parametrize("tensor_type", [H.Q4_K, H.Q4_0, H.Q8_0, H.IQ4_NL, H.Q5_K, H.Q6_K])
def test_one_tile_cut_across_many_ctas(tensor_type):
    """128 x 17408: one row tile, 34 chunks -> every CTA holds one chunk of the same tile and the last one adds 34 partials."""
    rows, cols = 128, 17408
    data, w = _weight(tensor_type, rows, cols, 5)
    for m in (1, 4, 16):
        x = np.random.default_rng(m).standard_normal((m, cols)).astype(np.float32)
        (y,) = ctx().linear_batch([(dev(x), w)])
        _check(host(y), orc.linear(tensor_type, data, rows, cols, x))


@pytest.mark.parametrize("rows,cols", [(17408, 5120), (5120, 17408)])
def test_full_size_decode_shapes(rows, cols):
    """The two largest matrices of the decode sweep at full size, Q4_K, one and four rows in one batch."""
    data, w = _weight(H.Q4_K, rows, cols, rows)
    x1 = np.random.default_rng(1).standard_normal((1, cols)).astype(np.float32)
    x4 = np.random.default_rng(4).standard_normal((4, cols)).astype(np.float32)
    y1, y4 = ctx().linear_batch([(dev(x1), w), (dev(x4), w)])
    _check(host(y1), orc.linear(H.Q4_K, data, rows, cols, x1))
    _check(host(y4), orc.linear(H.Q4_K, data, rows, cols, x4))
    # the single-call entry on the same weight
    _check(host(ctx().linear(dev(x1), w)), orc.linear(H.Q4_K, data, rows, cols, x1))


@pytest.mark.parametrize("tensor_type", [H.Q4_K, H.Q4_0, H.Q8_0, H.IQ4_NL, H.Q5_K, H.Q6_K])
@pytest.mark.parametrize("m,rows,cols", [(1, 3840, 1536), (1, 100, 512), (4, 192, 1024), (8, 64, 768), (12, 200, 1024)])
def test_gated_jobs_match_cpu_path(tensor_type, m, rows, cols):
    gate, wg = _weight(tensor_type, rows, cols, 21)
    up, wu = _weight(tensor_type, rows, cols, 22)
    x = np.random.default_rng(23).standard_normal((m, cols)).astype(np.float32)
    # a gated job and a plain job in one call
    yg, yp = ctx().linear_batch([(dev(x), wg, wu, "gated"), (dev(x), wu)])
    _check(host(yg), orc.gated_linear(tensor_type, gate, up, rows, cols, x), tight=1e-3)  # silu(g) * u: where u is large and silu(g) small the error of g is weighed by u against the rms of the outputs
    _check(host(yp), orc.linear(tensor_type, up, rows, cols, x))


def test_shared_input_is_quantised_once_and_results_match():
    """dual / triple linear (q, k, v of MiniCPM5: 1536 -> 1536, 512, 512) through the multi-weight entry."""
    cols = 1536
    datas, ws = zip(*[_weight(H.Q4_K, rows, cols, 40 + i) for i, rows in enumerate((1536, 512, 512))])
    x = np.random.default_rng(3).standard_normal((1, cols)).astype(np.float32)
    n0 = ctx().launch_count
    q, k, v = ctx().triple_linear(dev(x), *ws)
    assert ctx().launch_count - n0 == 2, "three projections of one input: one record pass and one decode launch"
    for y, data, rows in zip((q, k, v), datas, (1536, 512, 512)):
        _check(host(y), orc.linear(H.Q4_K, data, rows, cols, x))


def test_results_are_identical_from_run_to_run_and_close_to_single_launches():
    rng = np.random.default_rng(11)
    jobs, keep = [], []
    for i, (rows, cols, m) in enumerate([(3840, 3840, 1), (640, 15360, 4), (2048, 1024, 2)]):
        data, w = _weight(H.Q4_K, rows, cols, 60 + i)
        jobs.append((dev(rng.standard_normal((m, cols)).astype(np.float32)), w))
        keep.append(w)
    a = [host(y).copy() for y in ctx().linear_batch(jobs)]
    b = [host(y).copy() for y in ctx().linear_batch(jobs)]
    for u, v in zip(a, b):
        assert np.array_equal(u.view(np.uint32), v.view(np.uint32))
    ctx().set_option("disable_worklist", 1)
    try:
        c = [host(y).copy() for y in ctx().linear_batch(jobs)]
    finally:
        ctx().set_option("disable_worklist", 0)
    for u, v in zip(a, c):
        assert H.max_rel_error(u, v) <= 1e-5  # same integer arithmetic, different order of the f32 partial sums


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_half_precision_inputs_and_outputs(dtype):
    rows, cols, m = 300, 1024, 3
    data, w = _weight(H.Q4_K, rows, cols, 70)
    x = torch.from_numpy(np.random.default_rng(1).standard_normal((m, cols)).astype(np.float32)).to(dtype)
    (y,) = ctx().linear_batch([(x.cuda(), w)])
    want = orc.linear(H.Q4_K, data, rows, cols, x.float().numpy())
    want = torch.from_numpy(want).to(dtype).float().numpy()  # the output is rounded once to the output dtype
    err = H.max_rel_error(host(y), want)
    assert err <= (1e-3 if dtype == torch.float16 else 8e-3)  # half an ulp of the output type on top of the kernel's error


def test_activation_outlier_inside_a_slice():
    """One activation 1000x the rms of its 256-column slice: the slice is scaled by its maximum, so the small entries keep
    2^-16 of that maximum; the result must stay inside the 2e-3 contract."""
    rows, cols = 512, 2048
    data, w = _weight(H.Q4_K, rows, cols, 80)
    x = np.random.default_rng(2).standard_normal((2, cols)).astype(np.float32)
    x[0, 300] = 1000.0
    x[1, 1500] = -1000.0
    (y,) = ctx().linear_batch([(dev(x), w)])
    err = H.max_rel_error(host(y), orc.linear(H.Q4_K, data, rows, cols, x))
    assert err <= BOUND
    got = host(ctx().linear(dev(x), w))
    assert H.max_rel_error(got, orc.linear(H.Q4_K, data, rows, cols, x)) <= BOUND


def test_unsupported_jobs_fall_back_to_their_own_launches():
    """IQ4_NL and a 40-row job ride in the same call and run as their own launches."""
    rows, cols = 192, 1024
    d1, w1 = _weight(H.IQ4_NL, rows, cols, 90)
    d2, w2 = _weight(H.Q4_K, rows, cols, 91)
    x1 = np.random.default_rng(5).standard_normal((2, cols)).astype(np.float32)
    x2 = np.random.default_rng(6).standard_normal((40, cols)).astype(np.float32)
    y1, y2, y3 = ctx().linear_batch([(dev(x1), w1), (dev(x2), w2), (dev(x1), w2)])
    _check(host(y1), orc.linear(H.IQ4_NL, d1, rows, cols, x1))
    assert H.max_rel_error(host(y2), orc.linear(H.Q4_K, d2, rows, cols, x2)) <= BOUND
    _check(host(y3), orc.linear(H.Q4_K, d2, rows, cols, x1))


def test_argument_errors():
    from zllm_b200 import ffi

    rows, cols = 64, 512
    _, w = _weight(H.Q4_K, rows, cols, 95)
    _, w2 = _weight(H.Q4_K, rows, 256, 96)
    x = dev(np.zeros((1, cols), dtype=np.float32))
    with pytest.raises(ffi.ZqFailure):
        ctx().linear_batch([(x, w, w2, "gated")])  # gate and up differ in shape
