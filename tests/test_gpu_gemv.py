"""GPU parity of the decode GEMV family against the CPU oracle, through the C ABI.

Tolerance: the contract is max_i |a_i - e_i| / max(|e_i|, rms(e)) <= 2e-3 (fp32 accumulation).  The f16 decode
kernels keep activations at ~22 bits and integer-exact weights, so the tests also hold them to 2e-5; the integer-MMA
kernel carries activations as 16-bit integers per 256-column slice and is held to 3e-4.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import helpers as H
from tests.gpu_util import ctx, dev, host

pytestmark = pytest.mark.gpu


_VARIANT = {"name": "i8"}


@pytest.fixture(autouse=True, params=["i8", "i8_narrow", "tcgen05", "resident", "staged"])
def gemv_variant(request):
    """Every case runs on all decode kernels: the integer-MMA kernel (the default; 16-bit integer activations;
    "i8_narrow" runs up to 4 rows of a plain projection as 64-row tiles, two CTAs per SM), the
    tcgen05 kernel (Q4_K, opt-in), the f16 warp-MMA kernel with activations resident in shared memory, and the f16
    warp-MMA kernel with per-item activation staging."""
    ctx().set_option("enable_tcgen05_gemv", 1 if request.param == "tcgen05" else 0)
    ctx().set_option("force_staged_gemv", 1 if request.param == "staged" else 0)
    ctx().set_option("force_f16_gemv", 1 if request.param in ("resident", "tcgen05") else 0)
    ctx().set_option("narrow_gemv_tiles", 1 if request.param == "i8_narrow" else 0)
    _VARIANT["name"] = "i8" if request.param == "i8_narrow" else request.param
    yield request.param
    ctx().set_option("force_staged_gemv", 0)
    ctx().set_option("enable_tcgen05_gemv", 0)
    ctx().set_option("force_f16_gemv", 0)
    ctx().set_option("narrow_gemv_tiles", 0)
    _VARIANT["name"] = "i8"


TYPES = [H.Q4_0, H.Q8_0, H.Q4_K, H.IQ4_NL]
BOUND = 2e-3
TIGHT = 2e-5


def _check(got, want, tight=TIGHT):
    if _VARIANT["name"] == "i8":
        tight = max(tight, 3e-4)  # activations as 16-bit integers per 256-column slice: 2^-16 of the slice maximum
    err = H.max_rel_error(got, want)
    assert err <= BOUND, f"max relative error {err} above the 2e-3 contract"
    assert err <= tight, f"max relative error {err} above the decode path's own {tight}"


@pytest.mark.parametrize("tensor_type", TYPES)
@pytest.mark.parametrize("m", [1, 2, 4, 5, 8, 16])
def test_linear_matches_cpu_path(tensor_type, m):
    rows, cols = 200, 1024
    data = H.random_weight(tensor_type, rows, cols, seed=11 + m)
    x = np.random.default_rng(m).standard_normal((m, cols)).astype(np.float32)
    w = ctx().prepare_weight(tensor_type, data, rows, cols)
    got = host(ctx().linear(dev(x), w))
    # 9..16 rows run as single f16 limbs (activation rounding 2^-12), up to 8 rows keep f32-level accuracy
    _check(got, orc.linear(tensor_type, data, rows, cols, x), tight=TIGHT if m <= 8 else 1e-3)


@pytest.mark.parametrize("tensor_type,rows,cols", [
    (H.Q4_K, 3840, 3840), (H.Q4_0, 3840, 3840), (H.Q4_K, 128, 17408), (H.Q4_K, 1536, 1536), (H.Q4_K, 512, 1536),
    (H.Q8_0, 64, 1056), (H.Q8_0, 2, 32), (H.IQ4_NL, 130, 512), (H.Q4_0, 7, 96), (H.Q8_0, 300, 2560),
])
def test_linear_shapes_including_split_tiles_and_ragged_edges(tensor_type, rows, cols):
    """Full-size decode shapes, a tile split across many CTAs (128 x 17408), MiniCPM5 projections, rows and
    columns that are not multiples of the tile (reference shapes: src/kernel/cuda/linear.rs:2209-2230,
    src/kernel/metal/gguf/dispatch/tests.rs:864-895)."""
    data = H.random_weight(tensor_type, rows, cols, seed=rows + cols)
    x = np.random.default_rng(rows).standard_normal((1, cols)).astype(np.float32)
    w = ctx().prepare_weight(tensor_type, data, rows, cols)
    got = host(ctx().linear(dev(x), w))
    _check(got, orc.linear(tensor_type, data, rows, cols, x))


def test_reference_q8_0_known_answers():
    """src/kernel/cpu/ggml_quant.rs:416-426, 446-457: [32, 64] and [32, 64, 16, 32], layout out[token*rows+row]."""
    data = np.zeros(68, dtype=np.uint8)
    data[:2] = [0x00, 0x3C]
    data[2:34] = 1
    data[34:36] = [0x00, 0x40]
    data[36:68] = 1
    w = ctx().prepare_weight(H.Q8_0, data, 2, 32)
    assert list(host(ctx().linear(dev(np.ones((1, 32), dtype=np.float32)), w)).reshape(-1)) == [32.0, 64.0]
    x = np.concatenate([np.full(32, 1.0, dtype=np.float32), np.full(32, 0.5, dtype=np.float32)]).reshape(2, 32)
    assert list(host(ctx().linear(dev(x), w)).reshape(-1)) == [32.0, 64.0, 16.0, 32.0]


@pytest.mark.parametrize("tensor_type", [8, 12])
@pytest.mark.parametrize("m", [1, 9])
def test_reference_generator_cases(tensor_type, m):
    """src/kernel/cpu/ggml_quant.rs:428-479 inputs: packed_blocks and the (i*17 % 101 - 50)/64 ramp; the
    reference's own gate is 1e-3 + 1e-5*|e| against a scalar decode."""
    cols, rows = 256, 2
    idx = np.arange(m * cols, dtype=np.int64)
    x = (((idx * 17 % 101).astype(np.float32) - 50.0) / 64.0).reshape(m, cols)
    packed = H.reference_packed_blocks(tensor_type, rows)
    w = ctx().prepare_weight(tensor_type, packed, rows, cols)
    got = host(ctx().linear(dev(x), w))
    decoded = orc.dequantize(tensor_type, packed, rows * cols).reshape(rows, cols)
    want = x.astype(np.float64) @ decoded.astype(np.float64).T
    assert np.all(np.abs(got - want) <= 1.0e-3 + np.abs(want) * 1.0e-5)


@pytest.mark.parametrize("tensor_type", [H.Q4_K, H.Q4_0, H.IQ4_NL, H.Q8_0])
@pytest.mark.parametrize("m,rows,cols", [(1, 3840, 1536), (1, 100, 512), (4, 192, 1024), (8, 64, 768), (12, 200, 1024)])
def test_gated_silu_matches_cpu_path(tensor_type, m, rows, cols):
    if tensor_type == H.Q4_K and cols % 256:
        pytest.skip("Q4_K needs 256-aligned columns")
    gate = H.random_weight(tensor_type, rows, cols, seed=21)
    up = H.random_weight(tensor_type, rows, cols, seed=22)
    x = np.random.default_rng(23).standard_normal((m, cols)).astype(np.float32)
    wg, wu = ctx().prepare_weight(tensor_type, gate, rows, cols), ctx().prepare_weight(tensor_type, up, rows, cols)
    got = host(ctx().gated_linear(dev(x), wg, wu))
    _check(got, orc.gated_linear(tensor_type, gate, up, rows, cols, x), tight=5e-5 if m <= 8 else BOUND)


def test_gated_is_silu_gate_times_up_of_the_plain_projections():
    """src/kernel/cpu/ggml_quant.rs:481-516 restated on the device: gated == silu(gate)*up of two linears."""
    rows, cols = 2, 512
    idx = np.arange(cols, dtype=np.int64)
    x = (((idx * 13 % 89).astype(np.float32) - 44.0) / 96.0).reshape(1, cols)
    packed = H.reference_packed_blocks(12, rows * cols // 256)
    w = ctx().prepare_weight(12, packed, rows, cols)
    g = host(ctx().linear(dev(x), w)).astype(np.float32)
    got = host(ctx().gated_linear(dev(x), w, w))
    want = (g / (np.float32(1) + np.exp(-g))) * g
    np.testing.assert_allclose(got, want, rtol=2e-5, atol=1e-6)  # the plain projection may run on a different kernel than the gated one


@pytest.mark.parametrize("m", [1, 4])
def test_linear_add_matches_matvec_residual(m):
    """src/kernel/cpu/ggml_quant.rs:521-543"""
    rows, cols = 260, 512
    data = H.random_weight(H.Q4_K, rows, cols, seed=31)
    x = np.random.default_rng(32).standard_normal((m, cols)).astype(np.float32)
    r = np.random.default_rng(33).standard_normal((m, rows)).astype(np.float32)
    w = ctx().prepare_weight(H.Q4_K, data, rows, cols)
    got = host(ctx().linear_add(dev(x), w, dev(r)))
    want = orc.linear(H.Q4_K, data, rows, cols, x) + r
    _check(got, want)


def test_gated_mlp_add_residual_matches_cpu_path():
    """Backend::gated_mlp_add_residual (src/backend/mod.rs:483) at the MiniCPM5 FFN shape 1536 -> 3840 -> 1536."""
    hidden, inter = 1536, 3840
    gate, up = H.random_weight(H.Q4_K, inter, hidden, seed=41), H.random_weight(H.Q4_K, inter, hidden, seed=42)
    down = H.random_weight(H.Q4_K, hidden, inter, seed=43)
    x = np.random.default_rng(44).standard_normal((1, hidden)).astype(np.float32)
    r = np.random.default_rng(45).standard_normal((1, hidden)).astype(np.float32)
    c = ctx()
    wg, wu, wd = c.prepare_weight(H.Q4_K, gate, inter, hidden), c.prepare_weight(H.Q4_K, up, inter, hidden), c.prepare_weight(H.Q4_K, down, hidden, inter)
    got = host(c.gated_mlp_add_residual(dev(x), wg, wu, wd, dev(r)))
    act = orc.gated_linear(H.Q4_K, gate, up, inter, hidden, x)
    want = orc.linear(H.Q4_K, down, hidden, inter, act) + r
    _check(got, want, tight=5e-5)


def test_dual_and_triple_linear_share_the_input():
    cols = 1536
    shapes = [1536, 512, 512]
    datas = [H.random_weight(H.Q4_K, n, cols, seed=50 + i) for i, n in enumerate(shapes)]
    x = np.random.default_rng(53).standard_normal((1, cols)).astype(np.float32)
    ws = [ctx().prepare_weight(H.Q4_K, d, n, cols) for d, n in zip(datas, shapes)]
    outs = ctx().triple_linear(dev(x), *ws)
    for o, d, n in zip(outs, datas, shapes):
        _check(host(o), orc.linear(H.Q4_K, d, n, cols, x))


@pytest.mark.parametrize("x_dtype,y_dtype", [(torch.float16, torch.float16), (torch.bfloat16, torch.bfloat16), (torch.float16, torch.float32)])
def test_half_precision_activations(x_dtype, y_dtype):
    """The reference CUDA path takes f16 activations (src/kernel/cuda/linear.rs:1440); the oracle consumes the same
    rounded inputs, so only the output rounding is added to the bound."""
    rows, cols, m = 256, 1024, 3
    data = H.random_weight(H.Q4_K, rows, cols, seed=61)
    x = dev(np.random.default_rng(62).standard_normal((m, cols)).astype(np.float32), x_dtype)
    w = ctx().prepare_weight(H.Q4_K, data, rows, cols)
    got = host(ctx().linear(x, w, out_dtype=y_dtype))
    want = orc.linear(H.Q4_K, data, rows, cols, x.float().cpu().numpy())
    err = H.max_rel_error(got, want)
    tight = 3e-4 if _VARIANT["name"] == "i8" else TIGHT
    assert err <= (tight if y_dtype == torch.float32 else (5e-4 if y_dtype == torch.float16 else 4e-3))


def test_results_are_deterministic_across_launches():
    rows, cols = 128, 17408  # one tile split over many CTAs: the fix-up order must not depend on timing
    data = H.random_weight(H.Q4_K, rows, cols, seed=71)
    x = dev(np.random.default_rng(72).standard_normal((4, cols)).astype(np.float32))
    w = ctx().prepare_weight(H.Q4_K, data, rows, cols)
    first = host(ctx().linear(x, w)).copy()
    for _ in range(5):
        assert np.array_equal(host(ctx().linear(x, w)).view(np.uint32), first.view(np.uint32))


def test_shape_mismatch_is_an_error():
    from zllm_b200 import ffi

    w = ctx().prepare_weight(H.Q4_K, H.random_weight(H.Q4_K, 8, 256, seed=81), 8, 256)
    with pytest.raises(ffi.ZqFailure):
        ctx().linear(dev(np.zeros((1, 512), dtype=np.float32)), w)
    w2 = ctx().prepare_weight(H.Q4_K, H.random_weight(H.Q4_K, 16, 256, seed=82), 16, 256)
    with pytest.raises(ffi.ZqFailure):
        ctx().gated_linear(dev(np.zeros((1, 256), dtype=np.float32)), w, w2)
    with pytest.raises(ffi.ZqFailure):
        ctx().linear_add(dev(np.zeros((1, 256), dtype=np.float32)), w, dev(np.zeros((1, 9), dtype=np.float32)))


def test_linear_host_copies_in_and_out():
    rows, cols = 300, 768
    data = H.random_weight(H.Q8_0, rows, cols, seed=91)
    x = np.random.default_rng(92).standard_normal((2, cols)).astype(np.float32)
    w = ctx().prepare_weight(H.Q8_0, data, rows, cols)
    y = np.zeros((2, rows), dtype=np.float32)
    ctx().linear_host(x, w, y)
    _check(y, orc.linear(H.Q8_0, data, rows, cols, x))


def test_batch_bracket_defers_host_results_to_finish():
    """Backend::begin_batch / finish_batch (src/backend/mod.rs:307-323): host-buffer calls inside the bracket are only
    enqueued; after finish_batch every output buffer holds its result."""
    rows, cols = 300, 768
    datas = [H.random_weight(t, rows, cols, seed=95 + i) for i, t in enumerate((H.Q8_0, H.Q4_K, H.Q4_0))]
    ws = [ctx().prepare_weight(t, d, rows, cols) for t, d in zip((H.Q8_0, H.Q4_K, H.Q4_0), datas)]
    xs = [np.random.default_rng(96 + i).standard_normal((m, cols)).astype(np.float32) for i, m in enumerate((1, 3, 9))]
    ys = [np.zeros((x.shape[0], rows), dtype=np.float32) for x in xs]
    ctx().begin_batch()
    for x, w, y in zip(xs, ws, ys):
        ctx().linear_host(x, w, y)
    ctx().finish_batch()
    for t, d, x, y in zip((H.Q8_0, H.Q4_K, H.Q4_0), datas, xs, ys):
        _check(y, orc.linear(t, d, rows, cols, x), tight=1e-3 if x.shape[0] > 8 else TIGHT)
    from zllm_b200 import ffi
    with pytest.raises(ffi.ZqFailure):
        ctx().finish_batch()  # no bracket open


def test_batch_bracket_with_page_locked_buffers_and_a_shared_input():
    """Page-locked caller buffers are copied from / to directly; one page-locked input given to several layers of a
    bracket travels once; the bracket's layers run as one batch at the finish.  Also a mixed bracket (f32 and f16
    inputs, a prefill-sized layer among the decode ones) and the same call outside a bracket."""
    rows, cols = 384, 1024
    types = (H.Q4_K, H.Q4_0, H.Q8_0, H.IQ4_NL)
    datas = [H.random_weight(t, rows, cols, seed=120 + i) for i, t in enumerate(types)]
    ws = [ctx().prepare_weight(t, d, rows, cols) for t, d in zip(types, datas)]
    x_t = torch.from_numpy(np.random.default_rng(121).standard_normal((3, cols)).astype(np.float32)).pin_memory()
    x16_t = x_t.to(torch.float16).pin_memory()
    big_t = torch.from_numpy(np.random.default_rng(122).standard_normal((40, cols)).astype(np.float32)).pin_memory()
    ys = [torch.zeros((3, rows), dtype=torch.float32).pin_memory() for _ in types]
    y16 = torch.zeros((3, rows), dtype=torch.float32).pin_memory()
    ybig = np.zeros((40, rows), dtype=np.float32)  # pageable output
    ctx().begin_batch()
    for w, y in zip(ws, ys):
        ctx().linear_host(x_t.numpy(), w, y.numpy())
    ctx().linear_host(x16_t.numpy(), ws[0], y16.numpy())
    ctx().linear_host(big_t.numpy(), ws[2], ybig)
    ctx().finish_batch()
    for t, d, y in zip(types, datas, ys):
        _check(y.numpy(), orc.linear(t, d, rows, cols, x_t.numpy()))
    _check(y16.numpy(), orc.linear(types[0], datas[0], rows, cols, x16_t.float().numpy()))
    assert H.max_rel_error(ybig, orc.linear(types[2], datas[2], rows, cols, big_t.numpy())) <= BOUND
    y_out = torch.zeros((3, rows), dtype=torch.float32).pin_memory()
    ctx().linear_host(x_t.numpy(), ws[1], y_out.numpy())  # outside a bracket: waits inside the call
    _check(y_out.numpy(), orc.linear(types[1], datas[1], rows, cols, x_t.numpy()))


def test_an_error_inside_a_bracket_closes_it():
    from zllm_b200 import ffi

    w = ctx().prepare_weight(H.Q4_K, H.random_weight(H.Q4_K, 64, 256, seed=130), 64, 256)
    x = np.zeros((1, 256), dtype=np.float32)
    y = np.zeros((1, 64), dtype=np.float32)
    ctx().begin_batch()
    ctx().linear_host(x, w, y)
    with pytest.raises(ffi.ZqFailure):
        ffi.call("zq_linear_host", ctx().handle, w.handle, x.ctypes.data_as(__import__("ctypes").c_void_p), 7, 1, y.ctypes.data_as(__import__("ctypes").c_void_p), ffi.F32)  # unknown dtype
    with pytest.raises(ffi.ZqFailure):
        ctx().finish_batch()  # the failed call closed the bracket
    ctx().begin_batch()       # and a new one opens cleanly
    ctx().linear_host(x, w, y)
    ctx().finish_batch()


def test_host_batch_is_a_whole_bracket_in_one_call():
    rows, cols = 384, 1024
    types = (H.Q4_K, H.Q8_0)
    datas = [H.random_weight(t, rows, cols, seed=140 + i) for i, t in enumerate(types)]
    ws = [ctx().prepare_weight(t, d, rows, cols) for t, d in zip(types, datas)]
    xs = [np.random.default_rng(141 + i).standard_normal((m, cols)).astype(np.float32) for i, m in enumerate((2, 5))]
    ys = [np.zeros((x.shape[0], rows), dtype=np.float32) for x in xs]
    ctx().linear_host_batch([(x, w, y) for x, w, y in zip(xs, ws, ys)])
    for t, d, x, y in zip(types, datas, xs, ys):
        _check(y, orc.linear(t, d, rows, cols, x))
    from zllm_b200 import ffi
    ctx().begin_batch()
    with pytest.raises(ffi.ZqFailure):
        ctx().linear_host_batch([(xs[0], ws[0], ys[0])])  # a bracket is already open; like every error this closes it
    with pytest.raises(ffi.ZqFailure):
        ctx().finish_batch()
