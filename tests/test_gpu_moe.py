"""GPU parity of the MoE layer (router, grouping, routed experts, shared expert, combine) against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import helpers as H
from tests.gpu_util import ctx, dev, host

pytestmark = pytest.mark.gpu
BOUND = 2e-3


def _experts(tensor_type, n, hidden, inter, seed):
    gates = [H.random_weight(tensor_type, inter, hidden, seed=seed + 3 * e) for e in range(n)]
    ups = [H.random_weight(tensor_type, inter, hidden, seed=seed + 3 * e + 1) for e in range(n)]
    downs = [H.random_weight(tensor_type, hidden, inter, seed=seed + 3 * e + 2, std=0.05) for e in range(n)]
    return gates, ups, downs


@pytest.mark.parametrize("m,experts,top_k,hidden", [(1, 8, 2, 512), (5, 16, 4, 256), (64, 256, 8, 512), (33, 12, 3, 1024), (300, 64, 6, 1024), (1000, 12, 2, 256)])
@pytest.mark.parametrize("normalize", [True, False])
def test_router_matches_cpu_softmax_topk(m, experts, top_k, hidden, normalize):
    """src/moe/routing.rs:25-39 through the device router (src/kernel/cuda/routing.rs:15-62)."""
    from zllm_b200.backend import moe_route

    rng = np.random.default_rng(m + experts)
    x = rng.standard_normal((m, hidden)).astype(np.float32)
    router = (rng.standard_normal((experts, hidden)) / np.sqrt(hidden)).astype(np.float32)
    ids, w = moe_route(ctx(), dev(x), dev(router), top_k, 1.5, normalize)
    ctx().sync()
    want_ids, want_w = orc.moe_route_softmax(x, router, top_k, 1.5, normalize)
    got_ids = ids.cpu().numpy().astype(np.uint32)
    assert np.array_equal(got_ids, want_ids)
    np.testing.assert_allclose(w.cpu().numpy(), want_w, rtol=2e-5, atol=1e-7)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,experts,top_k,hidden", [(5, 16, 4, 256), (64, 256, 8, 1024), (13, 200, 6, 7168)])
def test_router_with_half_precision_rows(m, experts, top_k, hidden, dtype):
    """Decode-sized batches of f16 / bf16 rows take the kernel that keeps the rows as 16-bit values in shared memory; the
    oracle sees the same rounded rows, and a bias takes part in the softmax."""
    from zllm_b200.backend import moe_route

    rng = np.random.default_rng(3 * m + experts)
    x = torch.from_numpy(rng.standard_normal((m, hidden)).astype(np.float32)).to(dtype)
    router = (rng.standard_normal((experts, hidden)) / np.sqrt(hidden)).astype(np.float32)
    bias = (0.1 * rng.standard_normal(experts)).astype(np.float32)
    ids, w = moe_route(ctx(), x.cuda(), dev(router), top_k, 1.0, True, bias=dev(bias))
    ctx().sync()
    logits = (x.float().numpy().astype(np.float64) @ router.astype(np.float64).T + bias).astype(np.float32)
    rows = [orc.route_softmax_logits(logits[t], top_k, 1.0, True) for t in range(m)]
    want_ids, want_w = np.stack([r[0] for r in rows]).reshape(m, top_k), np.stack([r[1] for r in rows]).reshape(m, top_k)
    # a near-tie may order differently in f32 and f64 logits: compare where the logit gap is clear
    order = np.sort(logits, axis=1)[:, ::-1]
    clear = np.all(np.abs(np.diff(order[:, :top_k + 1], axis=1)) > 1e-5, axis=1)
    assert clear.mean() > 0.9
    assert np.array_equal(ids.cpu().numpy().astype(np.uint32)[clear], want_ids[clear])
    np.testing.assert_allclose(w.cpu().numpy()[clear], want_w[clear], rtol=1e-4, atol=1e-6)


def test_router_breaks_ties_by_lower_expert_id():
    from zllm_b200.backend import moe_route

    hidden, experts = 64, 6
    x = np.ones((1, hidden), dtype=np.float32)
    router = np.zeros((experts, hidden), dtype=np.float32)
    router[1] = router[3] = router[4] = 0.5   # three equal logits
    router[0] = 0.25
    ids, _ = moe_route(ctx(), dev(x), dev(router), 2, 1.0, True)
    ctx().sync()
    assert list(ids.cpu().numpy()[0]) == [1, 3]


@pytest.fixture(params=["grouped", "per_expert"])
def moe_path(request):
    """Both orchestrations: everything on the device in grouped launches (decode-sized batches), or host-grouped
    routes with one pair of calls per expert (what larger batches use)."""
    ctx().set_option("force_moe_per_expert", 1 if request.param == "per_expert" else 0)
    yield request.param
    ctx().set_option("force_moe_per_expert", 0)


@pytest.mark.parametrize("tensor_type", [H.Q4_K, H.Q8_0, H.Q4_0])
@pytest.mark.parametrize("m", [1, 6, 48])
@pytest.mark.parametrize("with_shared", [False, True])
def test_moe_forward_matches_cpu_path(tensor_type, m, with_shared, moe_path):
    """Routed + shared experts + residual against the oracle's moe_forward (decode and prefill orchestration:
    experts with few routed tokens run the decode kernel, experts with more than 16 the tensor-core GEMM)."""
    from zllm_b200.backend import MoeExperts, moe_forward, moe_route

    n_exp, top_k, hidden, inter = 8, 2, 512, 256
    gates, ups, downs = _experts(tensor_type, n_exp, hidden, inter, seed=100)
    rng = np.random.default_rng(7 + m)
    x = rng.standard_normal((m, hidden)).astype(np.float32)
    router = (rng.standard_normal((n_exp, hidden)) / np.sqrt(hidden)).astype(np.float32)
    residual = rng.standard_normal((m, hidden)).astype(np.float32)
    c = ctx()
    wg = [c.prepare_weight(tensor_type, g, inter, hidden) for g in gates]
    wu = [c.prepare_weight(tensor_type, u, inter, hidden) for u in ups]
    wd = [c.prepare_weight(tensor_type, d, hidden, inter) for d in downs]
    table = MoeExperts(c, wg, wu, wd)
    shared_np = shared_dev = None
    if with_shared:
        sg, su = H.random_weight(tensor_type, inter, hidden, seed=900), H.random_weight(tensor_type, inter, hidden, seed=901)
        sd = H.random_weight(tensor_type, hidden, inter, seed=902, std=0.05)
        shared_np = [(tensor_type, sg, inter, hidden), (tensor_type, su, inter, hidden), (tensor_type, sd, hidden, inter)]
        shared_dev = (c.prepare_weight(tensor_type, sg, inter, hidden), c.prepare_weight(tensor_type, su, inter, hidden), c.prepare_weight(tensor_type, sd, hidden, inter))
    xd = dev(x)
    ids, w = moe_route(c, xd, dev(router), top_k, 1.0, True)
    got = host(moe_forward(c, table, xd, ids, w, shared=shared_dev, residual=dev(residual)))
    ids_np, w_np = ids.cpu().numpy().astype(np.uint32), w.cpu().numpy()
    want = orc.moe_forward([(tensor_type, g, inter, hidden) for g in gates], [(tensor_type, u, inter, hidden) for u in ups], [(tensor_type, d, hidden, inter) for d in downs], x, ids_np, w_np,
                           shared=shared_np, residual=residual)
    assert H.max_rel_error(got, want) <= BOUND


@pytest.mark.parametrize("tensor_type", [H.Q4_K, H.Q8_0])
@pytest.mark.parametrize("m", [150, 700])
def test_moe_prefill_runs_grouped_tensor_core_gemms(tensor_type, m, moe_path):
    """Prefill-sized batches (>= 32 routed rows per expert): one grouped GEMM per projection over all experts, against
    the same oracle; the per-expert path (one pair of GEMM calls per expert) must agree too.  Expert 3 gets no tokens.

    Tolerance: each tensor-core GEMM meets the 2e-3 max bound on its own (tests/test_gpu_gemm.py).  The MoE layer
    chains two of them (gate/up -> SiLU -> down, the intermediate passing through f16 as the second GEMM's operand)
    and adds top-k results, so the WORST of ~10^5 outputs lands near 3e-3 while the relative L2 error stays below
    5e-4; the test holds the composite to 4e-3 max and 1e-3 L2."""
    from zllm_b200.backend import MoeExperts, moe_forward

    n_exp, top_k, hidden, inter = 4, 2, 512, 768
    gates, ups, downs = _experts(tensor_type, n_exp, hidden, inter, seed=700)
    rng = np.random.default_rng(70 + m)
    x = rng.standard_normal((m, hidden)).astype(np.float32)
    ids_np = np.stack([rng.permutation(3)[:top_k] for _ in range(m)]).astype(np.uint32)  # experts 0..2 only
    w_np = rng.random((m, top_k)).astype(np.float32)
    w_np /= w_np.sum(axis=1, keepdims=True)
    c = ctx()
    table = MoeExperts(c, [c.prepare_weight(tensor_type, g, inter, hidden) for g in gates], [c.prepare_weight(tensor_type, u, inter, hidden) for u in ups],
                       [c.prepare_weight(tensor_type, d, hidden, inter) for d in downs])
    ids = torch.from_numpy(ids_np.astype(np.int32)).cuda()
    got = host(moe_forward(c, table, dev(x), ids, dev(w_np)))
    want = orc.moe_forward([(tensor_type, g, inter, hidden) for g in gates], [(tensor_type, u, inter, hidden) for u in ups], [(tensor_type, d, hidden, inter) for d in downs], x, ids_np, w_np)
    assert H.max_rel_error(got, want) <= 2 * BOUND
    assert float(np.linalg.norm(got - want) / np.linalg.norm(want)) <= 1e-3


@pytest.mark.parametrize("gate_type,down_type", [(H.Q4_K, H.Q6_K), (H.Q5_K, H.Q5_K), (H.IQ4_NL, H.IQ4_NL), (H.Q6_K, H.Q4_K)])
def test_moe_decode_with_mixed_expert_types(gate_type, down_type, moe_path):
    """Files mix types inside an expert (a Q4_K_M file carries Q6_K down projections; the reference's CUDA experts accept
    Q5_K / Q6_K down matrices, src/backend/cuda/expert.rs:462-473): the grouped decode launches take every type the
    integer-MMA kernels unpack, one type for gate/up and one for down."""
    from zllm_b200.backend import MoeExperts, moe_forward

    n_exp, top_k, hidden, inter, m = 6, 2, 512, 256, 7
    gates = [H.random_weight(gate_type, inter, hidden, seed=610 + 3 * e) for e in range(n_exp)]
    ups = [H.random_weight(gate_type, inter, hidden, seed=611 + 3 * e) for e in range(n_exp)]
    downs = [H.random_weight(down_type, hidden, inter, seed=612 + 3 * e, std=0.05) for e in range(n_exp)]
    rng = np.random.default_rng(61)
    x = rng.standard_normal((m, hidden)).astype(np.float32)
    ids_np = np.stack([rng.permutation(n_exp)[:top_k] for _ in range(m)]).astype(np.uint32)
    w_np = rng.random((m, top_k)).astype(np.float32)
    c = ctx()
    table = MoeExperts(c, [c.prepare_weight(gate_type, g, inter, hidden) for g in gates], [c.prepare_weight(gate_type, u, inter, hidden) for u in ups],
                       [c.prepare_weight(down_type, d, hidden, inter) for d in downs])
    got = host(moe_forward(c, table, dev(x), torch.from_numpy(ids_np.astype(np.int32)).cuda(), dev(w_np)))
    want = orc.moe_forward([(gate_type, g, inter, hidden) for g in gates], [(gate_type, u, inter, hidden) for u in ups], [(down_type, d, hidden, inter) for d in downs], x, ids_np, w_np)
    assert H.max_rel_error(got, want) <= BOUND


def test_moe_prefill_grouping_on_the_device_equals_grouping_on_the_host():
    """Prefill with Q4_K experts groups the routes on the device (a stable counting sort over chunks of tokens) and
    hands the grouped GEMMs their work lists without a host round trip.  Slots, combine order and work lists are
    those of the host grouping (src/moe/routing.rs:136-156), so the two give the same bits: several chunks, an
    expert without tokens, an expert with several 256-token tiles, absent routes, a shared expert and a residual."""
    from zllm_b200 import ffi
    from zllm_b200.backend import MoeExperts, moe_forward

    n_exp, top_k, hidden, inter, m = 6, 3, 512, 256, 1300
    gates, ups, downs = _experts(H.Q4_K, n_exp, hidden, inter, seed=820)
    rng = np.random.default_rng(82)
    x = rng.standard_normal((m, hidden)).astype(np.float32)
    # expert 4 never chosen, expert 0 on most tokens
    ids_np = np.stack([np.concatenate(([0], rng.permutation([1, 2, 3, 5])[:top_k - 1])) if rng.random() < 0.8 else rng.permutation([1, 2, 3, 5])[:top_k] for _ in range(m)]).astype(np.uint32)
    w_np = rng.random((m, top_k)).astype(np.float32)
    absent = rng.random((m, top_k)) < 0.15
    ids_np[absent] = ffi.MOE_NO_ROUTE
    resid = rng.standard_normal((m, hidden)).astype(np.float32)
    c = ctx()
    table = MoeExperts(c, [c.prepare_weight(H.Q4_K, g, inter, hidden) for g in gates], [c.prepare_weight(H.Q4_K, u, inter, hidden) for u in ups], [c.prepare_weight(H.Q4_K, d, hidden, inter) for d in downs])
    sh = _experts(H.Q4_K, 1, hidden, inter, seed=990)
    shared = (c.prepare_weight(H.Q4_K, sh[0][0], inter, hidden), c.prepare_weight(H.Q4_K, sh[1][0], inter, hidden), c.prepare_weight(H.Q4_K, sh[2][0], hidden, inter))
    ids = torch.from_numpy(ids_np.view(np.int32)).cuda()
    xd, wd, rd = dev(x), dev(w_np), dev(resid)
    on_device = host(moe_forward(c, table, xd, ids, wd, shared=shared, residual=rd)).copy()
    again = host(moe_forward(c, table, xd, ids, wd, shared=shared, residual=rd)).copy()
    c.set_option("force_moe_host_grouping", 1)
    try:
        on_host = host(moe_forward(c, table, xd, ids, wd, shared=shared, residual=rd)).copy()
    finally:
        c.set_option("force_moe_host_grouping", 0)
    assert np.array_equal(on_device.view(np.uint32), again.view(np.uint32))
    assert np.array_equal(on_device.view(np.uint32), on_host.view(np.uint32))
    # and against the oracle (absent routes carry weight 0 there)
    ids_o, w_o = ids_np.copy(), w_np.copy()
    w_o[absent] = 0.0
    ids_o[absent] = 4
    want = orc.moe_forward([(H.Q4_K, g, inter, hidden) for g in gates], [(H.Q4_K, u, inter, hidden) for u in ups], [(H.Q4_K, d, hidden, inter) for d in downs], x, ids_o, w_o,
                           shared=[(H.Q4_K, sh[0][0], inter, hidden), (H.Q4_K, sh[1][0], inter, hidden), (H.Q4_K, sh[2][0], hidden, inter)], residual=resid)
    assert H.max_rel_error(on_device, want) <= 2 * BOUND


def test_shared_expert_of_another_width_takes_its_own_launches():
    """A shared expert shaped like the routed ones rides along in the grouped launches; any other shape runs as a
    separate gated MLP (src/moe/topk_moe.rs:84-104) and is added in the combine."""
    from zllm_b200.backend import MoeExperts, moe_forward, moe_route

    n_exp, top_k, hidden, inter, shared_inter, m = 8, 2, 512, 256, 128, 5
    gates, ups, downs = _experts(H.Q4_K, n_exp, hidden, inter, seed=500)
    rng = np.random.default_rng(55)
    x = rng.standard_normal((m, hidden)).astype(np.float32)
    router = (rng.standard_normal((n_exp, hidden)) / np.sqrt(hidden)).astype(np.float32)
    c = ctx()
    table = MoeExperts(c, [c.prepare_weight(H.Q4_K, g, inter, hidden) for g in gates], [c.prepare_weight(H.Q4_K, u, inter, hidden) for u in ups], [c.prepare_weight(H.Q4_K, d, hidden, inter) for d in downs])
    sg, su = H.random_weight(H.Q8_0, shared_inter, hidden, seed=910), H.random_weight(H.Q8_0, shared_inter, hidden, seed=911)
    sd = H.random_weight(H.Q8_0, hidden, shared_inter, seed=912, std=0.05)
    shared_dev = (c.prepare_weight(H.Q8_0, sg, shared_inter, hidden), c.prepare_weight(H.Q8_0, su, shared_inter, hidden), c.prepare_weight(H.Q8_0, sd, hidden, shared_inter))
    xd = dev(x)
    ids, w = moe_route(c, xd, dev(router), top_k, 1.0, True)
    got = host(moe_forward(c, table, xd, ids, w, shared=shared_dev))
    want = orc.moe_forward([(H.Q4_K, g, inter, hidden) for g in gates], [(H.Q4_K, u, inter, hidden) for u in ups], [(H.Q4_K, d, hidden, inter) for d in downs], x, ids.cpu().numpy().astype(np.uint32), w.cpu().numpy(),
                           shared=[(H.Q8_0, sg, shared_inter, hidden), (H.Q8_0, su, shared_inter, hidden), (H.Q8_0, sd, hidden, shared_inter)], residual=None)
    assert H.max_rel_error(got, want) <= BOUND


def test_moe_forward_rejects_bad_expert_ids():
    from zllm_b200 import ffi
    from zllm_b200.backend import MoeExperts, moe_forward

    n_exp, hidden, inter = 2, 256, 256
    gates, ups, downs = _experts(H.Q4_K, n_exp, hidden, inter, seed=300)
    c = ctx()
    table = MoeExperts(c, [c.prepare_weight(H.Q4_K, g, inter, hidden) for g in gates], [c.prepare_weight(H.Q4_K, u, inter, hidden) for u in ups], [c.prepare_weight(H.Q4_K, d, hidden, inter) for d in downs])
    x = dev(np.zeros((1, hidden), dtype=np.float32))
    bad_ids, w = torch.tensor([[0, 5]], dtype=torch.int32, device="cuda"), torch.tensor([[0.5, 0.5]], device="cuda")
    # host-grouped path: the ids are read on the host, the call itself fails
    c.set_option("force_moe_per_expert", 1)
    try:
        with pytest.raises(ffi.ZqFailure):
            moe_forward(c, table, x, bad_ids, w)
    finally:
        c.set_option("force_moe_per_expert", 0)
    # device-grouped path: nothing comes back to the host; the kernel skips the bad index (no out-of-range access),
    # records it in the status word, and the next sync reports it
    moe_forward(c, table, x, bad_ids, w)
    with pytest.raises(ffi.ZqFailure):
        c.sync()
    c.sync()  # reported once, then clear


def test_gather_and_scatter_add_rows_on_their_own():
    """Backend::moe_gather_rows / moe_scatter_add_rows (src/backend/mod.rs:1657-1662) as exported entries: an expert's
    tokens are gathered, its outputs are added into an f32 accumulator with their route weights
    (src/moe/routing.rs:180-213), row ids out of range are skipped and reported."""
    from zllm_b200 import ffi
    from zllm_b200.backend import moe_gather_rows, moe_scatter_add_rows

    rng = np.random.default_rng(3)
    x = rng.standard_normal((20, 64)).astype(np.float32)
    ids = np.array([19, 0, 7, 3], dtype=np.int32)
    for dtype in (torch.float32, torch.float16, torch.bfloat16):
        xd = torch.from_numpy(x).cuda().to(dtype)
        got = moe_gather_rows(ctx(), xd, torch.from_numpy(ids))
        ctx().sync()
        assert torch.equal(got.cpu(), xd.cpu()[ids.astype(np.int64)])
    acc = torch.zeros((20, 64), dtype=torch.float32, device="cuda")
    rows = rng.standard_normal((4, 64)).astype(np.float32)
    w = rng.random(4).astype(np.float32)
    moe_scatter_add_rows(ctx(), acc, torch.from_numpy(rows).cuda().to(torch.float16), torch.from_numpy(ids), torch.from_numpy(w).cuda())
    moe_scatter_add_rows(ctx(), acc, torch.from_numpy(rows).cuda().to(torch.float16), torch.from_numpy(ids), torch.from_numpy(w).cuda())
    ctx().sync()
    want = np.zeros((20, 64), dtype=np.float32)
    r16 = rows.astype(np.float16).astype(np.float32)
    for _ in range(2):
        for i, t in enumerate(ids):
            want[t] += r16[i] * w[i]
    np.testing.assert_allclose(acc.cpu().numpy(), want, rtol=1e-6, atol=1e-7)
    moe_scatter_add_rows(ctx(), acc, torch.from_numpy(rows).cuda(), torch.tensor([0, 1, 2, 99], dtype=torch.int32), None)
    with pytest.raises(ffi.ZqFailure):
        ctx().sync()
    ctx().sync()
