"""Tensor-parallel row split on GPUs: the fused peer-store reduce (``zq_linear_row_parallel`` / ``ZQ_JOB_ROW_PARALLEL``)
against the CPU oracle on the FULL weight, through the C ABI.

* one GPU: a peer group of one is plain ``zq_linear``; a loop-back group of two (both handles are this rank's own, so the
  second rank's flag is never set) makes the bounded wait run out: the call returns, ``zq_ctx_sync`` reports the status,
  the context stays usable.  Nothing faults or hangs: the wait limit is 50 ms.
* two or more GPUs (skipped otherwise): one process per GPU; every rank holds a 256-column-aligned slice of the weight
  (the reference's partition rule, src/backend/rocm/expert.rs:182-207) and of the input; results are compared with the
  oracle and must be bit-identical on all ranks and across repeated calls and CUDA-graph replays.

Tolerance: 2e-3 (the layer contract) and 3e-4 (the integer-MMA decode arithmetic) for up to 16 rows.
"""
import ctypes as C
import os
import socket

import numpy as np
import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu

BOUND = 2e-3
# (type, rows, cols, activation rows): every width has at least 8 units of 256 columns, so up to 8 ranks get a slice
CASES = [(H.Q4_K, 640, 2560, 1), (H.Q4_K, 640, 2560, 4), (H.Q4_0, 384, 2048, 16), (H.Q8_0, 200, 2048, 2), (H.Q4_K, 512, 2304, 40)]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_group_of_one_is_plain_linear():
    from oracle import oracle as orc
    from zllm_b200 import ffi
    from zllm_b200.backend import B200Context

    c = B200Context(0)
    blob = (C.c_uint8 * ffi.DIST_HANDLE_BYTES)()
    ffi.call("zq_dist_export", c.handle, 1 << 20, blob)
    ffi.call("zq_dist_init", c.handle, 0, 1, blob)
    rows, cols = 300, 1024
    data = H.random_weight(H.Q4_K, rows, cols, seed=1)
    w = c.prepare_weight(H.Q4_K, data, rows, cols)
    x = np.random.default_rng(2).standard_normal((3, cols)).astype(np.float32)
    y = c.linear_row_parallel(torch.from_numpy(x).cuda(), w)
    c.sync()
    assert H.max_rel_error(y.cpu().numpy(), orc.linear(H.Q4_K, data, rows, cols, x)) <= 3e-4
    w.release()
    c.close()


def test_missing_peer_runs_into_the_wait_limit_and_the_context_survives():
    from oracle import oracle as orc
    from zllm_b200 import ffi
    from zllm_b200.backend import B200Context

    c = B200Context(0)
    blob = (C.c_uint8 * ffi.DIST_HANDLE_BYTES)()
    ffi.call("zq_dist_export", c.handle, 1 << 20, blob)
    both = (C.c_uint8 * (2 * ffi.DIST_HANDLE_BYTES))(*(list(blob) * 2))  # rank 1 "is" this buffer too: nobody sets its flags
    ffi.call("zq_dist_init", c.handle, 0, 2, both)
    ffi.call("zq_dist_set_wait_ms", c.handle, 50)
    rows, cols = 256, 512
    data = H.random_weight(H.Q4_K, rows, cols, seed=3)
    w = c.prepare_weight(H.Q4_K, data, rows, cols)
    x = np.random.default_rng(4).standard_normal((1, cols)).astype(np.float32)
    c.linear_row_parallel(torch.from_numpy(x).cuda(), w)
    with pytest.raises(ffi.ZqFailure) as info:
        c.sync()
    assert info.value.code == 5 and "peer" in info.value.message
    # the status is reported once; the context goes on working
    y = c.linear(torch.from_numpy(x).cuda(), w)
    c.sync()
    assert H.max_rel_error(y.cpu().numpy(), orc.linear(H.Q4_K, data, rows, cols, x)) <= 3e-4
    w.release()
    c.close()


EP = dict(experts=16, top_k=4, hidden=512, inter=256)


def _ep_inputs(m_total):
    """Experts, router outputs and tokens of the expert-parallel cases, the same on every rank (seeded)."""
    E, K, Hd, I = EP["experts"], EP["top_k"], EP["hidden"], EP["inter"]
    gates = [H.random_weight(H.Q4_K, I, Hd, seed=900 + 3 * e) for e in range(E + 1)]
    ups = [H.random_weight(H.Q4_K, I, Hd, seed=901 + 3 * e) for e in range(E + 1)]
    downs = [H.random_weight(H.Q4_K, Hd, I, seed=902 + 3 * e, std=0.05) for e in range(E + 1)]
    rng = np.random.default_rng(m_total)
    x = rng.standard_normal((m_total, Hd)).astype(np.float32)
    ids = np.stack([rng.permutation(E)[:K] for _ in range(m_total)]).astype(np.uint32)
    w = rng.random((m_total, K)).astype(np.float32)
    w /= w.sum(axis=1, keepdims=True)
    res = rng.standard_normal((m_total, Hd)).astype(np.float32)
    return gates, ups, downs, x, ids, w, res


def _ep_run(c, rank, world, m_total):
    """This rank's share of an expert-parallel forward; returns its output rows."""
    from zllm_b200.backend import MoeExperts, moe_forward_ep

    E, K, Hd, I = EP["experts"], EP["top_k"], EP["hidden"], EP["inter"]
    gates, ups, downs, x, ids, w, res = _ep_inputs(m_total)
    base, extra = divmod(E, world)
    lo = rank * base + min(rank, extra)
    hi = lo + base + (1 if rank < extra else 0)
    table = MoeExperts(c, [c.prepare_weight(H.Q4_K, gates[e], I, Hd) for e in range(lo, hi)], [c.prepare_weight(H.Q4_K, ups[e], I, Hd) for e in range(lo, hi)],
                       [c.prepare_weight(H.Q4_K, downs[e], Hd, I) for e in range(lo, hi)])
    shared = (c.prepare_weight(H.Q4_K, gates[E], I, Hd), c.prepare_weight(H.Q4_K, ups[E], I, Hd), c.prepare_weight(H.Q4_K, downs[E], Hd, I))
    per = m_total // world
    t0, t1 = rank * per, (rank + 1) * per
    xs = torch.from_numpy(x[t0:t1]).cuda().to(torch.bfloat16)
    out = []
    for _ in range(2):  # twice: the buffers are reused call after call
        y = moe_forward_ep(c, table, xs, torch.from_numpy(ids[t0:t1].astype(np.int32)).cuda(), torch.from_numpy(w[t0:t1]).cuda(), shared=shared,
                           residual=torch.from_numpy(res[t0:t1]).cuda(), out_dtype=torch.float32)
        c.sync()
        out.append(y.cpu().numpy())
    assert np.array_equal(out[0].view(np.uint32), out[1].view(np.uint32)), "a repeated call differs"
    return out[0]


def _ep_oracle(m_total):
    from oracle import oracle as orc

    E, K, Hd, I = EP["experts"], EP["top_k"], EP["hidden"], EP["inter"]
    gates, ups, downs, x, ids, w, res = _ep_inputs(m_total)
    x16 = torch.from_numpy(x).to(torch.bfloat16).float().numpy()  # what the device consumes
    sh = ((H.Q4_K, gates[E], I, Hd), (H.Q4_K, ups[E], I, Hd), (H.Q4_K, downs[E], Hd, I))
    return orc.moe_forward([(H.Q4_K, g, I, Hd) for g in gates[:E]], [(H.Q4_K, u, I, Hd) for u in ups[:E]], [(H.Q4_K, d, Hd, I) for d in downs[:E]], x16, ids, w, shared=sh, residual=res)


def test_expert_parallel_group_of_one_matches_the_oracle():
    """One rank owns every expert: rows are 'sent' to the rank itself through the same buffers and kernels."""
    from zllm_b200 import ffi
    from zllm_b200.backend import B200Context

    c = B200Context(0)
    blob = (C.c_uint8 * ffi.DIST_HANDLE_BYTES)()
    ffi.call("zq_dist_export", c.handle, 1 << 20, blob)
    ffi.call("zq_dist_init", c.handle, 0, 1, blob)
    eb = (C.c_uint8 * ffi.DIST_HANDLE_BYTES)()
    ffi.call("zq_moe_ep_export", c.handle, 320, EP["hidden"], EP["top_k"], EP["experts"], ffi.BF16, eb)
    ffi.call("zq_moe_ep_init", c.handle, eb)
    for m_total, bound in ((8, BOUND), (320, 2 * BOUND)):  # device-grouped decode path / host-grouped tensor-core path
        got = _ep_run(c, 0, 1, m_total)
        assert H.max_rel_error(got, _ep_oracle(m_total)) <= bound
    c.close()


def _rank_main(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    from zllm_b200.backend import B200Context

    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    c = B200Context(rank)
    c.dist_init(slot_bytes=2 << 20)
    results = {}
    cases = CASES
    for ci, (tt, rows, cols, m) in enumerate(cases):
        full = (np.random.default_rng(100 + ci).standard_normal((rows, cols)) * 0.02).astype(np.float32)
        x = np.random.default_rng(200 + ci).standard_normal((m, cols)).astype(np.float32)
        res = np.random.default_rng(300 + ci).standard_normal((m, rows)).astype(np.float32)
        c0, c1 = _cols_of(cols, world, rank)
        shard = H.quantize(tt, np.ascontiguousarray(full[:, c0:c1]))
        w = c.prepare_weight(tt, shard, rows, c1 - c0)
        xs = torch.from_numpy(np.ascontiguousarray(x[:, c0:c1])).cuda()
        y1 = c.linear_row_parallel(xs, w, residual=torch.from_numpy(res).cuda())
        y2 = c.linear_row_parallel(xs, w, residual=torch.from_numpy(res).cuda())  # the other buffer half
        c.sync()
        results[f"case{ci}"] = y1.cpu().numpy()
        results[f"case{ci}_again"] = y2.cpu().numpy()
        w.release()
    # a batch with a column-parallel and two row-parallel jobs, captured in a CUDA graph and replayed
    rows, cols, m = 512, 2048, 2
    full = (np.random.default_rng(7).standard_normal((rows, cols)) * 0.02).astype(np.float32)
    x = np.random.default_rng(8).standard_normal((m, cols)).astype(np.float32)
    c0, c1 = _cols_of(cols, world, rank)
    w_row = c.prepare_weight(H.Q4_K, H.quantize(H.Q4_K, np.ascontiguousarray(full[:, c0:c1])), rows, c1 - c0)
    r0, r1 = rank * rows // world, (rank + 1) * rows // world
    w_col = c.prepare_weight(H.Q4_K, H.quantize(H.Q4_K, np.ascontiguousarray(full[r0:r1])), r1 - r0, cols)
    xs, xf = torch.from_numpy(np.ascontiguousarray(x[:, c0:c1])).cuda(), torch.from_numpy(x).cuda()
    jobs = [(xf, w_col), (xs, w_row, None, "row"), (xs, w_row, None, "row")]
    c.linear_batch(jobs)  # sizes the internal buffers
    c.sync()
    dist.barrier()
    side = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        c.set_stream(torch.cuda.current_stream().cuda_stream)
        ys = c.linear_batch(jobs)
    c.set_stream(torch.cuda.current_stream().cuda_stream)
    for _ in range(5):
        g.replay()
    torch.cuda.synchronize()
    c.sync()
    results["graph_col"] = ys[0].cpu().numpy()
    results["graph_row"] = ys[1].cpu().numpy()
    results["graph_row2"] = ys[2].cpu().numpy()
    # expert parallelism: 16 experts over the ranks, a decode-sized and a prefill-sized batch
    c.moe_ep_init(40 * 8 // world, EP["hidden"], EP["top_k"], EP["experts"], dtype=torch.bfloat16)
    for m_total in (8, 320):
        results[f"ep{m_total}"] = _ep_run(c, rank, world, m_total)
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), **results)
    dist.barrier()
    w_row.release()
    w_col.release()
    c.close()
    dist.destroy_process_group()


def _cols_of(cols, world, rank, block=256):
    units = cols // block
    base, extra = divmod(units, world)
    lo = rank * base + min(rank, extra)
    hi = lo + base + (1 if rank < extra else 0)
    return lo * block, hi * block


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_row_parallel_on_all_gpus_matches_the_oracle_on_the_full_weight(tmp_path):
    import torch.multiprocessing as mp

    from oracle import oracle as orc

    world = min(torch.cuda.device_count(), 8)
    port = _free_port()
    mp.spawn(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    outs = [np.load(os.path.join(str(tmp_path), f"rank{r}.npz")) for r in range(world)]
    cases = CASES
    for ci, (tt, rows, cols, m) in enumerate(cases):
        full = (np.random.default_rng(100 + ci).standard_normal((rows, cols)) * 0.02).astype(np.float32)
        x = np.random.default_rng(200 + ci).standard_normal((m, cols)).astype(np.float32)
        res = np.random.default_rng(300 + ci).standard_normal((m, rows)).astype(np.float32)
        # the oracle sees the concatenation of the ranks' quantised slices = the full quantised weight
        want = res.astype(np.float64)
        for r in range(world):
            c0, c1 = _cols_of(cols, world, r)
            if c1 > c0:
                shard = H.quantize(tt, np.ascontiguousarray(full[:, c0:c1]))
                want = want + orc.linear(tt, shard, rows, c1 - c0, np.ascontiguousarray(x[:, c0:c1])).astype(np.float64)
        for r in range(world):
            got = outs[r][f"case{ci}"]
            assert H.max_rel_error(got, want) <= (3e-4 if m <= 16 else BOUND), (ci, r)
            assert np.array_equal(got.view(np.uint32), outs[0][f"case{ci}"].view(np.uint32)), "ranks disagree"
            assert np.array_equal(got.view(np.uint32), outs[r][f"case{ci}_again"].view(np.uint32)), "a repeated call differs"
    for m_total, bound in ((8, BOUND), (320, 2 * BOUND)):
        got = np.concatenate([outs[r][f"ep{m_total}"] for r in range(world)])
        assert H.max_rel_error(got, _ep_oracle(m_total)) <= bound, f"expert-parallel forward, {m_total} tokens"
    rows, cols, m = 512, 2048, 2
    full = (np.random.default_rng(7).standard_normal((rows, cols)) * 0.02).astype(np.float32)
    x = np.random.default_rng(8).standard_normal((m, cols)).astype(np.float32)
    want = np.zeros((m, rows))
    for r in range(world):
        c0, c1 = _cols_of(cols, world, r)
        want = want + orc.linear(H.Q4_K, H.quantize(H.Q4_K, np.ascontiguousarray(full[:, c0:c1])), rows, c1 - c0, np.ascontiguousarray(x[:, c0:c1])).astype(np.float64)
    for r in range(world):
        assert H.max_rel_error(outs[r]["graph_row"], want) <= 3e-4
        assert np.array_equal(outs[r]["graph_row"].view(np.uint32), outs[r]["graph_row2"].view(np.uint32))
        r0, r1 = r * rows // world, (r + 1) * rows // world
        col_want = orc.linear(H.Q4_K, H.quantize(H.Q4_K, np.ascontiguousarray(full[r0:r1])), r1 - r0, cols, x)
        assert H.max_rel_error(outs[r]["graph_col"], col_want) <= 3e-4
