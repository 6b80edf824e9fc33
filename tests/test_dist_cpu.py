"""Host-side multi-GPU logic on CPU ranks (gloo, world_size 2): shard plans, row-parallel reduce, expert-parallel
dispatch/combine bookkeeping with a stand-in expert function."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from zllm_b200 import dist as zd


@pytest.mark.parametrize("k,n", [(3840, 3840), (3840, 15360), (15360, 3840), (5120, 17408), (17408, 5120)])
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_shard_plan_covers_the_matrix_on_legal_boundaries(k, n, world):
    rows, cols = [], []
    for r in range(world):
        mode, (r0, r1), (c0, c1) = zd.shard_plan(k, n, world, r)
        rows.append((r0, r1))
        cols.append((c0, c1))
        if mode == "row":
            assert c0 % 256 == 0 and c1 % 256 == 0          # K-quant super-blocks are never cut
            assert (r0, r1) == (0, n)
        elif mode == "column":
            assert r0 % 128 == 0 and (c0, c1) == (0, k)
    spans = rows if n >= k or world == 1 else cols
    total = n if n >= k or world == 1 else k
    assert spans[0][0] == 0 and spans[-1][1] == total
    for a, b in zip(spans, spans[1:]):
        assert a[1] == b[0]
    if world > 1 and n < k:
        sizes = [c1 - c0 for c0, c1 in cols]
        assert max(sizes) - min(sizes) <= 256                # e.g. 68 super-blocks over 8 ranks: 4x9 + 4x8


def test_row_split_rejects_unaligned_columns():
    """src/backend/rocm/expert.rs:203-207: shapes that cannot be cut on super-block boundaries are errors."""
    with pytest.raises(ValueError):
        zd.shard_plan(4000, 128, 2, 0)


def test_expert_owner_matches_expert_range():
    for experts, world in [(256, 8), (10, 4), (7, 2), (5, 8)]:
        ids = torch.arange(experts)
        owner = zd.expert_owner(ids, experts, world)
        for r in range(world):
            lo, hi = zd.expert_range(experts, world, r)
            assert torch.all(owner[lo:hi] == r)


def _toy_expert(rows, local_ids, w, lo):
    gid = local_ids.long() + lo
    return (rows.float() * (gid.float() + 1.0).unsqueeze(1) + gid.float().unsqueeze(1)) * w.unsqueeze(1)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(5)
        experts, k, hidden, m_total = 6, 2, 16, 10
        x_all = torch.randn((m_total, hidden), generator=g)
        ids_all = torch.stack([torch.randperm(experts, generator=g)[:k] for _ in range(m_total)]).int()
        w_all = torch.rand((m_total, k), generator=g)
        per = m_total // world
        sl = slice(rank * per, (rank + 1) * per)
        lo, _ = zd.expert_range(experts, world, rank)
        got = zd.expert_parallel_forward(x_all[sl], ids_all[sl], w_all[sl], experts, lambda r, i, w: _toy_expert(r, i, w, lo))
        # single-process reference: per token, ascending expert id
        want = torch.zeros((per, hidden))
        for t in range(per):
            order = torch.argsort(ids_all[sl][t].long())
            for j in order:
                e = int(ids_all[sl][t, j])
                want[t] += (x_all[sl][t] * (e + 1.0) + e) * w_all[sl][t, j]
        ok_ep = torch.equal(got, want)
        part = torch.full((3, 4), float(rank + 1))
        zd.row_parallel_reduce(part)
        ok_rp = bool(torch.all(part == sum(range(1, world + 1))))
        out.put((rank, ok_ep, ok_rp))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_dispatch_and_row_parallel_reduce_on_two_ranks():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok_ep, ok_rp in results:
        assert ok_ep, f"rank {rank}: expert-parallel result differs from the single-process order"
        assert ok_rp, f"rank {rank}: all-reduce sum wrong"
