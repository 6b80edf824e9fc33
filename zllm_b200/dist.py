"""Multi-GPU plumbing for the quantized linear path: one process per GPU, ``torch.distributed`` (NCCL on GPUs,
gloo in the CPU tests).  Only the host-side logic lives here; every projection is a call into the CUDA library.

* Dense projections are tensor-parallel.  Up-projections (more outputs than inputs) are split by output rows and
  need no collective; down-projections are split by input columns on 256-column boundaries, because a K-quant
  super-block cannot be cut (the rule of the reference's 2-GPU operator pair, src/backend/rocm/expert.rs:182-207),
  and their f32 partial results are summed with one all-reduce (the reference exchanges and adds the two partials,
  src/backend/rocm/expert.rs:1394-1409).
* MoE experts are expert-parallel: rank r owns a contiguous block of experts, tokens stay data-parallel, routed
  rows travel with one all-to-all each way.  The reference has no such path (its experts are cached per device),
  so only its ordering rule is kept: a token's expert outputs are added in ascending expert id.
"""
from __future__ import annotations

from typing import Callable, List, Tuple

import torch
import torch.distributed as dist


def shard_plan(k: int, n: int, world: int, rank: int, block: int = 256, row_tile: int = 128) -> Tuple[str, Tuple[int, int], Tuple[int, int]]:
    """Shard of W[n, k] for ``rank``: ``(mode, (row_lo, row_hi), (col_lo, col_hi))``.

    mode "column": output rows split in ``row_tile`` multiples (last shards may be short or empty);
    mode "row": input columns split on ``block`` boundaries, shard sizes differ by at most one block."""
    if world == 1:
        return "none", (0, n), (0, k)
    if n >= k:
        per = -(-n // world)
        per = -(-per // row_tile) * row_tile
        return "column", (min(n, rank * per), min(n, (rank + 1) * per)), (0, k)
    if k % block:
        raise ValueError(f"row-parallel split needs columns aligned to {block}, got {k}")
    units = k // block
    base, extra = divmod(units, world)
    lo = rank * base + min(rank, extra)
    hi = lo + base + (1 if rank < extra else 0)
    return "row", (0, n), (lo * block, hi * block)


def expert_range(num_experts: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous block of experts owned by ``rank`` (sizes differ by at most one)."""
    base, extra = divmod(num_experts, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def expert_owner(expert_ids: torch.Tensor, num_experts: int, world: int) -> torch.Tensor:
    base, extra = divmod(num_experts, world)
    cut = extra * (base + 1)
    ids = expert_ids.long()
    small = torch.div(ids, base + 1, rounding_mode="floor")
    large = extra + torch.div(ids - cut, max(base, 1), rounding_mode="floor")
    return torch.where(ids < cut, small, large)


def row_parallel_reduce(partial: torch.Tensor, group=None) -> torch.Tensor:
    """Sum of the f32 partial outputs of a K-split projection over all ranks (in place)."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
    return partial


def expert_parallel_forward(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, num_experts: int,
                            run_local: Callable[[torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor], group=None) -> torch.Tensor:
    """Routed experts over expert-parallel ranks.

    ``x`` [m, hidden] are this rank's tokens, ``ids``/``weights`` [m, k] their routes.  ``run_local(rows, local_ids,
    route_weights)`` runs this rank's experts on received rows and returns ``weight * expert(row)`` as f32
    [n, hidden].  Returns the f32 routed sum per local token, contributions added in ascending expert id."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    m, k = ids.shape
    hidden = x.shape[1]
    flat_ids = ids.reshape(-1).long()
    flat_w = weights.reshape(-1).float()
    token_of = torch.arange(m, device=x.device).repeat_interleave(k)
    # order routes by (expert, token): rows for one destination are contiguous and, per token, ascending in expert
    order = torch.argsort(flat_ids * m + token_of, stable=True)
    s_ids, s_tok, s_w = flat_ids[order], token_of[order], flat_w[order]
    owner = expert_owner(s_ids, num_experts, world)
    send_counts = torch.bincount(owner, minlength=world)
    rows = x[s_tok].contiguous()
    lo, _ = expert_range(num_experts, world, rank)
    if world == 1:
        out_rows = run_local(rows, (s_ids - lo).int(), s_w)
    else:
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=group)
        send_l, recv_l = send_counts.tolist(), recv_counts.tolist()
        n_recv = int(sum(recv_l))
        r_rows = torch.empty((n_recv, hidden), dtype=x.dtype, device=x.device)
        dist.all_to_all_single(r_rows, rows, recv_l, send_l, group=group)
        meta = torch.stack([s_ids.float(), s_w], dim=1).contiguous()   # expert ids < 2^24 are exact in f32
        r_meta = torch.empty((n_recv, 2), dtype=torch.float32, device=x.device)
        dist.all_to_all_single(r_meta, meta, recv_l, send_l, group=group)
        r_out = run_local(r_rows, (r_meta[:, 0].long() - lo).int(), r_meta[:, 1].contiguous()) if n_recv else torch.empty((0, hidden), dtype=torch.float32, device=x.device)
        out_rows = torch.empty((rows.shape[0], hidden), dtype=torch.float32, device=x.device)
        dist.all_to_all_single(out_rows, r_out.contiguous(), send_l, recv_l, group=group)
    # combine: per token, its k rows in ascending expert id, added one after the other (fixed order, no atomics)
    back = torch.argsort(s_tok * num_experts + s_ids, stable=True)
    per_token = out_rows[back].view(m, k, hidden)
    acc = per_token[:, 0].clone()
    for j in range(1, k):
        acc += per_token[:, j]
    return acc
