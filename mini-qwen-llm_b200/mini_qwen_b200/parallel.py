"""Expert parallelism for the MoE block: experts are sharded across the G GPUs of one box, tokens
stay data-parallel, and rows travel to their experts and back in one all-to-all each way.

The reference has no distributed code at all; this is the one place where the path has a real
exchange step.  Layout facts the exchange relies on:

* rank r owns the contiguous expert range ``[r*E/G, (r+1)*E/G)``;
* a rank's slots are already sorted by GLOBAL expert id (the permute plan), hence grouped by
  destination rank: the rows for rank d are ``permuted[off[d*E/G] : off[(d+1)*E/G]]``;
* what a rank receives is ordered by (source rank, local expert).  The grouped kernels take that
  order as it is: G*E/G groups over E/G weight matrices (group g uses weight g % (E/G)), so no
  second sort or copy is needed on the receiving side;
* the way back is the same exchange with send and receive sizes swapped, which lands every row at
  the position it left from.

The functions here only use ``torch.distributed`` collectives on whatever device the tensors live
on (NCCL over NVLink on GPUs; gloo in the CPU tests of the exchange logic).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

import torch
import torch.distributed as dist


@dataclass
class ExchangePlan:
    send_splits: List[int]        # rows this rank sends to each rank (dispatch direction)
    recv_splits: List[int]        # rows this rank receives from each rank
    seg_offsets: torch.Tensor     # int32 [G * E_local + 1]: received rows grouped by (source, local expert)
    recv_rows: int


def gather_counts(counts: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather of the per-expert slot counts: ``counts`` int32 [E] -> int32 [G, E]."""
    G = dist.get_world_size(group)
    flat = torch.empty(G * counts.numel(), dtype=counts.dtype, device=counts.device)
    dist.all_gather_into_tensor(flat, counts.contiguous().reshape(-1), group=group)
    return flat.reshape(G, counts.numel())


def make_plan(all_counts: torch.Tensor, rank: int, device=None) -> ExchangePlan:
    """Split sizes and receive-side group offsets from the gathered counts [G, E].

    The split sizes must be known on the host (they are arguments of the collective), so this is
    the one host synchronisation of an expert-parallel layer call.
    """
    G, E = all_counts.shape
    if E % G != 0:
        raise ValueError(f"{E} experts do not shard evenly over {G} ranks")
    el = E // G
    host = all_counts.detach().to("cpu", torch.int64)
    per_dest = host.reshape(G, G, el).sum(dim=2)            # [source, destination]
    send_splits = per_dest[rank].tolist()
    recv_splits = per_dest[:, rank].tolist()
    mine = host[:, rank * el:(rank + 1) * el].reshape(-1)   # (source, local expert) order
    seg = torch.zeros(G * el + 1, dtype=torch.int32)
    seg[1:] = torch.cumsum(mine, 0).to(torch.int32)
    recv_rows = int(seg[-1])
    if recv_rows != sum(recv_splits):
        raise RuntimeError("inconsistent expert counts across ranks")
    dev = device if device is not None else all_counts.device
    return ExchangePlan(send_splits, recv_splits, seg.to(dev, non_blocking=True), recv_rows)


def dispatch(rows: torch.Tensor, plan: ExchangePlan, group=None) -> torch.Tensor:
    """Expert-sorted local rows [S, H] -> the rows of this rank's experts [R, H]."""
    if rows.shape[0] != sum(plan.send_splits):
        raise ValueError("row count does not match the plan's send sizes")
    out = torch.empty(plan.recv_rows, rows.shape[1], dtype=rows.dtype, device=rows.device)
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=plan.recv_splits,
                           input_split_sizes=plan.send_splits, group=group)
    return out


def combine(rows: torch.Tensor, plan: ExchangePlan, group=None) -> torch.Tensor:
    """Expert outputs [R, H] back to the ranks their rows came from, in the order they left."""
    if rows.shape[0] != plan.recv_rows:
        raise ValueError("row count does not match the plan's receive size")
    out = torch.empty(sum(plan.send_splits), rows.shape[1], dtype=rows.dtype, device=rows.device)
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=plan.send_splits,
                           input_split_sizes=plan.recv_splits, group=group)
    return out
