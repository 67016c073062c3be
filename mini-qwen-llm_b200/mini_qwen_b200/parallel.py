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


class PeerExchange:
    """Buffers and kernels for the exchange over peer memory (NVLink loads/stores), one per block.

    Every rank owns a receive buffer and an expert-output buffer of ``cap_rows`` rows that all ranks
    of the group can address (torch symmetric memory supplies the allocation and the peer
    addresses; the data path is this library's kernels).  ``cap_rows`` defaults to the worst case,
    every slot of every rank landing on one GPU, so no routing can overflow it.

    Received slots are ordered by local expert and, inside an expert, by source rank.

    Ordering between ranks is three stream-ordered barriers per layer call: after the counts have
    been shared, after the dispatch kernels and after the down projection.  The barrier is a
    one-warp kernel that writes an epoch into every peer's signal array and polls its own, with a
    bounded number of polls (an expired wait sets a status bit; it never hangs).  The ranks must
    therefore enter a layer call within the poll budget of one another (one to two seconds), and
    ``check_status()`` has to be called after a step before its output is trusted: an expired barrier
    leaves a plan that moves and computes nothing, so the output of that call is meaningless.
    """

    def __init__(self, group, device, cap_rows: int, hidden: int, dtype: torch.dtype):
        import os

        # every byte moves in this library's kernels with plain peer loads and stores: the buffers need no
        # NVLink multicast binding (a rank that dies while bound to one disturbs its peers' GPUs)
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        from . import _cabi
        self._cabi = _cabi
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.cap_rows, self.hidden, self.dtype = cap_rows, hidden, dtype
        self.max_polls = 0             # poll budget of the rank barriers (0 = the library's default, 1-2 s)
        if self.world * cap_rows >= 2 ** 31:
            raise ValueError("expert-parallel buffer too large for 32-bit slot addresses")
        self.recv = symm_mem.empty(cap_rows * hidden, dtype=dtype, device=device)
        self.y = symm_mem.empty(cap_rows * hidden, dtype=dtype, device=device)
        h_recv = symm_mem.rendezvous(self.recv, group)
        h_y = symm_mem.rendezvous(self.y, group)
        self._handles = (h_recv, h_y)
        self.recv_ptrs = torch.tensor(list(h_recv.buffer_ptrs), dtype=torch.int64, device=device)
        self.y_ptrs = torch.tensor(list(h_y.buffer_ptrs), dtype=torch.int64, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self._done = None              # counter of the partial-sum kernel (decode by replication)
        self._tab = None               # symmetric int32 [2, cap_rows]: slot table and home table
        self._counts = None            # symmetric [G, E] int32, created on first use (E is not known here)
        self._sig = symm_mem.empty(max(self.world, 32), dtype=torch.int32, device=device)
        self._sig.zero_()
        h_sig = symm_mem.rendezvous(self._sig, group)
        self.sig_ptrs = torch.tensor(list(h_sig.buffer_ptrs), dtype=torch.int64, device=device)
        self._epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self._symm = symm_mem
        self._handles += (h_sig,)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)      # every rank's signal array is zeroed before anyone signals

    def recv_rows(self) -> torch.Tensor:
        return self.recv.view(self.cap_rows, self.hidden)

    def y_rows(self) -> torch.Tensor:
        return self.y.view(self.cap_rows, self.hidden)

    def rank_barrier(self) -> None:
        """Stream-ordered barrier across the group: kernels launched after it start once every rank's
        kernels launched before it have finished."""
        c = self._cabi
        dev = self.status.device
        rc = c.load().mq_ep_barrier(c.ptr(self.sig_ptrs), c.ptr(self._epoch), self.world, self.rank, self.max_polls,
                                    c.ptr(self.status), c.stream_ptr(dev))
        c.check(rc, "mq_ep_barrier")
        c.count_launches(1)

    def share_counts(self, off32: torch.Tensor) -> torch.Tensor:
        """All-gather of the per-expert counts by peer stores; returns this rank's [G, E] table, valid
        after the next rank_barrier()."""
        E = off32.numel() - 1
        dev = off32.device
        self._counts_table(E, dev)
        c = self._cabi
        rc = c.load().mq_ep_share_counts(c.ptr(off32), E, self.world, self.rank, c.ptr(self.counts_ptrs),
                                         c.stream_ptr(dev))
        c.check(rc, "mq_ep_share_counts")
        c.count_launches(1)
        return self._counts.view(self.world, E)

    def _counts_table(self, E: int, dev) -> None:
        if self._counts is None or self._counts.numel() != self.world * E:
            self._counts = self._symm.empty(self.world * E, dtype=torch.int32, device=dev)
            self._counts.zero_()       # a row a late rank never writes then reads as "no slots", not as garbage
            h = self._symm.rendezvous(self._counts, self.group)
            self._handles += (h,)
            self.counts_ptrs = torch.tensor(list(h.buffer_ptrs), dtype=torch.int64, device=dev)
            torch.cuda.synchronize(dev)
            dist.barrier(group=self.group)   # every rank's table is zeroed before anyone writes into it

    def exchange_plan(self, off32: torch.Tensor):
        """``share_counts``, ``rank_barrier`` and ``plan`` in one launch: (send_base, seg_offsets)."""
        E = off32.numel() - 1
        dev = off32.device
        self._counts_table(E, dev)
        send_base = torch.empty(E, dtype=torch.int32, device=dev)
        seg = torch.empty(E // self.world + 1, dtype=torch.int32, device=dev)
        c = self._cabi
        rc = c.load().mq_ep_exchange_plan(c.ptr(off32), E, self.world, self.rank, c.ptr(self.counts_ptrs),
                                          c.ptr(self.sig_ptrs), c.ptr(self._epoch), c.ptr(send_base), c.ptr(seg),
                                          self.max_polls, c.ptr(self.status), c.stream_ptr(dev))
        c.check(rc, "mq_ep_exchange_plan")
        c.count_launches(1)
        return send_base, seg

    def plan(self, all_counts: torch.Tensor):
        """Device-side plan (no host sync): (send_base int32 [E], seg_offsets int32 [E/G + 1])."""
        G, E = all_counts.shape
        dev = all_counts.device
        send_base = torch.empty(E, dtype=torch.int32, device=dev)
        seg = torch.empty(E // G + 1, dtype=torch.int32, device=dev)
        c = self._cabi
        rc = c.load().mq_ep_plan(c.ptr(all_counts), G, self.rank, E, c.ptr(send_base), c.ptr(seg), c.stream_ptr(dev))
        c.check(rc, "mq_ep_plan")
        c.count_launches(1)
        return send_base, seg

    def dispatch(self, x: torch.Tensor, perm, off32, send_base, top_k: int, num_experts: int) -> torch.Tensor:
        """Fused permute + dispatch, one row per slot; returns slot_dst int32 [S] (owner * cap_rows + slot).
        Also fills the owners' home tables (where each slot's output row goes back to)."""
        c = self._cabi
        S = perm.numel()
        self._tables()
        slot_dst = torch.empty(S, dtype=torch.int32, device=x.device)
        rc = c.load().mq_ep_dispatch(c.ptr(x), c.dtype_code(x), c.ptr(perm), c.ptr(off32), c.ptr(send_base), S, top_k,
                                     x.shape[1], num_experts, self.world, self.rank, c.ptr(self.recv_ptrs),
                                     c.ptr(self.home_ptrs), self.cap_rows, c.ptr(slot_dst), c.ptr(self.status),
                                     c.stream_ptr(x.device))
        c.check(rc, "mq_ep_dispatch")
        c.count_launches(1 if S else 0)
        return slot_dst

    def _tables(self) -> None:
        """Symmetric int32 [2, cap_rows], created on first use: row 0 the slot table (for every received
        slot, the row of the receive buffer that holds its token; written by ``dispatch_unique``), row 1
        the home table (source rank << 26 | position in the source's sorted order)."""
        if self._tab is None:
            dev = self.status.device
            self._tab = self._symm.empty(2 * self.cap_rows, dtype=torch.int32, device=dev)
            self._tab.zero_()
            h = self._symm.rendezvous(self._tab, self.group)
            self._handles += (h,)
            ptrs = list(h.buffer_ptrs)
            self.ridx_ptrs = torch.tensor(ptrs, dtype=torch.int64, device=dev)
            self.home_ptrs = torch.tensor([q + 4 * self.cap_rows for q in ptrs], dtype=torch.int64, device=dev)
            torch.cuda.synchronize(dev)
            dist.barrier(group=self.group)

    def slot_table(self) -> torch.Tensor:
        self._tables()
        return self._tab[:self.cap_rows]

    def home_table(self) -> torch.Tensor:
        self._tables()
        return self._tab[self.cap_rows:]

    def dispatch_unique(self, x: torch.Tensor, topk_ids32, perm, off32, send_base, top_k: int, num_experts: int,
                        src_stride: int) -> torch.Tensor:
        """Dispatch that sends a token row once per destination rank; returns slot_dst as ``dispatch`` does.
        The receivers read their rows through ``slot_table()``."""
        c = self._cabi
        T = x.shape[0]
        self._tables()
        uniq = torch.empty(self.world, T, dtype=torch.int32, device=x.device)
        rc = c.load().mq_ep_unique_rows(c.ptr(topk_ids32), T, top_k, num_experts, self.world, c.ptr(uniq),
                                        c.stream_ptr(x.device))
        c.check(rc, "mq_ep_unique_rows")
        slot_dst = torch.empty(T * top_k, dtype=torch.int32, device=x.device)
        rc = c.load().mq_ep_dispatch_unique(c.ptr(x), c.dtype_code(x), c.ptr(uniq), c.ptr(perm), c.ptr(off32),
                                            c.ptr(send_base), T, top_k, x.shape[1], num_experts, self.world, self.rank,
                                            src_stride, c.ptr(self.recv_ptrs), c.ptr(self.ridx_ptrs),
                                            c.ptr(self.home_ptrs), self.cap_rows, c.ptr(slot_dst), c.ptr(self.status), c.stream_ptr(x.device))
        c.check(rc, "mq_ep_dispatch_unique")
        c.count_launches(2 if T else 0)
        return slot_dst

    def combine(self, weights, inv, slot_dst, num_tokens: int, top_k: int, residual=None) -> torch.Tensor:
        """Fused combine + unpermute from the owners' output buffers (plus the layer's residual add, if given)."""
        c = self._cabi
        out = torch.empty(num_tokens, self.hidden, dtype=self.dtype, device=weights.device)
        if residual is not None:
            assert residual.shape == out.shape and residual.dtype == out.dtype and residual.is_contiguous()
        rc = c.load().mq_ep_combine(c.ptr(self.y_ptrs), c.dtype_code(out), c.ptr(weights), c.ptr(inv), c.ptr(slot_dst),
                                    c.ptr(residual), num_tokens, top_k, self.hidden, self.cap_rows, c.ptr(out),
                                    c.stream_ptr(weights.device))
        c.check(rc, "mq_ep_combine")
        c.count_launches(1 if num_tokens else 0)
        return out

    # ---- decode batches by replication: every rank holds all tokens, runs its own experts, sends partial sums
    def gather_tokens(self, x: torch.Tensor) -> torch.Tensor:
        """This rank's rows into every peer's token buffer, then the rank barrier; returns all tokens of the step,
        [G*T, H] in rank order (a view of the receive buffer).  Every rank must pass the same number of rows."""
        T, H = x.shape
        if self.world * T > self.cap_rows or H != self.hidden or x.dtype != self.dtype:
            raise ValueError("token buffer too small or of another shape / dtype")
        c = self._cabi
        rc = c.load().mq_ep_gather_tokens(c.ptr(x), c.dtype_code(x), T, H, self.world, self.rank, c.ptr(self.recv_ptrs),
                                          c.ptr(self.sig_ptrs), c.ptr(self._epoch), self.max_polls, c.ptr(self.status),
                                          c.stream_ptr(x.device))
        c.check(rc, "mq_ep_gather_tokens")
        c.count_launches(1)
        return self.recv.view(self.cap_rows, self.hidden)[: self.world * T]

    def send_partials(self, rows, weights, ids32, inv, tokens_per_rank: int, top_k: int, experts_per_rank: int) -> None:
        """Every token's partial weighted sum over this rank's slots goes, in fp32, to the rank that owns the
        token (into its expert-output buffer, read as fp32); then the rank barrier."""
        T, G = tokens_per_rank, self.world
        if G * T * self.hidden * 4 > self.cap_rows * self.hidden * self.y.element_size():
            raise ValueError("partial-sum buffer too small")
        if self._done is None:
            self._done = torch.zeros(1, dtype=torch.int32, device=rows.device)
        c = self._cabi
        rc = c.load().mq_ep_send_partials(c.ptr(rows), c.dtype_code(rows), c.ptr(weights), c.ptr(ids32), c.ptr(inv),
                                          G * T, top_k, self.hidden, T, G, self.rank, experts_per_rank,
                                          c.ptr(self.y_ptrs), c.ptr(self._done), c.ptr(self.sig_ptrs), c.ptr(self._epoch),
                                          self.max_polls, c.ptr(self.status), c.stream_ptr(rows.device))
        c.check(rc, "mq_ep_send_partials")
        c.count_launches(1)

    def sum_partials(self, tokens_per_rank: int, residual=None) -> torch.Tensor:
        """This rank's tokens: the G partial sums added in rank order, cast (and the layer's residual added)."""
        T = tokens_per_rank
        out = torch.empty(T, self.hidden, dtype=self.dtype, device=self.y.device)
        c = self._cabi
        rc = c.load().mq_ep_sum_partials(c.ptr(self.y), c.dtype_code(out), c.ptr(residual), T, self.hidden, self.world,
                                         c.ptr(out), c.stream_ptr(out.device))
        c.check(rc, "mq_ep_sum_partials")
        c.count_launches(1)
        return out

    def check_status(self) -> None:
        """Raises if a receive buffer overflowed (synchronises)."""
        bits = int(self.status.item())
        if bits & 2:
            raise RuntimeError("expert-parallel receive buffer overflowed; construct the block with a larger "
                               "ep_max_tokens / capacity")
        if bits & 1:
            raise RuntimeError("an expert-parallel barrier timed out: a rank of the group did not arrive")
