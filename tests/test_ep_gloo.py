"""Expert-parallel exchange logic on CPU: world_size-2 (and 4) gloo ranks run the plan / dispatch /
combine functions of mini_qwen_b200.parallel around the oracle's router, permute and expert MLP,
and must reproduce the single-process oracle on the concatenated batch."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, skew):
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for p in (root, os.path.join(root, "mini-qwen-llm_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    from mini_qwen_b200 import parallel, synthetic
    from oracle import moe_oracle as O

    torch.set_num_threads(1)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        T_local, H, E, K, I = 24, 32, 8, 2, 16
        lay = synthetic.dense_layer(11, T_local * world, H, E, K, I, torch.float32)   # same on every rank
        bias = synthetic.zipf_router_bias(3, E, strength=3.0) if skew else None        # leaves experts empty
        el = E // world
        x = lay.x[rank * T_local:(rank + 1) * T_local]

        ids, wts = O.router(x, lay.router, K, bias)
        wts = O.renormalise(wts)
        permuted, off = O.permute(x, ids, E)
        counts = (off[1:] - off[:-1]).to(torch.int32)
        all_counts = parallel.gather_counts(counts)
        assert all_counts.shape == (world, E) and torch.equal(all_counts[rank], counts)
        plan = parallel.make_plan(all_counts, rank)
        assert sum(plan.send_splits) == T_local * K
        assert plan.seg_offsets.numel() == world * el + 1 and int(plan.seg_offsets[-1]) == plan.recv_rows

        recv = parallel.dispatch(permuted, plan)
        seg = plan.seg_offsets.tolist()
        out_rows = torch.zeros_like(recv)
        for g in range(world * el):
            s, t = seg[g], seg[g + 1]
            if t > s:
                e = rank * el + g % el                       # group g -> local expert g % el
                out_rows[s:t] = O.expert_mlp(recv[s:t], lay.gate[e], lay.up[e], lay.down[e])
        back = parallel.combine(out_rows, plan)
        assert back.shape == permuted.shape
        out = O.unpermute(back, wts, ids, T_local)

        ref, ref_ids, _, _ = O.block_forward(lay.x, lay.router, lay.gate, lay.up, lay.down, K, True, bias)
        lo, hi = rank * T_local, (rank + 1) * T_local
        assert torch.equal(ids, ref_ids[lo:hi])              # routing is local and identical
        torch.testing.assert_close(out, ref[lo:hi], rtol=1e-5, atol=1e-6)

        # mismatched sizes are rejected on the host, before any collective
        with pytest.raises(ValueError):
            parallel.dispatch(permuted[:-1], plan)
        with pytest.raises(ValueError):
            parallel.combine(out_rows[:-1] if out_rows.shape[0] else torch.zeros(1, H), plan)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,skew", [(2, False), (2, True), (4, True)])
def test_expert_parallel_exchange_matches_oracle(world, skew):
    mp.spawn(_worker, args=(world, _free_port(), skew), nprocs=world, join=True)


def test_plan_rejects_uneven_sharding():
    from mini_qwen_b200 import parallel
    with pytest.raises(ValueError):
        parallel.make_plan(torch.zeros(3, 8, dtype=torch.int32), 0)
