"""The expert-parallel plan/dispatch kernels driven on ONE GPU: the G ranks are emulated by G sets of
buffers on the same device and the kernels of each rank are launched one after the other (none of
them waits on another rank), then the receive side is checked against a direct computation."""
import numpy as np
import pytest
import torch

from mini_qwen_b200 import _cabi
from mini_qwen_b200.kernels import moe_permute_plan

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def _ptrs(tensors):
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device=DEV)


@pytest.mark.parametrize("T,K,E,G", [(1, 2, 4, 2), (300, 4, 16, 4), (2500, 8, 128, 8), (1024, 8, 128, 2)])
def test_unique_rows_index(T, K, E, G):
    g = torch.Generator().manual_seed(T + G)
    ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32)
    uniq = torch.full((G, T), -7, dtype=torch.int32, device=DEV)
    c = _cabi
    c.check(c.load().mq_ep_unique_rows(c.ptr(ids.to(DEV)), T, K, E, G, c.ptr(uniq), c.stream_ptr(DEV)), "unique")
    flags = np.zeros((T, G), dtype=bool)
    dest = ids.numpy() // (E // G)
    for d in range(G):
        flags[:, d] = (dest == d).any(axis=1)
    want = np.where(flags, np.cumsum(flags, axis=0) - 1, -1)
    assert np.array_equal(uniq.cpu().numpy().T, want)


@pytest.mark.parametrize("unique", [True, False])
@pytest.mark.parametrize("G,T,K,E,H", [(2, 37, 2, 4, 64), (4, 300, 4, 16, 256), (8, 500, 8, 64, 512)])
def test_dispatch_delivers_every_slot(G, T, K, E, H, unique):
    c = _cabi
    lib = c.load()
    st = c.stream_ptr(DEV)
    el = E // G
    cap = G * T * K
    g = torch.Generator().manual_seed(G * 100 + T)
    xs = [torch.randn(T, H, generator=g).to(torch.bfloat16).to(DEV) for _ in range(G)]
    ids = [torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32).to(DEV)
           for _ in range(G)]
    recv = [torch.zeros(cap, H, dtype=torch.bfloat16, device=DEV) for _ in range(G)]
    ridx = [torch.full((cap,), -1, dtype=torch.int32, device=DEV) for _ in range(G)]
    home = [torch.full((cap,), -1, dtype=torch.int32, device=DEV) for _ in range(G)]
    recv_ptrs, ridx_ptrs, home_ptrs = _ptrs(recv), _ptrs(ridx), _ptrs(home)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    plans = [moe_permute_plan(ids[r], E, want_int64_offsets=False) for r in range(G)]
    counts = torch.stack([p[2][1:] - p[2][:-1] for p in plans]).contiguous()          # [G, E]
    segs = []
    for r in range(G):
        perm, inv, off32, _ = plans[r]
        send_base = torch.empty(E, dtype=torch.int32, device=DEV)
        seg = torch.empty(el + 1, dtype=torch.int32, device=DEV)
        c.check(lib.mq_ep_plan(c.ptr(counts), G, r, E, c.ptr(send_base), c.ptr(seg), st), "plan")
        segs.append(seg.cpu())
        slot_dst = torch.empty(T * K, dtype=torch.int32, device=DEV)
        if unique:
            uniq = torch.empty(G, T, dtype=torch.int32, device=DEV)
            c.check(lib.mq_ep_unique_rows(c.ptr(ids[r]), T, K, E, G, c.ptr(uniq), st), "unique")
            c.check(lib.mq_ep_dispatch_unique(c.ptr(xs[r]), c.dtype_code(xs[r]), c.ptr(uniq), c.ptr(perm),
                                              c.ptr(off32), c.ptr(send_base), T, K, H, E, G, r, T, c.ptr(recv_ptrs),
                                              c.ptr(ridx_ptrs), c.ptr(home_ptrs), cap, c.ptr(slot_dst),
                                              c.ptr(status), st), "dispatch_unique")
        else:
            c.check(lib.mq_ep_dispatch(c.ptr(xs[r]), c.dtype_code(xs[r]), c.ptr(perm), c.ptr(off32), c.ptr(send_base),
                                       T * K, K, H, E, G, r, c.ptr(recv_ptrs), c.ptr(home_ptrs), cap, c.ptr(slot_dst),
                                       c.ptr(status), st), "dispatch")
        # slot_dst names the owner and the slot of every sorted position
        sd = slot_dst.cpu().long()
        owner = torch.repeat_interleave(torch.arange(E), (off32[1:] - off32[:-1]).cpu().long()) // el
        assert torch.equal(sd // cap, owner)
    torch.cuda.synchronize()
    assert status.item() == 0
    # receive side of rank d: expert j's group holds rank 0's slots, then rank 1's, ..., each in sorted order
    for d in range(G):
        table, homes, buf = ridx[d].cpu(), home[d].cpu(), recv[d].cpu()
        pos = 0
        for j in range(el):
            e = d * el + j
            assert int(segs[d][j]) == pos
            for s in range(G):
                perm_s, off_s = plans[s][0].cpu(), plans[s][2].cpu()
                lo, hi = int(off_s[e]), int(off_s[e + 1])
                toks = (perm_s[lo:hi] // K).long()
                n = hi - lo
                want_home = (s << 26) | torch.arange(lo, hi)
                assert torch.equal(homes[pos:pos + n].long(), want_home)
                if unique:
                    rows = table[pos:pos + n].long()
                    assert bool(((rows >= s * T) & (rows < (s + 1) * T)).all())
                    assert torch.equal(buf[rows], xs[s].cpu()[toks])
                else:
                    assert torch.equal(buf[pos:pos + n], xs[s].cpu()[toks])
                pos += n
        assert int(segs[d][-1]) == pos


def test_exchange_plan_single_rank_matches_plan():
    """G = 1: the fused counts/barrier/plan launch meets only itself and must give the plain plan."""
    c = _cabi
    lib = c.load()
    st = c.stream_ptr(DEV)
    E, T, K = 32, 200, 4
    g = torch.Generator().manual_seed(5)
    ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32).to(DEV)
    _, _, off32, _ = moe_permute_plan(ids, E, want_int64_offsets=False)
    counts = torch.zeros(E, dtype=torch.int32, device=DEV)
    sig = torch.zeros(32, dtype=torch.int32, device=DEV)
    epoch = torch.zeros(1, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    sb, seg = (torch.empty(E, dtype=torch.int32, device=DEV), torch.empty(E + 1, dtype=torch.int32, device=DEV))
    counts_ptrs, sig_ptrs = _ptrs([counts]), _ptrs([sig])  # kept alive: the launches read them asynchronously
    for _ in range(2):                                    # the epoch advances; a second call must pass as well
        c.check(lib.mq_ep_exchange_plan(c.ptr(off32), E, 1, 0, c.ptr(counts_ptrs), c.ptr(sig_ptrs),
                                        c.ptr(epoch), c.ptr(sb), c.ptr(seg), 0, c.ptr(status), st), "exchange_plan")
    assert status.item() == 0 and epoch.item() == 2
    assert torch.equal(counts, off32[1:] - off32[:-1])
    assert torch.equal(seg, off32) and torch.equal(sb, off32[:-1])


def test_bounded_waits_run_out_and_leave_a_plan_that_moves_nothing():
    """The rank barrier's wait is bounded.  Two "ranks" are emulated with two signal arrays and two counts
    tables on one device; rank 1 never launches anything, so rank 0's poll of its slot cannot succeed.
    With a budget of 1024 polls the kernels return, MQ_DEV_WAIT_EXPIRED is set, the plan written is the
    one that sends and computes nothing, a dispatch driven by that plan writes no row, the stream stays
    usable, and once rank 1 does signal, the same barrier passes."""
    c = _cabi
    lib = c.load()
    st = c.stream_ptr(DEV)
    E, T, K, H, G = 8, 40, 2, 64, 2
    g = torch.Generator().manual_seed(11)
    ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32).to(DEV)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(DEV)
    perm, inv, off32, _ = moe_permute_plan(ids, E, want_int64_offsets=False)
    counts = [torch.full((G * E,), 12345, dtype=torch.int32, device=DEV) for _ in range(G)]   # stale garbage
    sig = [torch.zeros(32, dtype=torch.int32, device=DEV) for _ in range(G)]
    counts_ptrs, sig_ptrs = _ptrs(counts), _ptrs(sig)
    epoch = torch.zeros(1, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    sb = torch.full((E,), -5, dtype=torch.int32, device=DEV)
    seg = torch.full((E // G + 1,), -5, dtype=torch.int32, device=DEV)

    # 1. plain barrier: rank 1's slot of rank 0's array stays 0 < epoch 1
    c.check(lib.mq_ep_barrier(c.ptr(sig_ptrs), c.ptr(epoch), G, 0, 1024, c.ptr(status), st), "barrier")
    torch.cuda.synchronize()
    assert status.item() & 1 and epoch.item() == 1
    assert sig[1][0].item() == 1                      # rank 0 did signal its peer before it waited

    # 2. fused counts + barrier + plan: expiry leaves the safe plan, not one built from the stale counts
    status.zero_()
    c.check(lib.mq_ep_exchange_plan(c.ptr(off32), E, G, 0, c.ptr(counts_ptrs), c.ptr(sig_ptrs), c.ptr(epoch),
                                    c.ptr(sb), c.ptr(seg), 1024, c.ptr(status), st), "exchange_plan")
    torch.cuda.synchronize()
    assert status.item() & 1 and epoch.item() == 2
    assert bool((sb == 0x3FFFFFFF).all()) and bool((seg == 0).all())

    # 3. a dispatch on that plan drops every row (flags the overflow bit) and touches no buffer
    cap = G * T * K
    recv = [torch.zeros(cap, H, dtype=torch.bfloat16, device=DEV) for _ in range(G)]
    home = [torch.full((cap,), -1, dtype=torch.int32, device=DEV) for _ in range(G)]
    recv_ptrs, home_ptrs = _ptrs(recv), _ptrs(home)
    slot_dst = torch.zeros(T * K, dtype=torch.int32, device=DEV)
    c.check(lib.mq_ep_dispatch(c.ptr(x), c.dtype_code(x), c.ptr(perm), c.ptr(off32), c.ptr(sb), T * K, K, H, E, G, 0,
                               c.ptr(recv_ptrs), c.ptr(home_ptrs), cap, c.ptr(slot_dst), c.ptr(status), st), "dispatch")
    torch.cuda.synchronize()
    assert status.item() & 2 and bool((slot_dst == -1).all())
    assert all(not bool(r.any()) for r in recv) and all(bool((h == -1).all()) for h in home)

    # 4. the stream still works, and with rank 1 present (its epoch written into rank 0's array, as its own
    # barrier kernel would) the next barrier passes without touching the status word
    status.zero_()
    sig[0][1] = 3
    c.check(lib.mq_ep_barrier(c.ptr(sig_ptrs), c.ptr(epoch), G, 0, 1024, c.ptr(status), st), "barrier")
    torch.cuda.synchronize()
    assert status.item() == 0 and epoch.item() == 3


def test_stack_tensors_concatenates_device_tensors():
    """mq_stack_tensors: the expert-major stack a host without a tensor library builds from per-expert tensors."""
    c = _cabi
    lib = c.load()
    st = c.stream_ptr(DEV)
    g = torch.Generator().manual_seed(3)
    for shape, dtype in (((96, 64), torch.bfloat16), ((33, 5), torch.int32), ((7,), torch.uint8)):
        parts = [torch.randint(0, 127, shape, generator=g).to(dtype).to(DEV) for _ in range(5)]
        nbytes = parts[0].numel() * parts[0].element_size()
        out = torch.empty((5,) + shape, dtype=dtype, device=DEV)
        ptrs = _ptrs(parts)
        aligned = int(all(p.data_ptr() % 16 == 0 for p in parts))
        c.check(lib.mq_stack_tensors(c.ptr(ptrs), 5, nbytes, aligned, c.ptr(out), st), "stack")
        torch.cuda.synchronize()
        assert torch.equal(out, torch.stack(parts))
