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
    uniq = torch.full((T, G), -7, dtype=torch.int32, device=DEV)
    c = _cabi
    c.check(c.load().mq_ep_unique_rows(c.ptr(ids.to(DEV)), T, K, E, G, c.ptr(uniq), c.stream_ptr(DEV)), "unique")
    flags = np.zeros((T, G), dtype=bool)
    dest = ids.numpy() // (E // G)
    for d in range(G):
        flags[:, d] = (dest == d).any(axis=1)
    want = np.where(flags, np.cumsum(flags, axis=0) - 1, -1)
    assert np.array_equal(uniq.cpu().numpy(), want)


@pytest.mark.parametrize("G,T,K,E,H", [(2, 37, 2, 4, 64), (4, 300, 4, 16, 256), (8, 500, 8, 64, 512)])
def test_dispatch_unique_delivers_every_slot(G, T, K, E, H):
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
    recv_ptrs, ridx_ptrs = _ptrs(recv), _ptrs(ridx)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    plans = [moe_permute_plan(ids[r], E, want_int64_offsets=False) for r in range(G)]
    counts = torch.stack([p[2][1:] - p[2][:-1] for p in plans]).contiguous()          # [G, E]
    segs = []
    for r in range(G):
        perm, inv, off32, _ = plans[r]
        send_base = torch.empty(E, dtype=torch.int32, device=DEV)
        seg = torch.empty(E + 1, dtype=torch.int32, device=DEV)
        c.check(lib.mq_ep_plan(c.ptr(counts), G, r, E, c.ptr(send_base), c.ptr(seg), None, 0, None, st), "plan")
        segs.append(seg.cpu())
        uniq = torch.empty(T, G, dtype=torch.int32, device=DEV)
        c.check(lib.mq_ep_unique_rows(c.ptr(ids[r]), T, K, E, G, c.ptr(uniq), st), "unique")
        slot_dst = torch.empty(T * K, dtype=torch.int32, device=DEV)
        c.check(lib.mq_ep_dispatch_unique(c.ptr(xs[r]), c.dtype_code(xs[r]), c.ptr(uniq), c.ptr(perm), c.ptr(off32),
                                          c.ptr(send_base), T, K, H, E, G, r, T, c.ptr(recv_ptrs), c.ptr(ridx_ptrs),
                                          cap, c.ptr(slot_dst), c.ptr(status), st), "dispatch_unique")
    torch.cuda.synchronize()
    assert status.item() == 0
    # receive side of rank d: group (s, j) holds, in sorted order, the rows of rank s's tokens routed to expert d*el+j
    for d in range(G):
        table = ridx[d].cpu()
        buf = recv[d].cpu()
        pos = 0
        for s in range(G):
            perm_s, off_s = plans[s][0].cpu(), plans[s][2].cpu()
            for j in range(el):
                e = d * el + j
                assert int(segs[d][s * el + j]) == pos
                toks = perm_s[int(off_s[e]):int(off_s[e + 1])] // K
                rows = table[pos:pos + toks.numel()].long()
                assert bool(((rows >= s * T) & (rows < (s + 1) * T)).all())
                assert torch.equal(buf[rows], xs[s].cpu()[toks.long()])
                pos += toks.numel()
        assert int(segs[d][-1]) == pos
