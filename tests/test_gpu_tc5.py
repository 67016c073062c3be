"""GPU parity of the tcgen05/TMEM grouped GEMM (bf16, N % 128 == 0, K % 64 == 0) against the CPU
oracle, from a single tile up to the benchmark shapes; the device status word must stay 0."""
import pytest
import torch

from mini_qwen_b200.kernels import moe_grouped_gemm, moe_grouped_swiglu
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def offsets_from_counts(counts):
    off = torch.zeros(len(counts) + 1, dtype=torch.int64)
    off[1:] = torch.cumsum(torch.tensor(counts), 0)
    return off


CASES = [
    ([128], 128, 64),                 # one tile, one k block
    ([128], 256, 256),                # one tile, 4 k blocks (one trip round the ring)
    ([100], 128, 512),                # partial tile, ring wraps
    ([130, 0, 5, 300], 256, 192),     # tiles straddling expert ends, an empty expert
    ([1, 1, 1, 1, 1, 1, 1, 1], 512, 128),
    ([257] * 16, 2048, 768),          # down-projection shape
    ([700, 13, 0, 0, 1500, 128, 127, 129], 768, 2048),
]


@pytest.mark.parametrize("counts,N,Kd", CASES)
def test_tc5_grouped_gemm(counts, N, Kd):
    E, S = len(counts), sum(counts)
    g = torch.Generator().manual_seed(S + N + Kd)
    a = torch.randn(S, Kd, generator=g).to(torch.bfloat16)
    w = (torch.randn(E, N, Kd, generator=g) * 0.05).to(torch.bfloat16)
    off = offsets_from_counts(counts)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = moe_grouped_gemm(a.to(DEV), w.to(DEV), off.to(DEV), status=status)
    assert status.item() == 0, "a bounded wait ran out inside the kernel"
    ref = O.grouped_gemm(a, w, off)
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=2e-2, atol=2e-3)
    # fp32 accumulation of exact bf16 products: only rounding-boundary flips may differ
    assert (out.cpu() != ref).float().mean() < 0.01


@pytest.mark.parametrize("counts,I,H", [([128], 128, 64), ([90, 0, 200], 256, 256), ([300] * 8, 768, 2048)])
def test_tc5_grouped_swiglu(counts, I, H):
    E, S = len(counts), sum(counts)
    g = torch.Generator().manual_seed(S + I + H)
    a = torch.randn(S, H, generator=g).to(torch.bfloat16)
    wg = (torch.randn(E, I, H, generator=g) * 0.05).to(torch.bfloat16)
    wu = (torch.randn(E, I, H, generator=g) * 0.05).to(torch.bfloat16)
    off = offsets_from_counts(counts)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    h = moe_grouped_swiglu(a.to(DEV), torch.cat([wg, wu], 1).to(DEV), off.to(torch.int32).to(DEV), status=status)
    assert status.item() == 0
    ref = torch.zeros(S, I, dtype=torch.bfloat16)
    for e in range(E):
        s, t = int(off[e]), int(off[e + 1])
        if t > s:
            ref[s:t] = torch.nn.functional.silu(a[s:t] @ wg[e].T) * (a[s:t] @ wu[e].T)
    torch.testing.assert_close(h.cpu().float(), ref.float(), rtol=2e-2, atol=2e-3)


def test_tc5_rows_outside_experts_untouched():
    # offsets that do not start at 0 / end at S: rows outside stay zero
    a = torch.randn(300, 64, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    w = torch.randn(2, 128, 64, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    off = torch.tensor([10, 150, 280])
    out = moe_grouped_gemm(a.to(DEV), w.to(DEV), off.to(DEV)).cpu()
    assert float(out[:10].abs().max()) == 0 and float(out[280:].abs().max()) == 0
    ref = torch.zeros(300, 128, dtype=torch.bfloat16)
    ref[10:150] = (a[10:150].float() @ w[0].float().T).to(torch.bfloat16)
    ref[150:280] = (a[150:280].float() @ w[1].float().T).to(torch.bfloat16)
    torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=2e-3)


@pytest.mark.parametrize("T,K,E,I,H", [(64, 2, 4, 128, 64), (300, 4, 8, 256, 256), (1024, 8, 16, 768, 2048)])
def test_tc5_swiglu_with_fused_gather(T, K, E, I, H):
    """The gather-fused gate/up kernel (rows fetched through the permutation by producer warps) must
    give the very bits of the two-step path (row gather, then the same kernel on contiguous rows)."""
    from mini_qwen_b200.kernels import moe_grouped_swiglu_gather, moe_permute_plan
    from mini_qwen_b200.kernels.moe_permute import gather_rows
    g = torch.Generator().manual_seed(T + I)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(DEV)
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32).to(DEV)
    perm, inv, off32, _ = moe_permute_plan(ids, E, want_int64_offsets=False)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    fused = moe_grouped_swiglu_gather(x, perm, K, w13, off32, status=status)
    assert status.item() == 0
    two_step = moe_grouped_swiglu(gather_rows(x, perm, K), w13, off32)
    assert torch.equal(fused, two_step)


@pytest.mark.parametrize("counts,N,Kd", [([5, 0, 130, 17], 128, 64), ([260, 31, 0, 300, 1, 90], 256, 512),
                                         ([700, 3, 256, 255, 257, 0, 16, 48], 2048, 768)])
def test_tc5_scatter_gemm_writes_each_row_at_its_own_address(counts, N, Kd):
    """Per-row destinations: every output row lands at the row its code names, in one of three buffers,
    with the bits of the plain call; rows no code names stay untouched."""
    from mini_qwen_b200.kernels.moe_grouped_gemm import moe_grouped_gemm_scatter
    E = len(counts)
    S = sum(counts)
    g = torch.Generator().manual_seed(S + N)
    a = torch.randn(S, Kd, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(E, N, Kd, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    off = offsets_from_counts(counts).to(torch.int32).to(DEV)
    plain = moe_grouped_gemm(a, w, off)
    rows_per_buf = S + 3
    bufs = [torch.full((rows_per_buf, N), 7.0, dtype=torch.bfloat16, device=DEV) for _ in range(3)]
    bases = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=DEV)
    which = torch.randint(0, 3, (S,), generator=g)
    place = torch.randperm(rows_per_buf, generator=g)[:S]            # distinct rows, so no two codes collide
    code = ((which << 26) | place).to(torch.int32).to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    moe_grouped_gemm_scatter(a, w, off, code, bases, status=status)
    assert status.item() == 0
    got = torch.stack([bufs[int(b)][int(r)] for b, r in zip(which, place)])
    assert torch.equal(got, plain)
    written = sum(int((b != 7.0).any(dim=1).sum()) for b in bufs)
    assert written <= S                                               # nothing outside the named rows
