"""W4A16 on the tcgen05 tensor cores (weights dequantised into tensor memory): against the mma.sync
kernels of the same library and against the CPU oracle, for decode-size and ragged groups."""
import pytest
import torch

from mini_qwen_b200 import synthetic
from mini_qwen_b200.kernels import moe_permute_plan
from mini_qwen_b200.kernels.moe_permute import gather_rows
from mini_qwen_b200.kernels.w4a16_gemm import (w4a16_grouped_gemm, w4a16_grouped_swiglu, w4a16_tc_gemm,
                                               w4a16_tc_prep, w4a16_tc_swiglu)
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def kperm_index(n):
    """position of natural column c in the shuffled order (0,4,1,5,2,6,3,7 inside every 8)"""
    c = torch.arange(n)
    return (c & ~7) | (((c & 3) << 1) | ((c >> 2) & 1))


def close(got, want):
    """Two kernels of this library on the same inputs: both take fp32 sums, in different orders, of terms far
    larger than the result, so they are compared relative to the result's magnitude.  The comparisons with
    the CPU oracle below use cases.w4_output_bar."""
    scale = max(1.0, float(want.abs().max()))
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-3 * scale)


def test_prep_rows_shuffle_and_sums():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(37, 512, generator=g).to(torch.bfloat16)
    perm = torch.randperm(37 * 2, generator=g).to(torch.int32)
    xp, xs = w4a16_tc_prep(x.to(DEV), perm.to(DEV), 2)
    rows = x[(perm // 2).long()]
    order = torch.tensor([0, 4, 1, 5, 2, 6, 3, 7])
    want = rows.reshape(74, 64, 8)[:, :, order].reshape(74, 512)
    assert torch.equal(xp.cpu(), want)
    sums = rows.float().reshape(74, 4, 128).sum(-1)
    torch.testing.assert_close(xs.cpu()[:, :4], sums, rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("T,H,E,K,I", [(4, 256, 4, 2, 128), (16, 512, 8, 4, 256), (64, 2048, 16, 8, 768),
                                       (300, 512, 4, 2, 256)])
def test_tc_projections_match_mma_sync_kernels_and_oracle(T, H, E, K, I):
    lay = synthetic.w4a16_layer(40 + T, T, H, E, K, I, group=128)
    x = lay.x.to(DEV)
    g = torch.Generator().manual_seed(T)
    ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32).to(DEV)
    perm, inv, off32, _ = moe_permute_plan(ids, E, want_int64_offsets=False)
    gate = tuple(t.to(DEV) for t in (lay.gate.qweight, lay.gate.scales.to(torch.bfloat16), lay.gate.qzeros))
    up = tuple(t.to(DEV) for t in (lay.up.qweight, lay.up.scales.to(torch.bfloat16), lay.up.qzeros))
    down = tuple(t.to(DEV) for t in (lay.down.qweight, lay.down.scales.to(torch.bfloat16), lay.down.qzeros))
    status = torch.zeros(1, dtype=torch.int32, device=DEV)

    xp, xs = w4a16_tc_prep(x, perm, K)
    h_tc = w4a16_tc_swiglu(xp, xs, gate, up, off32, status=status)
    rows = gather_rows(x, perm, K)
    h_ref = w4a16_grouped_swiglu(rows, gate, up, off32)
    pos = kperm_index(I).to(DEV)
    close(h_tc[:, pos], h_ref)

    _, xs2 = w4a16_tc_prep(h_tc, shuffle=False, want_rows=False)
    out_tc = w4a16_tc_gemm(h_tc, xs2, *down, off32, status=status)
    out_ref = w4a16_grouped_gemm(h_tc[:, pos].contiguous(), *down, off32)
    close(out_tc, out_ref)
    assert status.item() == 0

    # against the CPU oracle: all rows, the oracle's own spread under exact sums as the yardstick
    import cases
    sets = tuple((p.qweight, p.scales.to(torch.bfloat16), p.qzeros) for p in (lay.gate, lay.up))
    h32 = cases.w4_grouped_reference(rows.cpu(), sets, off32.cpu(), torch.float32)
    h64 = cases.w4_grouped_reference(rows.cpu(), sets, off32.cpu(), torch.float64)
    cases.w4_output_bar(h_tc[:, pos].cpu(), h32, h64)


@pytest.mark.parametrize("T", [1, 16, 64])
def test_block_on_the_tensor_memory_kernel_matches_reference_outputs(T):
    """The whole W4A16 decode block with ``w4_kernel = "tc"`` against the reference's stored outputs."""
    import cases
    from test_gpu_block import cpu, w4_block
    lay, g = cases.config3(), cases.golden("c3")
    blk = w4_block(lay)
    blk.w4_kernel = "tc"
    x = lay.x[:T].to(DEV)
    out = blk(x)
    ref64 = cases.w4_block_reference(lay, lay.x[:T], lay.router.to(torch.bfloat16), torch.float64)
    cases.w4_output_bar(cpu(out), cases.from_bits(g[f"out_T{T}"], torch.bfloat16), ref64)
    blk.check_status()
