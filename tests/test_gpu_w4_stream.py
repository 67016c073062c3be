"""The TMA-staged W4A16 stream kernel (csrc/w4a16_stream.cu) through the C ABI: plain and prepared
activations, shuffled output, gathered rows, groups of more than 8 rows, empty groups, column counts that
are not a multiple of the panel block, a single linear, int64 offsets.  Results are held to the CPU
oracle with the bar of cases.w4_output_bar (the oracle's own spread under exact sums)."""
import pytest
import torch

import cases
from mini_qwen_b200 import _cabi, synthetic
from mini_qwen_b200.kernels import moe_permute_plan
from mini_qwen_b200.kernels.moe_permute import gather_rows
from mini_qwen_b200.kernels.w4a16_gemm import (w4a16_gemm, w4a16_grouped_gemm, w4a16_grouped_swiglu,
                                               w4a16_stream_gemm, w4a16_stream_swiglu, w4a16_tc_prep)

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def kperm_index(n):
    """position of natural column c in the shuffled order (0,4,1,5,2,6,3,7 inside every 8)"""
    c = torch.arange(n)
    return (c & ~7) | (((c & 3) << 1) | ((c >> 2) & 1))


def dev_set(p):
    return tuple(t.to(DEV) for t in (p.qweight, p.scales.to(torch.bfloat16), p.qzeros))


def cpu_set(p):
    return (p.qweight, p.scales.to(torch.bfloat16), p.qzeros)


def routed(T, E, K, seed, skew=False):
    g = torch.Generator().manual_seed(seed)
    if skew:      # most slots on two experts, several experts empty
        ids = torch.stack([torch.tensor([0, 1] + torch.randperm(E - 2, generator=g)[:K - 2].add(2).tolist())
                           for _ in range(T)])
        ids[:, 2:] = ids[:, 2:] % max(3, E // 2)
        ids = torch.stack([torch.unique(r)[:K] if torch.unique(r).numel() >= K else torch.arange(K) for r in ids])
    else:
        ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)])
    return ids.to(torch.int32).to(DEV)


@pytest.mark.parametrize("T,H,E,K,I,skew", [(1, 256, 4, 2, 128, False), (8, 512, 8, 4, 384, False),
                                            (64, 2048, 16, 8, 768, False), (40, 512, 8, 4, 256, True),
                                            (300, 384, 4, 2, 128, False)])
def test_stream_kernel_gate_up_and_down_match_the_oracle(T, H, E, K, I, skew):
    lay = synthetic.w4a16_layer(70 + T, T, H, E, K, I, group=128)
    x = lay.x.to(DEV)
    perm, inv, off32, _ = moe_permute_plan(routed(T, E, K, T, skew), E, want_int64_offsets=False)
    gate, up, down = dev_set(lay.gate), dev_set(lay.up), dev_set(lay.down)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    rows = gather_rows(x, perm, K)
    off = off32.cpu()

    # CPU: the gate/up result in fp32 sums and in exact sums
    h32 = cases.w4_grouped_reference(rows.cpu(), (cpu_set(lay.gate), cpu_set(lay.up)), off, torch.float32)
    h64 = cases.w4_grouped_reference(rows.cpu(), (cpu_set(lay.gate), cpu_set(lay.up)), off, torch.float64)

    xp, xs = w4a16_tc_prep(x, perm, K)
    xp16, xs16 = w4a16_tc_prep(x, perm, K, f16=True)             # rows scaled by their power of two, fp16
    x16_tok, xs16_tok = w4a16_tc_prep(x, f16=True)               # the same per token, gathered inside the kernel
    pos = kperm_index(I).to(DEV)
    variants = {
        "fp16 rows": w4a16_stream_swiglu(xp16, xs16, gate, up, off32, shuffle_out=False, status=status),
        "fp16 rows, gathered through perm": w4a16_stream_swiglu(x16_tok, xs16_tok, gate, up, off32, shuffle_out=False,
                                                                status=status, perm=perm, top_k=K),
        "prepared, sums given, shuffled out": w4a16_stream_swiglu(xp, xs, gate, up, off32, status=status)[:, pos],
        "prepared, sums given": w4a16_stream_swiglu(xp, xs, gate, up, off32, shuffle_out=False, status=status),
        "prepared, sums by MMA": w4a16_stream_swiglu(xp, None, gate, up, off32, shuffle_out=False, status=status),
        "natural order": w4a16_stream_swiglu(rows, None, gate, up, off32, x_shuffled=False, shuffle_out=False,
                                             status=status),
    }
    for name, h in variants.items():
        try:
            cases.w4_output_bar(h.cpu(), h32, h64)
        except AssertionError as exc:
            raise AssertionError(f"gate/up, {name}: {exc}") from None
    # the same arithmetic in every variant: identical bits
    first = variants["prepared, sums given"]
    assert torch.equal(variants["prepared, sums given, shuffled out"], first)
    assert torch.equal(variants["fp16 rows"], variants["fp16 rows, gathered through perm"])
    # the scaling by a power of two is exact: N(0,1) rows hold no element 2^28 times smaller than their largest,
    # so the fp16 format gives the bf16 format's bits
    assert torch.equal(variants["fp16 rows"], first)
    # the format itself: the stored values times the inverse factor are the bf16 values, the factor puts the row's
    # largest magnitude into [2^14, 2^15)
    unscale = xs16[:, 31:32]
    assert torch.equal((xp16.float() * unscale).to(torch.bfloat16), xp)
    amax = xp16.float().abs().amax(dim=1)
    assert bool(((amax >= 2.0 ** 14) & (amax < 2.0 ** 15)).all())
    torch.testing.assert_close(xs16[:, : H // 128] * unscale, xs[:, : H // 128], rtol=1e-6, atol=0)
    assert status.item() == 0

    # down projection on the gate/up result (natural order, shuffled, shuffled with sums)
    h = first.contiguous()
    o32 = cases.w4_grouped_reference(h.cpu(), (cpu_set(lay.down),), off, torch.float32)
    o64 = cases.w4_grouped_reference(h.cpu(), (cpu_set(lay.down),), off, torch.float64)
    h_shuf = w4a16_stream_swiglu(xp, xs, gate, up, off32, status=status)
    _, hs = w4a16_tc_prep(h_shuf, shuffle=False, want_rows=False)
    for name, o in {
        "natural order": w4a16_stream_gemm(h, None, *down, off32, x_shuffled=False, status=status),
        "shuffled": w4a16_stream_gemm(h_shuf, None, *down, off32, status=status),
        "shuffled, sums given": w4a16_stream_gemm(h_shuf, hs, *down, off32, status=status),
        "cp.async kernel": w4a16_grouped_gemm(h, *down, off32, zero_init=False),
    }.items():
        try:
            cases.w4_output_bar(o.cpu(), o32, o64)
        except AssertionError as exc:
            raise AssertionError(f"down, {name}: {exc}") from None
    assert status.item() == 0


def test_grouped_wrappers_accept_the_int64_offsets_moe_permute_returns():
    lay = synthetic.w4a16_layer(5, 24, 256, 4, 2, 128, group=128)
    x = lay.x.to(DEV)
    perm, inv, off32, off64 = moe_permute_plan(routed(24, 4, 2, 9), 4, want_int64_offsets=True)
    rows = gather_rows(x, perm, 2)
    gate, up, down = dev_set(lay.gate), dev_set(lay.up), dev_set(lay.down)
    h_a, h_b = w4a16_grouped_swiglu(rows, gate, up, off32), w4a16_grouped_swiglu(rows, gate, up, off64)
    assert off64.dtype == torch.int64 and torch.equal(h_a, h_b)
    assert torch.equal(w4a16_grouped_gemm(h_a, *down, off32), w4a16_grouped_gemm(h_a, *down, off64))
    with pytest.raises(AssertionError, match="contiguous"):
        w4a16_grouped_gemm(h_a, down[0].transpose(1, 2), down[1], down[2], off32)


@pytest.mark.parametrize("M,K,N", [(1, 2048, 4096), (4, 2048, 512), (16, 2048, 4096), (13, 1024, 96)])
def test_single_linear_at_the_attention_projection_shapes(M, K, N):
    """w4a16_gemm as the reference's LinearW4A16 would call it for the attention projections of the same model
    (hidden 2048 -> 4096 query / 512 key-value columns, mini_qwen/model/layers/attention.py:136-148)."""
    from oracle import moe_oracle as O
    g = torch.Generator().manual_seed(M + N)
    w = torch.randn(K, N, generator=g) * 0.05
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    qw, sc, qz = O.minmax_quantize(w, 128)
    got = w4a16_gemm(x.to(DEV), qw.contiguous().to(DEV), sc.to(DEV), qz.to(DEV), 128)
    ref = O.w4a16_linear(x, qw, sc, qz, 128)
    torch.testing.assert_close(got.cpu().float(), ref.float(), rtol=cases.RTOL, atol=cases.ATOL)
