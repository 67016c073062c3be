"""GPU parity tests, kernel by kernel, through the C ABI (the Python wrappers are ctypes calls
into libmqmoe.so).  Checker: the CPU oracle on the same seeded inputs, and the stored outputs of
the reference (tests/golden).  Integer results must be bit-exact; floating results within the
tolerance written next to each comparison."""
import numpy as np
import pytest
import torch

import cases
from mini_qwen_b200.kernels import (moe_grouped_gemm, moe_grouped_swiglu, moe_permute, moe_permute_plan,
                                    moe_router, moe_unpermute, w4a16_gemm, w4a16_grouped_gemm,
                                    w4a16_grouped_swiglu)
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def cpu(t):
    return t.detach().cpu()


# ------------------------------------------------------------------------------------------ router
def check_router(x, w, K, bias=None, golden_ids=None, renorm=False):
    ids, wts = moe_router(x.to(DEV), w.to(DEV), K, bias=None if bias is None else bias.to(DEV), renormalize=renorm)
    assert ids.dtype == torch.int64 and wts.dtype == torch.float32 and ids.shape == (x.shape[0], K)
    ref_ids, ref_w = O.router(x, w, K, bias)
    if renorm:
        ref_w = O.renormalise(ref_w)
    assert torch.equal(cpu(ids), ref_ids), "expert ids differ from the fp32 oracle"
    if golden_ids is not None:
        assert torch.equal(cpu(ids), golden_ids.to(torch.int64)), "expert ids differ from the reference's"
    # fp32 scores: summation order and expf differ by a few ulp
    torch.testing.assert_close(cpu(wts), ref_w, rtol=2e-5, atol=1e-7)
    return ids, wts


@pytest.mark.parametrize("i", range(len(cases.KERNEL_SHAPES)))
def test_router_reference_shapes(i):
    T, E, K, H, D = cases.KERNEL_SHAPES[i]
    hidden, router_w = cases.kernel_router_inputs(T, E, K, H)
    check_router(hidden, router_w, K, golden_ids=torch.from_numpy(cases.golden("kernel_cases")[f"router_ids_{i}"]))


@pytest.mark.parametrize("i", range(len(cases.SCRIPT_CASES)))
def test_router_script_cases(i):
    c = cases.SCRIPT_CASES[i]
    x, gate_w, *_ = cases.script_case_inputs(c)
    check_router(x, gate_w, c["K"], golden_ids=torch.from_numpy(cases.golden("script_cases")[f"ids_{i}"]),
                 renorm=False)


def test_router_config1_fp32():
    lay = cases.config1()
    check_router(lay.x, lay.router, lay.top_k, golden_ids=torch.from_numpy(cases.golden("c1")["ids"]))


def test_router_config2_prefill_bit_exact_ids():
    lay = cases.config2()
    check_router(lay.x, lay.router, lay.top_k, golden_ids=torch.from_numpy(cases.golden("c2")["ids"]))


@pytest.mark.parametrize("T", cases.C3_TS)
def test_router_config3_decode(T):
    lay = cases.config3()
    g = cases.golden("c3")
    check_router(lay.x[:T], lay.router.to(torch.bfloat16), lay.top_k, golden_ids=torch.from_numpy(g[f"ids_T{T}"]))
    # fp16 router weights with bf16 activations (the checkpoint's own dtype)
    check_router(lay.x[:T], lay.router, lay.top_k)


def test_router_config4_skewed_bias():
    lay = cases.config4()
    check_router(lay.x, lay.router, lay.top_k, bias=cases.config4_bias(),
                 golden_ids=torch.from_numpy(cases.golden("c4")["ids"]))


def test_router_ties_go_to_lower_id():
    x = torch.zeros(70, 16)
    w = torch.zeros(40, 16)
    ids, wts = moe_router(x.to(DEV), w.to(DEV), 5)
    assert cpu(ids).tolist() == [[0, 1, 2, 3, 4]] * 70
    assert torch.allclose(cpu(wts), torch.full((70, 5), 1 / 40))
    # two equal columns in the middle of the ranking
    w = torch.randn(12, 16, generator=torch.Generator().manual_seed(3))
    w[7] = w[2]
    x = torch.randn(9, 16, generator=torch.Generator().manual_seed(4))
    ids, _ = moe_router(x.to(DEV), w.to(DEV), 12)
    ids = cpu(ids)
    for row in ids.tolist():
        assert row.index(2) + 1 == row.index(7)


@pytest.mark.parametrize("T,E,K,H,dt", [(5, 5, 5, 12, torch.float32), (3, 33, 7, 20, torch.bfloat16),
                                        (130, 200, 32, 72, torch.float16), (100, 1024, 8, 64, torch.bfloat16),
                                        (65, 64, 1, 8, torch.float32)])
def test_router_ragged_shapes(T, E, K, H, dt):
    g = torch.Generator().manual_seed(T * 1000 + E)
    x = torch.randn(T, H, generator=g).to(dt)
    w = torch.randn(E, H, generator=g).to(dt)
    check_router(x, w, K, renorm=True)


def test_router_empty_batch_and_errors():
    ids, wts = moe_router(torch.zeros(0, 16, device=DEV), torch.zeros(4, 16, device=DEV), 2)
    assert ids.shape == (0, 2) and wts.shape == (0, 2)
    with pytest.raises(AssertionError):
        moe_router(torch.zeros(2, 16, device=DEV), torch.zeros(4, 16, device=DEV), 5)      # K > E
    with pytest.raises(ValueError):
        moe_router(torch.zeros(2, 16, device=DEV), torch.zeros(2048, 16, device=DEV), 2)   # E > 1024


# ------------------------------------------------------------------------------------------ permute
def check_plan(ids, E):
    K = ids.shape[1]
    perm, inv, off32, off64 = moe_permute_plan(ids.to(DEV), E)
    ref_perm, ref_inv = O.sort_slots(ids)
    ref_off = O.expert_offsets(ids, E)
    assert torch.equal(cpu(off64), ref_off) and torch.equal(cpu(off32).to(torch.int64), ref_off)
    assert torch.equal(cpu(perm).to(torch.int64), ref_perm), "permutation differs from a stable argsort"
    assert torch.equal(cpu(inv).to(torch.int64), ref_inv)
    return perm, inv, off32


@pytest.mark.parametrize("T,K,E,seed", [(1, 8, 128, 0), (8, 8, 128, 1), (64, 8, 128, 2), (256, 8, 128, 3),
                                         (257, 8, 128, 4), (333, 3, 7, 5), (4096, 8, 128, 6), (5000, 2, 1000, 7)])
def test_permute_plan_random(T, K, E, seed):
    g = torch.Generator().manual_seed(seed)
    ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]) if E >= K else None
    check_plan(ids, E)
    check_plan(ids.to(torch.int32), E)


def test_permute_plan_golden_routings():
    check_plan(torch.from_numpy(cases.golden("c2")["ids"]).to(torch.int64), 128)
    ids4 = torch.from_numpy(cases.golden("c4")["ids"]).to(torch.int64)        # skewed, empty experts, 131072 slots
    perm, inv, off = check_plan(ids4, 128)
    assert torch.equal(cpu(off).to(torch.int64), torch.from_numpy(cases.golden("c4")["offsets"]))


def test_permute_all_slots_one_expert():
    # reference: tests/test_moe_kernels.py:130-151 (every id = 0 -> experts 1.. are empty)
    T, K, E, H = 8, 4, 16, 256
    ids = torch.zeros(T, K, dtype=torch.int64)
    x = torch.randn(T, H, generator=torch.Generator().manual_seed(0)).to(torch.bfloat16)
    permuted, off = moe_permute(x.to(DEV), ids.to(DEV), E)
    assert off.dtype == torch.int64 and off[0] == 0 and off[1] == T * K and off[2] == T * K and off[-1] == T * K
    assert torch.equal(cpu(permuted), x.repeat_interleave(K, 0))


@pytest.mark.parametrize("dt,H", [(torch.bfloat16, 256), (torch.float32, 12), (torch.float16, 8), (torch.float32, 5)])
def test_moe_permute_rows(dt, H):
    T, K, E = 37, 4, 16
    g = torch.Generator().manual_seed(11)
    x = torch.randn(T, H, generator=g).to(dt)
    ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)])
    permuted, off = moe_permute(x.to(DEV), ids.to(DEV), E)
    ref_p, ref_off = O.permute(x, ids, E)
    assert permuted.shape == (T * K, H) and off[0] == 0 and off[-1] == T * K
    assert torch.equal(cpu(permuted), ref_p) and torch.equal(cpu(off), ref_off)


def test_permute_full_size_properties():
    # 16384 tokens x 8: sortedness, stability and inverse, without the oracle
    ids = torch.from_numpy(cases.golden("c4")["ids"]).to(torch.int32).to(DEV)
    perm, inv, off32, _ = moe_permute_plan(ids, 128)
    S = ids.numel()
    flat = ids.reshape(-1)
    sorted_ids = flat[perm.long()]
    assert bool((sorted_ids[1:] >= sorted_ids[:-1]).all())
    same = sorted_ids[1:] == sorted_ids[:-1]
    assert bool((perm[1:][same] > perm[:-1][same]).all())                    # ascending slot inside an expert
    assert torch.equal(perm[inv.long()].long(), torch.arange(S, device=DEV))
    assert torch.equal(off32[1:] - off32[:-1], torch.bincount(flat.long(), minlength=128).to(torch.int32))


# ------------------------------------------------------------------------------------------ unpermute
@pytest.mark.parametrize("dt,T,K,E,H", [(torch.bfloat16, 4, 4, 16, 256), (torch.float32, 9, 3, 8, 20),
                                        (torch.float16, 64, 8, 128, 2048), (torch.bfloat16, 1, 8, 128, 2048)])
def test_unpermute_vs_oracle(dt, T, K, E, H):
    g = torch.Generator().manual_seed(13)
    ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)])
    rows = torch.randn(T * K, H, generator=g).to(dt)
    w = torch.rand(T, K, generator=g)
    out = moe_unpermute(rows.to(DEV), w.to(DEV), ids.to(DEV), T)
    ref = O.unpermute(rows, w, ids, T)
    assert out.dtype == dt and out.shape == (T, H)
    if dt == torch.float32:
        torch.testing.assert_close(cpu(out), ref, rtol=1e-6, atol=1e-6)
    else:
        # fp32 sums that differ in the last bit can land on either side of a 16-bit rounding boundary
        torch.testing.assert_close(cpu(out).float(), ref.float(), rtol=2 ** -7, atol=1e-6)
        assert (cpu(out) != ref).float().mean() < 0.01


def test_permute_unpermute_round_trip():
    # reference: tests/test_moe_kernels.py:72-100: identity experts -> out = sum_k w[t,k] * x[t]
    T, E, K, H = 8, 16, 4, 256
    g = torch.Generator().manual_seed(13)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    router_w = torch.randn(E, H, generator=g).to(torch.bfloat16)
    ids, w = moe_router(x.to(DEV), router_w.to(DEV), K)
    permuted, _ = moe_permute(x.to(DEV), ids, E)
    out = moe_unpermute(permuted, w, ids, T)
    expect = (cpu(w).sum(-1, keepdim=True) * x.float())
    assert (cpu(out).float() - expect).abs().max() < 1e-2


# ------------------------------------------------------------------------------------------ grouped GEMM
@pytest.mark.parametrize("i", range(len(cases.KERNEL_SHAPES)))
def test_grouped_gemm_reference_shapes(i):
    T, E, K, H, D = cases.KERNEL_SHAPES[i]
    g = cases.golden("kernel_cases")
    hidden, router_w = cases.kernel_router_inputs(T, E, K, H)
    ids, _ = O.router(hidden, router_w, K)
    permuted, off = O.permute(hidden, ids, E)
    _, wg = cases.kernel_gemm_inputs(T, E, K, H, D)
    out = moe_grouped_gemm(permuted.to(DEV), wg.to(DEV), off.to(DEV))
    ref = cases.from_bits(g[f"gemm_out_{i}"], torch.bfloat16)
    assert out.shape == (T * K, D)
    assert (cpu(out).float() - ref.float()).abs().max() < 1e-2          # the reference's own bound
    torch.testing.assert_close(cpu(out).float(), ref.float(), rtol=2e-2, atol=2e-3)


def random_offsets(E, S, g, empty_every=3):
    cuts = torch.sort(torch.randint(0, S + 1, (E - 1,), generator=g)).values
    off = torch.cat([torch.tensor([0]), cuts, torch.tensor([S])])
    for e in range(0, E, empty_every):          # force some empty experts
        off[e + 1] = off[e]
    off = torch.cummax(off, 0).values
    off[-1] = S
    return off


@pytest.mark.parametrize("dt,S,E,N,Kd", [(torch.float32, 128, 8, 512, 256), (torch.float32, 50, 5, 24, 40),
                                         (torch.bfloat16, 300, 7, 72, 136), (torch.float16, 64, 4, 64, 64),
                                         (torch.bfloat16, 1000, 16, 256, 512), (torch.float32, 33, 3, 7, 5)])
def test_grouped_gemm_vs_oracle(dt, S, E, N, Kd):
    g = torch.Generator().manual_seed(S + N)
    a = torch.randn(S, Kd, generator=g).to(dt)
    w = (torch.randn(E, N, Kd, generator=g) * 0.05).to(dt)
    off = random_offsets(E, S, g)
    out = moe_grouped_gemm(a.to(DEV), w.to(DEV), off.to(DEV))
    ref = O.grouped_gemm(a, w, off)
    if dt == torch.float32:
        torch.testing.assert_close(cpu(out), ref, rtol=1e-5, atol=1e-5)
    else:
        torch.testing.assert_close(cpu(out).float(), ref.float(), rtol=2e-2, atol=2e-3)


def test_grouped_gemm_no_rows():
    w = torch.randn(4, 16, 32, device=DEV, dtype=torch.bfloat16)
    out = moe_grouped_gemm(torch.zeros(0, 32, device=DEV, dtype=torch.bfloat16), w, torch.zeros(5, dtype=torch.int64, device=DEV))
    assert out.shape == (0, 16)


@pytest.mark.parametrize("dt,S,E,I,H", [(torch.float32, 128, 8, 512, 256), (torch.bfloat16, 200, 6, 64, 128),
                                        (torch.bfloat16, 37, 3, 24, 40)])
def test_grouped_swiglu_vs_oracle(dt, S, E, I, H):
    g = torch.Generator().manual_seed(S + I)
    a = torch.randn(S, H, generator=g).to(dt)
    wg = (torch.randn(E, I, H, generator=g) * 0.05).to(dt)
    wu = (torch.randn(E, I, H, generator=g) * 0.05).to(dt)
    off = random_offsets(E, S, g)
    h = moe_grouped_swiglu(a.to(DEV), torch.cat([wg, wu], 1).to(DEV), off.to(torch.int32).to(DEV))
    ref = torch.zeros(S, I, dtype=dt)
    for e in range(E):
        s, t = int(off[e]), int(off[e + 1])
        if t > s:
            ref[s:t] = torch.nn.functional.silu(a[s:t] @ wg[e].T) * (a[s:t] @ wu[e].T)
    if dt == torch.float32:
        torch.testing.assert_close(cpu(h), ref, rtol=1e-5, atol=1e-5)
    else:
        torch.testing.assert_close(cpu(h).float(), ref.float(), rtol=2e-2, atol=2e-3)


# ------------------------------------------------------------------------------------------ W4A16
@pytest.mark.parametrize("i", range(len(cases.W4_GEMM_SHAPES)))
def test_w4a16_gemm_reference_shapes(i):
    # reference: tests/test_w4a16_gemm.py:89-125 (vs the fp64 product of the dequantised weight)
    M, K, N, gs = cases.W4_GEMM_SHAPES[i]
    x, w = cases.w4_gemm_inputs(M, K, N)
    qw, sc, qz = O.minmax_quantize(w, gs)
    out = w4a16_gemm(x.to(DEV), qw.to(DEV), sc.to(DEV), qz.to(DEV), gs)
    ref = cases.from_bits(cases.golden("quant_cases")[f"out_{i}"], torch.bfloat16)
    assert out.shape == (M, N) and out.dtype == torch.bfloat16
    err = (cpu(out).float() - ref.float()).abs().max().item()
    assert err < (1e-2 if K == 128 else 2.0)                             # the reference's own bounds
    torch.testing.assert_close(cpu(out).float(), ref.float(), rtol=2e-2, atol=2e-3)
    # and tighter: at most one bf16 ulp away from the fp32 oracle
    ora = O.w4a16_linear(x, qw, sc, qz, gs)
    assert ((cpu(out).float() - ora.float()).abs() <= ora.float().abs() * 2 ** -7 + 1e-3).all()


@pytest.mark.parametrize("S,E,N,Kd,gs", [(40, 5, 64, 256, 128), (70, 3, 96, 128, 32), (9, 4, 40, 64, 64),
                                          (130, 2, 768, 2048, 128)])
def test_w4a16_grouped_vs_oracle(S, E, N, Kd, gs):
    g = torch.Generator().manual_seed(S * 7 + N)
    x = torch.randn(S, Kd, generator=g).to(torch.bfloat16)
    trios = [O.minmax_quantize(torch.randn(Kd, N, generator=g) * 0.05, gs) for _ in range(E)]
    qw, sc, qz = (torch.stack([t[j] for t in trios]) for j in range(3))
    off = random_offsets(E, S, g, empty_every=4)
    out = w4a16_grouped_gemm(x.to(DEV), qw.to(DEV), sc.to(DEV), qz.to(DEV), off.to(torch.int32).to(DEV), gs)
    ref = torch.zeros(S, N, dtype=torch.bfloat16)
    for e in range(E):
        s, t = int(off[e]), int(off[e + 1])
        if t > s:
            ref[s:t] = O.w4a16_linear(x[s:t], qw[e], sc[e], qz[e], gs)
    torch.testing.assert_close(cpu(out).float(), ref.float(), rtol=2e-2, atol=2e-3)
    assert (cpu(out) != ref).float().mean() < 0.02


def test_w4a16_grouped_swiglu_vs_oracle():
    S, E, I, H, gs = 45, 4, 96, 256, 128
    g = torch.Generator().manual_seed(5)
    x = torch.randn(S, H, generator=g).to(torch.bfloat16)
    gate = [O.minmax_quantize(torch.randn(H, I, generator=g) * 0.05, gs) for _ in range(E)]
    up = [O.minmax_quantize(torch.randn(H, I, generator=g) * 0.05, gs) for _ in range(E)]
    st = lambda trios: tuple(torch.stack([t[j] for t in trios]).to(DEV) for j in range(3))
    off = random_offsets(E, S, g, empty_every=4)
    h = w4a16_grouped_swiglu(x.to(DEV), st(gate), st(up), off.to(torch.int32).to(DEV), gs)
    ref = torch.zeros(S, I, dtype=torch.bfloat16)
    for e in range(E):
        s, t = int(off[e]), int(off[e + 1])
        if t > s:
            ref[s:t] = torch.nn.functional.silu(O.w4a16_linear(x[s:t], *gate[e], gs)) * O.w4a16_linear(x[s:t], *up[e], gs)
    torch.testing.assert_close(cpu(h).float(), ref.float(), rtol=2e-2, atol=2e-3)


def test_w4a16_zero_point_extremes():
    # every (q, z) pair in 0..15 once: exact integers times a power-of-two scale must come out exact
    K, N, gs = 256, 16, 128
    q = torch.arange(K * N, dtype=torch.int32).reshape(K, N) % 16
    z = torch.arange(2 * N, dtype=torch.int32).reshape(2, N) % 16
    qw, qz = O.pack_int4(q.T.contiguous()).T.contiguous(), O.pack_int4(z)
    sc = torch.full((2, N), 0.25, dtype=torch.bfloat16)
    x = torch.ones(3, K, dtype=torch.bfloat16)
    out = w4a16_gemm(x.to(DEV), qw.to(DEV), sc.to(DEV), qz.to(DEV), gs)
    assert torch.equal(cpu(out), O.w4a16_linear(x, qw, sc, qz, gs))


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("T,E,K,H,dtype,renorm,biased", [
    (1, 128, 8, 2048, torch.bfloat16, True, False), (8, 128, 8, 2048, torch.bfloat16, True, False),
    (16, 128, 8, 2048, torch.float16, False, False), (64, 128, 8, 2048, torch.bfloat16, True, True),
    (5, 16, 4, 256, torch.float32, True, False), (33, 256, 8, 512, torch.bfloat16, False, True),
    (64, 8, 2, 136, torch.float32, True, False)])
def test_fused_small_batch_routing_equals_the_separate_kernels_and_the_oracle(T, E, K, H, dtype, renorm, biased):
    """mq_route_small (logits + top-k + plan + preparation in one launch) against the CPU oracle (ids, plan
    bit-exact) and against the separate launches it replaces."""
    from mini_qwen_b200.kernels.moe_router import moe_route_small, route_small_workspace
    from mini_qwen_b200.kernels.w4a16_gemm import w4a16_tc_prep
    g = torch.Generator().manual_seed(T * 1000 + E)
    x = torch.randn(T, H, generator=g).to(dtype)
    w = (torch.randn(E, H, generator=g) * 0.02).to(dtype)
    bias = (torch.randn(E, generator=g) * 0.5) if biased else None
    prepare = dtype == torch.bfloat16 and H % 128 == 0
    ws = route_small_workspace(E, DEV)
    for _ in range(2):                                   # the second call finds the workspace as the first left it
        ids32, wts, perm, inv, off32, xp, xs = moe_route_small(
            x.to(DEV), w.to(DEV), K, bias=None if bias is None else bias.to(DEV), renormalize=renorm,
            prepare=prepare, workspace=ws)
        ref_ids, ref_w = O.router(x, w, K, bias)
        if renorm:
            ref_w = O.renormalise(ref_w)
        assert torch.equal(cpu(ids32).to(torch.int64), ref_ids)
        torch.testing.assert_close(cpu(wts), ref_w, rtol=1e-4, atol=1e-6)
        ref_perm, ref_inv = O.sort_slots(ref_ids)
        assert torch.equal(cpu(perm).to(torch.int64), ref_perm) and torch.equal(cpu(inv).to(torch.int64), ref_inv)
        assert torch.equal(cpu(off32).to(torch.int64), O.expert_offsets(ref_ids, E))
        if prepare:
            xp2, xs2 = w4a16_tc_prep(x.to(DEV))          # per token, no gather
            assert torch.equal(xp, xp2) and torch.equal(xs[:, : H // 128], xs2[:, : H // 128])
            # ... and in the fp16 format (rows scaled by their power of two, its inverse in column 31)
            *_, xp16, xs16 = moe_route_small(x.to(DEV), w.to(DEV), K, bias=None if bias is None else bias.to(DEV),
                                             renormalize=renorm, prepare="f16", workspace=ws)
            xp3, xs3 = w4a16_tc_prep(x.to(DEV), f16=True)
            assert xp16.dtype == torch.float16 and torch.equal(xp16, xp3)
            assert torch.equal(xs16[:, : H // 128], xs3[:, : H // 128]) and torch.equal(xs16[:, 31], xs3[:, 31])
    # the separate launches give the same weights bit for bit or within an fp32 rounding of the logits
    ids_b, w_b, ids32_b = moe_router(x.to(DEV), w.to(DEV), K, bias=None if bias is None else bias.to(DEV),
                                     renormalize=renorm, return_int32_ids=True)
    assert torch.equal(ids32_b, ids32)
    torch.testing.assert_close(w_b, wts, rtol=1e-5, atol=1e-7)


def test_fused_routing_workspace_is_reusable_across_batch_sizes():
    """One workspace, batches of 64, then 8, then 1, then 33 tokens: the kernel's counter must not sit where an
    earlier, larger batch left its logits (it once did: no CTA then took the plan step and the outputs of the
    smaller batch were never written)."""
    from mini_qwen_b200.kernels.moe_router import moe_route_small, route_small_workspace
    E, K, H = 128, 8, 2048
    g = torch.Generator().manual_seed(5)
    w = (torch.randn(E, H, generator=g) * 0.02).to(torch.bfloat16)
    ws = route_small_workspace(E, DEV)
    for T in (64, 8, 1, 33, 2):
        x = torch.randn(T, H, generator=g).to(torch.bfloat16)
        ids32, wts, perm, inv, off32, _, _ = moe_route_small(x.to(DEV), w.to(DEV), K, renormalize=True, workspace=ws)
        ref_ids, ref_w = O.router(x, w, K, None)
        assert torch.equal(cpu(ids32).to(torch.int64), ref_ids), f"T={T}"
        ref_perm, ref_inv = O.sort_slots(ref_ids)
        assert torch.equal(cpu(perm).to(torch.int64), ref_perm) and torch.equal(cpu(inv).to(torch.int64), ref_inv)
        assert torch.equal(cpu(off32).to(torch.int64), O.expert_offsets(ref_ids, E))
        torch.testing.assert_close(cpu(wts), O.renormalise(ref_w), rtol=1e-4, atol=1e-6)
