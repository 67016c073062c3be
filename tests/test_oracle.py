"""Pins the CPU oracle (oracle/moe_oracle.py) to the stored outputs of the reference
implementation (tests/golden/*.npz, produced by tests/golden/make_golden.py)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

import cases
from oracle import moe_oracle as O


def _eq(a: torch.Tensor, b: torch.Tensor):
    assert a.shape == b.shape and a.dtype == b.dtype
    assert torch.equal(a, b), f"max abs diff {(a.float() - b.float()).abs().max().item()}"


@pytest.mark.parametrize("i", range(len(cases.SCRIPT_CASES)))
def test_script_cases(i):
    c = cases.SCRIPT_CASES[i]
    g = cases.golden("script_cases")
    x, gate_w, gw, uw, dw = cases.script_case_inputs(c)
    out, ids, wts, off = O.block_forward(x, gate_w, gw, uw, dw, c["K"], c["norm"])
    _eq(ids, torch.from_numpy(g[f"ids_{i}"]))
    _eq(wts, torch.from_numpy(g[f"weights_{i}"]))
    _eq(off, torch.from_numpy(g[f"offsets_{i}"]))
    permuted, _ = O.permute(x, ids, c["E"])
    _eq(permuted, cases.from_bits(g[f"permuted_{i}"], c["dtype"]))
    _eq(out, cases.from_bits(g[f"out_{i}"], c["dtype"]))


@pytest.mark.parametrize("i", range(len(cases.KERNEL_SHAPES)))
def test_kernel_cases(i):
    T, E, K, H, D = cases.KERNEL_SHAPES[i]
    g = cases.golden("kernel_cases")
    hidden, router_w = cases.kernel_router_inputs(T, E, K, H)
    ids, w = O.router(hidden, router_w, K)
    _eq(ids, torch.from_numpy(g[f"router_ids_{i}"]))
    _eq(w, torch.from_numpy(g[f"router_w_{i}"]))
    permuted, off = O.permute(hidden, ids, E)
    _eq(off, torch.from_numpy(g[f"permute_off_{i}"]))
    _, wg = cases.kernel_gemm_inputs(T, E, K, H, D)
    _eq(O.grouped_gemm(permuted, wg, off), cases.from_bits(g[f"gemm_out_{i}"], torch.bfloat16))


def test_sort_slots_is_stable_and_inverse():
    ids = torch.tensor([[3, 1], [1, 3], [0, 1], [3, 0]])
    perm, inv = O.sort_slots(ids)
    assert perm.tolist() == [4, 7, 1, 2, 5, 0, 3, 6]
    assert torch.equal(perm[inv], torch.arange(8))
    assert O.expert_offsets(ids, 5).tolist() == [0, 2, 5, 5, 8, 8]


def test_router_tie_rule():
    # equal scores: ascending expert id
    x = torch.zeros(2, 4)
    w = torch.zeros(6, 4)
    ids, wts = O.router(x, w, 3)
    assert ids.tolist() == [[0, 1, 2], [0, 1, 2]]
    assert torch.allclose(wts, torch.full((2, 3), 1 / 6))


@pytest.mark.parametrize("i", range(len(cases.W4_GEMM_SHAPES)))
def test_w4a16_linear(i):
    M, K, N, gs = cases.W4_GEMM_SHAPES[i]
    g = cases.golden("quant_cases")
    x, w = cases.w4_gemm_inputs(M, K, N)
    qw, sc, qz = O.minmax_quantize(w, gs)
    assert int(qw.to(torch.int64).sum()) == int(g[f"qweight_sum_{i}"][0])
    ref = cases.from_bits(g[f"out_{i}"], torch.bfloat16)          # fp64 product rounded to bf16
    got = O.w4a16_linear(x, qw, sc, qz, gs)                        # fp32 product rounded to bf16
    # the two differ only where fp32 summation error crosses a bf16 rounding boundary (<= 1 bf16 ulp;
    # 1e-4 absolute covers outputs that cancel to almost zero)
    diff = (got.float() - ref.float()).abs()
    assert (diff <= ref.float().abs() * 2 ** -7 + 1e-4).all()
    assert (diff > 0).float().mean() < 0.02


def test_gptq_zero_fixup():
    g = cases.golden("quant_cases")
    stored = O.pack_int4(torch.arange(16, dtype=torch.int32).reshape(1, 16))
    qw, sc, qz = O.gptq_buffers(torch.zeros(16, 16, dtype=torch.int32), stored, torch.ones(1, 16) * 0.0123)
    _eq(qz, torch.from_numpy(g["gptq_zeros"]))
    _eq(sc, cases.from_bits(g["gptq_scales"], torch.bfloat16))
    assert O.unpack_int4(qz).tolist() == [[1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 15]]


def test_config1_fp32():
    lay, g = cases.config1(), cases.golden("c1")
    out, ids, wts, off = O.block_forward(lay.x, lay.router, lay.gate, lay.up, lay.down, lay.top_k, True)
    raw_ids, raw_w = O.router(lay.x, lay.router, lay.top_k)
    _eq(raw_ids, torch.from_numpy(g["ids"]).to(torch.int64))
    _eq(raw_w, torch.from_numpy(g["weights"]))
    _eq(off, torch.from_numpy(g["offsets"]))
    _eq(out, torch.from_numpy(g["out"]))


def _w4_expert_fn(lay):
    """Expert e of a W4Layer through the oracle (buffers as LinearW4A16.from_gptq stores them)."""
    cache = {}

    def fn(e, x_e):
        if e not in cache:
            cache[e] = [O.gptq_buffers(p.qweight[e], p.qzeros[e], p.scales[e]) for p in (lay.gate, lay.up, lay.down)]
        gate, up, down = cache[e]
        return O.w4a16_expert(x_e, gate, up, down, lay.group_size)
    return fn


@pytest.mark.parametrize("T", cases.C3_TS)
def test_config3_w4a16(T):
    lay, g = cases.config3(), cases.golden("c3")
    x = lay.x[:T]
    router = lay.router.to(torch.bfloat16)
    out, ids, wts, off = O.block_forward(x, router, None, None, None, lay.top_k, True, expert_fn=_w4_expert_fn(lay))
    raw_ids, raw_w = O.router(x, router, lay.top_k)
    _eq(raw_ids, torch.from_numpy(g[f"ids_T{T}"]).to(torch.int64))
    _eq(raw_w, torch.from_numpy(g[f"weights_T{T}"]))
    _eq(off, torch.from_numpy(g[f"offsets_T{T}"]))
    _eq(out, cases.from_bits(g[f"out_T{T}"], torch.bfloat16))


def test_config2_bf16_prefill():
    lay, g = cases.config2(), cases.golden("c2")
    out, ids, wts, off = O.block_forward(lay.x, lay.router, lay.gate, lay.up, lay.down, lay.top_k, True)
    raw_ids, raw_w = O.router(lay.x, lay.router, lay.top_k)
    _eq(raw_ids, torch.from_numpy(g["ids"]).to(torch.int64))
    _eq(raw_w, torch.from_numpy(g["weights"]))
    _eq(off, torch.from_numpy(g["offsets"]))
    _eq(out[: cases.C2_SAMPLE_ROWS], cases.from_bits(g["out"], torch.bfloat16))


def test_config4_skewed_routing():
    lay, g = cases.config4(), cases.golden("c4")
    bias = cases.config4_bias()
    raw_ids, raw_w = O.router(lay.x, lay.router, lay.top_k, bias)
    _eq(raw_ids, torch.from_numpy(g["ids"]).to(torch.int64))
    _eq(raw_w, torch.from_numpy(g["weights"]))
    off = O.expert_offsets(raw_ids, 128)
    _eq(off, torch.from_numpy(g["offsets"]))
    counts = off[1:] - off[:-1]
    assert int((counts == 0).sum()) >= 1          # the workload leaves some experts empty


@pytest.mark.parametrize("i", range(len(cases.GLUE_CASES)))
def test_decoder_layer_glue(i):
    """RMSNorm in, residual add out: bit-exact against the reference's own layer arithmetic."""
    c = cases.GLUE_CASES[i]
    g = cases.golden("glue_cases")
    lay, h, norm_w = cases.glue_case_inputs(c)
    out, xn, ids = O.moe_half_layer(h, norm_w, c["eps"], lay.router, lay.gate, lay.up, lay.down, c["K"])
    assert torch.equal(xn, cases.from_bits(g[f"normed_{i}"], c["dtype"]))
    assert torch.equal(ids, torch.from_numpy(g[f"ids_{i}"]))
    assert torch.equal(out, cases.from_bits(g[f"out_{i}"], c["dtype"]))
