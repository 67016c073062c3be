"""CPU checks of the host side: int4 format, quantiser, LinearW4A16 constructors, the module tree
of the block, and that libmqmoe.so loads and exports every symbol include/mqmoe.h declares.
No kernel is launched here."""
import ctypes
import os
import re

import pytest
import torch
import torch.nn as nn

import cases
from mini_qwen_b200 import Qwen3MoEConfig, _cabi
from mini_qwen_b200.kernels import moe_grouped_gemm, moe_permute, moe_router, moe_unpermute, w4a16_gemm
from mini_qwen_b200.model.layers import LinearW4A16, Qwen3MoEBlock
from mini_qwen_b200.quantization import _per_group_minmax_quantize, pack_int4, quantize_awq, unpack_int4
from oracle import moe_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_pack_unpack_roundtrip_along_k():
    # reference: tests/test_w4a16_gemm.py:67-75
    K, N = 128, 64
    w = torch.randint(0, 16, (K, N), dtype=torch.int32, generator=torch.Generator().manual_seed(0))
    packed = pack_int4(w.T).T
    assert packed.shape == (K // 8, N) and packed.dtype == torch.int32
    assert torch.equal(unpack_int4(packed.T).T, w)


def test_pack_unpack_roundtrip_along_n():
    # reference: tests/test_w4a16_gemm.py:78-84
    z = torch.randint(0, 16, (8, 64), dtype=torch.int32, generator=torch.Generator().manual_seed(1))
    packed = pack_int4(z)
    assert packed.shape == (8, 8)
    assert torch.equal(unpack_int4(packed), z)


def test_pack_layout_and_sign():
    x = torch.tensor([[1, 2, 3, 4, 5, 6, 7, 8]], dtype=torch.int32)
    assert pack_int4(x).item() == 0x87654321 - (1 << 32)     # nibble 7 >= 8 -> negative int32
    assert torch.equal(pack_int4(x), O.pack_int4(x))
    with pytest.raises(AssertionError):
        pack_int4(torch.zeros(3, 7, dtype=torch.int32))


def test_minmax_quantiser_matches_oracle():
    w = torch.randn(256, 64, generator=torch.Generator().manual_seed(2))
    for a, b in zip(_per_group_minmax_quantize(w, 128), O.minmax_quantize(w, 128)):
        assert torch.equal(a, b)
    with pytest.raises(AssertionError):
        _per_group_minmax_quantize(torch.randn(100, 64), 128)
    with pytest.raises(NotImplementedError):
        quantize_awq(None, None)


def test_from_gptq_zero_plus_one_clamps():
    g = cases.golden("quant_cases")
    stored = pack_int4(torch.arange(16, dtype=torch.int32).reshape(1, 16))
    layer = LinearW4A16.from_gptq(torch.zeros(16, 16, dtype=torch.int32), stored, torch.ones(1, 16) * 0.0123)
    assert torch.equal(layer.qzeros, torch.from_numpy(g["gptq_zeros"]))
    assert torch.equal(layer.scales, cases.from_bits(g["gptq_scales"], torch.bfloat16))
    assert unpack_int4(layer.qzeros)[0, -2:].tolist() == [15, 15]      # stored 14 -> 15, stored 15 stays 15
    raw = LinearW4A16.from_gptq(torch.zeros(16, 16, dtype=torch.int32), stored, torch.ones(1, 16), zero_plus_one=False)
    assert torch.equal(raw.qzeros, stored)


def test_from_float_shapes_and_state_dict_keys():
    lin = nn.Linear(256, 64, bias=False)
    q = LinearW4A16.from_float(lin, group_size=128)
    assert q.qweight.shape == (32, 64) and q.scales.shape == (2, 64) and q.qzeros.shape == (2, 8)
    assert set(q.state_dict()) == {"qweight", "scales", "qzeros"}
    qw, sc, qz = O.minmax_quantize(lin.weight.data.float().T.contiguous(), 128)
    assert torch.equal(q.qweight, qw) and torch.equal(q.scales, sc) and torch.equal(q.qzeros, qz)


def test_block_module_tree_matches_hf_names():
    cfg = Qwen3MoEConfig(hidden_size=32, intermediate_size=16, num_experts=4, num_experts_per_tok=2)
    blk = Qwen3MoEBlock(cfg)
    keys = set(blk.state_dict())
    assert "gate.weight" in keys
    for e in range(4):
        for p in ("gate_proj", "up_proj", "down_proj"):
            assert f"experts.{e}.{p}.weight" in keys
    assert blk.num_experts == 4 and blk.num_experts_per_tok == 2 and blk.norm_topk_prob is True
    # stacking keeps the per-expert tensors addressable and shares their storage
    before = {k: v.clone() for k, v in blk.state_dict().items()}
    blk.finalize()
    for k, v in blk.state_dict().items():
        assert torch.equal(v, before[k])
    assert blk.experts[1].up_proj.weight.data_ptr() == blk._stacks["w13"][1, 16:].data_ptr()
    # an in-place load writes through to the stacks
    blk.load_state_dict({k: torch.full_like(v, 0.5) for k, v in before.items()})
    assert float(blk._stacks["w2"].min()) == 0.5
    # replacing a projection invalidates the stacks
    epoch = blk._epoch[0]
    blk.experts[0].gate_proj = nn.Linear(32, 16, bias=False)
    assert blk._epoch[0] == epoch + 1


def test_block_quantize_to_w4a16_swaps_modules():
    cfg = Qwen3MoEConfig(hidden_size=64, intermediate_size=32, num_experts=2, num_experts_per_tok=1)
    blk = Qwen3MoEBlock(cfg)
    blk.quantize_to_w4a16(group_size=32)
    assert all(isinstance(getattr(ex, p), LinearW4A16) for ex in blk.experts for p in ("gate_proj", "up_proj", "down_proj"))
    blk.finalize()
    assert blk._stacks["w4"] and blk._stacks["gate_proj"][0].shape == (2, 8, 32)
    assert blk.experts[1].down_proj.qweight.data_ptr() == blk._stacks["down_proj"][0][1].data_ptr()


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "mqmoe.h")).read()
    declared = set(re.findall(r"\b(mq_[a-z0-9_]+)\s*\(", header))
    declared -= {"mq_status", "mq_dtype"}
    assert declared == set(_cabi.PROTOTYPES), declared ^ set(_cabi.PROTOTYPES)
    lib = _cabi.load()
    for name in declared:
        assert isinstance(getattr(lib, name), ctypes._CFuncPtr)
    assert lib.mq_version() >= 1
    assert lib.mq_status_string(2).decode().startswith("size outside")


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_cabi, "_lib", None)
    monkeypatch.setenv("MQMOE_LIB", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _cabi.load()


def test_cpu_tensors_are_rejected():
    x = torch.randn(4, 32)
    with pytest.raises(ValueError, match="CUDA"):
        moe_router(x, torch.randn(8, 32), 2)
    with pytest.raises(ValueError, match="CUDA"):
        moe_permute(x, torch.zeros(4, 2, dtype=torch.int64), 8)
    with pytest.raises(ValueError, match="CUDA"):
        moe_grouped_gemm(x, torch.randn(8, 16, 32), torch.zeros(9, dtype=torch.int64))
    with pytest.raises(ValueError, match="CUDA"):
        moe_unpermute(torch.randn(8, 32), torch.rand(4, 2), torch.zeros(4, 2, dtype=torch.int64), 4)
    with pytest.raises(AssertionError):
        w4a16_gemm(x.to(torch.bfloat16), torch.zeros(4, 8, dtype=torch.int32),
                   torch.zeros(1, 8, dtype=torch.bfloat16), torch.zeros(1, 1, dtype=torch.int32), 32)


def test_argument_checks_return_status_without_a_gpu():
    lib = _cabi.load()
    # nothing is launched when the argument check fails, so these are safe on a CPU-only host
    assert lib.mq_router_topk(None, 0, None, 0, None, 4, 32, 8, 9, 0, None, 0, None, None, None, None) == 2   # K > E
    assert lib.mq_router_topk(None, 0, None, 0, None, 4, 32, 8, 2, 0, None, 0, None, None, None, None) == 1   # null
    assert lib.mq_router_topk(None, 7, None, 0, None, 4, 32, 8, 2, 0, None, 0, None, None, None, None) == 1   # dtype
    assert lib.mq_permute_plan(None, 1, 4, 2, 128, None, None, None, None, None, 0, None) == 1             # no offsets
    assert lib.mq_permute_plan(None, 1, 4, 2, 2048, None, None, None, None, None, 0, None) == 2            # E > 1024
    assert lib.mq_w4a16_grouped_gemm(None, None, None, None, None, 4, 1, 1, 8, 128, 48, None, None) == 2      # group % 32
    assert lib.mq_unpermute_combine(None, 1, None, None, 4, 33, 64, None, None) == 2                        # K > 32
    assert lib.mq_permute_workspace_bytes(131072, 128) >= 64 * 128 * 4


def test_from_stacked_shares_storage():
    cfg = Qwen3MoEConfig(hidden_size=32, intermediate_size=16, num_experts=4, num_experts_per_tok=2)
    w13, w2, r = torch.randn(4, 32, 32), torch.randn(4, 32, 16), torch.randn(4, 32)
    blk = Qwen3MoEBlock.from_stacked(cfg, r, w13, w2)
    assert blk.experts[2].up_proj.weight.data_ptr() == w13[2, 16:].data_ptr()
    assert torch.equal(blk.state_dict()["experts.3.down_proj.weight"], w2[3])
    assert blk._ready()["w13"].data_ptr() == w13.data_ptr()       # no restack needed


def test_static_router_scratch_covers_every_batch_up_to_16384_tokens():
    """mq_router_topk_static promises room for any batch up to 16384 tokens at the Qwen3-30B-A3B router
    shape.  The request is not monotonic in T (the logits are kept in several K slices for small
    batches), so every T is checked against the 10 MiB array, and the first refused batch size is pinned."""
    lib = _cabi.load()
    limit = 10 << 20
    worst = max(lib.mq_router_workspace_bytes(T, 2048, 128) for T in range(1, 16385))
    assert worst <= limit, worst
    assert worst == 2 * 9440 * 128 * 4                  # the documented peak: two slices at 9440 tokens
    assert lib.mq_router_workspace_bytes(20480, 2048, 128) == limit     # the largest batch that fits
    # one token more is refused by the argument check, before anything touches a device
    assert lib.mq_router_topk_static(None, 1, None, 1, None, 20481, 2048, 128, 8, 0, None, None, None, None) == 6


def test_ep_entry_points_reject_bad_poll_budgets_without_a_gpu():
    lib = _cabi.load()
    assert lib.mq_ep_barrier(None, None, 2, 0, 0, None, None) == 1                  # null pointers
    assert lib.mq_stack_tensors(None, 3, 64, 1, None, None) == 1                     # null pointers
    assert lib.mq_stack_tensors(None, 0, 64, 1, None, None) == 0                     # nothing to do
    assert lib.mq_stack_tensors(None, 70000, 64, 1, None, None) == 1


def test_decode_replication_entry_points_reject_bad_arguments_without_a_gpu():
    lib = _cabi.load()
    assert lib.mq_ep_gather_tokens(None, 1, 4, 2048, 2, 0, None, None, None, 0, None, None) == 1     # null pointers
    assert lib.mq_ep_gather_tokens(None, 1, 4, 2048, 2, 2, None, None, None, 0, None, None) == 1     # rank >= G
    assert lib.mq_ep_gather_tokens(None, 1, 4, 2047, 2, 0, None, None, None, 0, None, None) == 2     # rows not 16-byte multiples
    # tokens must be G * T
    assert lib.mq_ep_send_partials(None, 1, None, None, None, 9, 8, 2048, 4, 2, 0, 64, None, None, None, None, 0,
                                   None, None) == 1
    assert lib.mq_ep_send_partials(None, 1, None, None, None, 8, 33, 2048, 4, 2, 0, 64, None, None, None, None, 0,
                                   None, None) == 2                                             # K > 32
    assert lib.mq_ep_sum_partials(None, 1, None, 4, 2048, 2, None, None) == 1                        # null pointers
    assert lib.mq_ep_sum_partials(None, 1, None, 4, 2046, 2, None, None) == 2                        # H not a multiple of 4
    assert lib.mq_rms_norm(None, 1, None, 1e-6, 4, 2048, None, None) == 1                            # null pointers
    assert lib.mq_rms_norm(None, 1, None, 1e-6, 0, 2048, None, None) == 0                            # nothing to do
    assert lib.mq_unpermute_combine_residual(None, 1, None, None, None, 4, 33, 64, None, None) == 2  # K > 32
