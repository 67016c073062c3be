"""Seeded inputs shared by the golden-vector generator (tests/golden/make_golden.py) and the
tests.  Everything here is a pure function of its seed, drawn on the CPU generator."""
from __future__ import annotations

import functools
import os

import numpy as np
import torch

from mini_qwen_b200 import synthetic

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden(name: str):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def from_bits(a: np.ndarray, dtype) -> torch.Tensor:
    """Inverse of make_golden.bits()."""
    t = torch.from_numpy(np.ascontiguousarray(a))
    return t.view(torch.bfloat16) if dtype == torch.bfloat16 else t


# ---- the five cases of the reference's scripts/test_moe_synthetic.py:106-133 -------------------
SCRIPT_CASES = [
    dict(T=1, E=4, K=2, H=8, D=4, seed=0, dtype=torch.float32, norm=True),
    dict(T=4, E=8, K=3, H=16, D=8, seed=1, dtype=torch.float32, norm=True),
    dict(T=2, E=16, K=4, H=32, D=16, seed=2, dtype=torch.bfloat16, norm=True),
    dict(T=2, E=8, K=2, H=16, D=8, seed=3, dtype=torch.float32, norm=False),
    dict(T=1, E=128, K=8, H=64, D=32, seed=42, dtype=torch.bfloat16, norm=True),
]


def script_case_inputs(c):
    """Same draw order as the reference script's run_test (global generator, N(0,1) weights)."""
    torch.manual_seed(c["seed"])
    dt = c["dtype"]
    x = torch.randn(c["T"], c["H"], dtype=dt)
    gate_w = torch.randn(c["E"], c["H"], dtype=dt)
    gw = torch.stack([torch.randn(c["D"], c["H"], dtype=dt) for _ in range(c["E"])])
    uw = torch.stack([torch.randn(c["D"], c["H"], dtype=dt) for _ in range(c["E"])])
    dw = torch.stack([torch.randn(c["H"], c["D"], dtype=dt) for _ in range(c["E"])])
    return x, gate_w, gw, uw, dw


# ---- shapes of the reference's tests/test_moe_kernels.py:19-23 ---------------------------------
KERNEL_SHAPES = [(4, 16, 4, 256, 128), (8, 16, 4, 256, 128), (1, 16, 4, 256, 128)]


def kernel_router_inputs(T, E, K, H):
    g = torch.Generator().manual_seed(42)
    hidden = torch.randn(T, H, generator=g).to(torch.bfloat16)
    router_w = torch.randn(E, H, generator=g).to(torch.bfloat16)
    return hidden, router_w


def kernel_gemm_inputs(T, E, K, H, D):
    g = torch.Generator().manual_seed(99)
    x = torch.randn(T * K, H, generator=g).to(torch.bfloat16)
    w = (torch.randn(E, D, H, generator=g) * 0.1).to(torch.bfloat16)
    return x, w


# ---- W4A16 single-linear shapes of the reference's tests/test_w4a16_gemm.py:89-125 -------------
W4_GEMM_SHAPES = [(1, 128, 8, 128), (1, 1024, 4096, 128), (4, 1024, 4096, 128), (16, 1024, 4096, 128),
                  (3, 256, 64, 32)]


def w4_gemm_inputs(M, K, N):
    g = torch.Generator().manual_seed(1000 + M + K + N)
    w = torch.randn(K, N, generator=g)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    return x, w


# ---- benchmark configurations ------------------------------------------------------------------
@functools.lru_cache(maxsize=1)
def config1():
    """Tiny fp32 layer: T=64, H=256, E=8, top-2, I=512, seed 0."""
    return synthetic.dense_layer(0, T=64, H=256, E=8, K=2, I=512, dtype=torch.float32)


C2_SAMPLE_ROWS = 64


@functools.lru_cache(maxsize=1)
def config2():
    """Qwen3-30B-A3B-shaped bf16 prefill layer: T=4096, H=2048, E=128, top-8, I=768, seed 1."""
    return synthetic.dense_layer(1, T=4096, H=2048, E=128, K=8, I=768, dtype=torch.bfloat16)


C3_TS = (1, 8, 16, 64)


@functools.lru_cache(maxsize=1)
def config3():
    """Same shape in W4A16, seed 2; decode batches are the first T rows of the 64 drawn."""
    return synthetic.w4a16_layer(2, T=64, H=2048, E=128, K=8, I=768, group=128)


C4_SAMPLE_ROWS = 16
C4_BIAS_STRENGTH = 1.0


@functools.lru_cache(maxsize=1)
def config4():
    """Skewed-routing layer: T=16384 bf16, seed 4, routed with config4_bias()."""
    return synthetic.dense_layer(4, T=16384, H=2048, E=128, K=8, I=768, dtype=torch.bfloat16)


def config4_bias():
    return synthetic.zipf_router_bias(5, 128, s=1.2, strength=C4_BIAS_STRENGTH)
