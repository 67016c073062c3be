"""Seeded synthetic MoE layers with the shapes and value distributions of the benchmark
configurations (no dataset or checkpoint is involved; the configurations are the workload).

Everything is drawn from a CPU ``torch.Generator`` so that a CPU checker and the CUDA
kernels can be handed identical bits.  The draw order is part of the contract with the
stored golden outputs: x, router, gate, up, down (dense) and x, router, then per
projection q, z, s (W4A16).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .quantization.packing import pack_int4


@dataclass
class DenseLayer:
    x: torch.Tensor        # [T, H]
    router: torch.Tensor   # [E, H]
    gate: torch.Tensor     # [E, I, H]
    up: torch.Tensor       # [E, I, H]
    down: torch.Tensor     # [E, H, I]
    top_k: int


@dataclass
class W4Proj:
    qweight: torch.Tensor  # [E, K/8, N] int32, packed along K
    qzeros: torch.Tensor   # [E, K/g, N/8] int32, packed along N (as stored in a GPTQ file)
    scales: torch.Tensor   # [E, K/g, N] fp16 (as stored in a GPTQ file)


@dataclass
class W4Layer:
    x: torch.Tensor        # [T, H] bf16
    router: torch.Tensor   # [E, H] fp16
    gate: W4Proj
    up: W4Proj
    down: W4Proj
    top_k: int
    group_size: int


def dense_layer(seed: int, T: int, H: int, E: int, K: int, I: int, dtype=torch.bfloat16) -> DenseLayer:
    """Weights ~N(0, 0.02), hidden states ~N(0, 1), drawn in fp32 then cast to ``dtype``."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).to(dtype)
    router = (torch.randn(E, H, generator=g) * 0.02).to(dtype)
    gate = (torch.randn(E, I, H, generator=g) * 0.02).to(dtype)
    up = (torch.randn(E, I, H, generator=g) * 0.02).to(dtype)
    down = (torch.randn(E, H, I, generator=g) * 0.02).to(dtype)
    return DenseLayer(x, router, gate, up, down, K)


def _w4_proj(g: torch.Generator, E: int, Kd: int, N: int, group: int) -> W4Proj:
    q = torch.randint(0, 16, (E, N, Kd), generator=g, dtype=torch.int32)
    qweight = pack_int4(q).transpose(1, 2).contiguous()                       # [E, Kd/8, N]
    z = torch.randint(0, 16, (E, Kd // group, N), generator=g, dtype=torch.int32)
    qzeros = pack_int4(z)                                                     # [E, G, N/8]
    scales = (torch.rand(E, Kd // group, N, generator=g) * 0.015 + 0.005).to(torch.float16)
    return W4Proj(qweight, qzeros, scales)


def w4a16_layer(seed: int, T: int, H: int, E: int, K: int, I: int, group: int = 128) -> W4Layer:
    """int4 values uniform in [0, 15] (8 per int32 along K), per-group fp16 scales uniform in
    [0.005, 0.02], per-group stored zero points uniform in [0, 15] (zero_plus_one convention),
    fp16 router, bf16 hidden states."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    router = (torch.randn(E, H, generator=g) * 0.02).to(torch.float16)
    gate = _w4_proj(g, E, H, I, group)
    up = _w4_proj(g, E, H, I, group)
    down = _w4_proj(g, E, I, H, group)
    return W4Layer(x, router, gate, up, down, K, group)


def zipf_router_bias(seed: int, E: int, s: float = 1.2, strength: float = 1.0) -> torch.Tensor:
    """Logit bias that makes expert popularity follow Zipf(s) over a seeded random expert
    permutation: bias[perm[r-1]] = -strength * s * ln(r), r = 1..E."""
    g = torch.Generator().manual_seed(seed)
    order = torch.randperm(E, generator=g)
    bias = torch.empty(E, dtype=torch.float32)
    bias[order] = torch.tensor([-strength * s * math.log(r) for r in range(1, E + 1)], dtype=torch.float32)
    return bias


# ---- W4A16 layers drawn directly on a device (whole 48-layer stacks: 15 GB of packed weights) -------------
def gptq_zero_fix(qzeros: torch.Tensor) -> torch.Tensor:
    """What ``LinearW4A16.from_gptq(..., zero_plus_one=True)`` does to the stored zero points
    (mini_qwen/model/layers/linear_w4a16.py:96-99 of the reference): every nibble + 1, clamped to 15,
    repacked.  Works on any device and shape."""
    u = qzeros.to(torch.int64) & 0xFFFFFFFF
    out = torch.zeros_like(u)
    for i in range(8):
        nib = torch.clamp(((u >> (4 * i)) & 0xF) + 1, max=15)
        out |= nib << (4 * i)
    out = torch.where(out >= 2 ** 31, out - 2 ** 32, out)
    return out.to(torch.int32)


def w4a16_stacks_on_device(device, seed: int, experts: int, H: int, I: int, group: int = 128):
    """``experts`` experts of a W4A16 layer drawn on ``device`` with the distributions of the W4A16
    configurations: int4 values uniform in [0, 15] (i.e. uniform packed words), fp16 scales uniform in
    [0.005, 0.02] stored as bf16, stored zero points uniform in [0, 15] passed through the zero_plus_one
    fix-up.  Returns (gate, up, down), each (qweight [E,K/8,N] int32, scales [E,K/g,N] bf16,
    qzeros [E,K/g,N/8] int32) in the convention of the module buffers.  A pure function of (seed, shapes) on a
    given device type."""
    gen = torch.Generator(device=device).manual_seed(seed)

    def proj(kd, n):
        qw = torch.randint(-2 ** 31, 2 ** 31 - 1, (experts, kd // 8, n), generator=gen, device=device, dtype=torch.int32)
        sc = (torch.rand(experts, kd // group, n, generator=gen, device=device) * 0.015 + 0.005)
        sc = sc.to(torch.float16).to(torch.bfloat16)
        qz = torch.randint(-2 ** 31, 2 ** 31 - 1, (experts, kd // group, n // 8), generator=gen, device=device,
                           dtype=torch.int32)
        return qw, sc, gptq_zero_fix(qz)
    return proj(H, I), proj(H, I), proj(I, H)


def router_weight_on_device(device, seed: int, E: int, H: int) -> torch.Tensor:
    """Router weight ~N(0, 0.02) drawn as fp16 (the W4A16 configurations keep it in fp16) and held in bf16, as
    the reference's GPTQ loader casts it (mini_qwen/model/loader.py:253-259)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn(E, H, generator=gen, device=device) * 0.02).to(torch.float16).to(torch.bfloat16)


def rms_norm_weightless(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Weight-free RMS norm that keeps activations O(1) between chained MoE layers (the 48-layer stack has no
    attention and no learnt norms; without it SwiGLU's quadratic growth overflows within a few layers)."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)
