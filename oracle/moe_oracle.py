"""CPU oracle for the MoE block of mini-qwen-llm (router -> permute -> experts -> combine).

THIS FILE IS TEST INFRASTRUCTURE.  It restates, in plain torch CPU ops, the
arithmetic of the reference's PyTorch per-expert-loop path.  Only the test
suite, the smoke check and the benchmark's CPU-baseline leg may import it; the
product package never does.

Parity status: PINNED.  ``tests/golden/make_golden.py`` imports the reference
itself, runs it on seeded inputs and stores its outputs; ``tests/test_oracle.py``
checks every function below against those stored outputs bit for bit (integer
results) or to float equality (floating results computed with the same ops).

Each function cites the reference lines it follows (paths inside the reference
project).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

_NIBBLE_SHIFTS = (0, 4, 8, 12, 16, 20, 24, 28)


# --------------------------------------------------------------------------- router
def router_scores(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 logits and fp32 softmax (mini_qwen/kernels/moe_router.py:19-20).

    ``bias`` (fp32 [E]) is added to the logits before the softmax; the reference has no
    bias, it exists for the skewed-routing workload only.
    """
    logits = F.linear(x.float(), w.float())
    if bias is not None:
        logits = logits + bias.float()
    return F.softmax(logits, dim=-1)


def router(x, w, top_k: int, bias=None):
    """Top-k of the softmax scores (mini_qwen/kernels/moe_router.py:21-22).

    Returns (ids int64 [T,K], weights fp32 [T,K]) sorted by descending weight.  Equal
    scores are ordered by ascending expert id (a stable descending sort); torch.topk
    gives the same answer whenever the first K+1 scores of a row are distinct.
    """
    scores = router_scores(x, w, bias)
    order = torch.sort(scores, dim=-1, descending=True, stable=True)
    return order.indices[:, :top_k].contiguous(), order.values[:, :top_k].contiguous()


def renormalise(weights: torch.Tensor) -> torch.Tensor:
    """mini_qwen/model/layers/moe.py:55-56."""
    return weights / weights.sum(dim=-1, keepdim=True)


# --------------------------------------------------------------------------- permute
def sort_slots(ids: torch.Tensor):
    """Stable sort of the T*K flat slots by expert id (moe_permute.py:22-23).

    Returns (perm, inv): perm[p] = flat slot t*K+k stored at sorted position p,
    inv[t*K+k] = p (moe_unpermute.py:23-25).
    """
    flat = ids.reshape(-1)
    perm = torch.argsort(flat, stable=True)
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(perm.numel(), dtype=perm.dtype)
    return perm, inv


def expert_offsets(ids: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Exclusive prefix sum of the per-expert slot counts (moe_permute.py:26-27)."""
    counts = torch.bincount(ids.reshape(-1), minlength=num_experts)
    off = torch.zeros(num_experts + 1, dtype=torch.int64)
    off[1:] = torch.cumsum(counts, 0)
    return off


def permute(x: torch.Tensor, ids: torch.Tensor, num_experts: int):
    """moe_permute.py:19-33: rows of x gathered in expert-sorted slot order."""
    K = ids.shape[1]
    perm, _ = sort_slots(ids)
    return x[perm // K], expert_offsets(ids, num_experts)


# --------------------------------------------------------------------------- experts
def grouped_gemm(permuted: torch.Tensor, weights: torch.Tensor, offsets: torch.Tensor) -> torch.Tensor:
    """One projection per expert with fp32 accumulation
    (mini_qwen/kernels/moe_grouped_gemm.py:17-37). weights is [E, D, H]."""
    E, D, _ = weights.shape
    out = torch.zeros(permuted.shape[0], D, dtype=permuted.dtype)
    for e in range(E):
        s, t = int(offsets[e]), int(offsets[e + 1])
        if t > s:
            out[s:t] = (permuted[s:t].float() @ weights[e].float().T).to(permuted.dtype)
    return out


def expert_mlp(x_e, w_gate, w_up, w_down):
    """SwiGLU expert with nn.Linear semantics in the tensors' own dtype
    (mini_qwen/model/layers/moe.py:24-25): every intermediate is rounded to that dtype."""
    return F.linear(F.silu(F.linear(x_e, w_gate)) * F.linear(x_e, w_up), w_down)


def unpermute(out_perm, weights, ids, num_tokens: int):
    """Weighted sum over the K slots of each token, in fp32, k ascending
    (mini_qwen/kernels/moe_unpermute.py:20-31)."""
    T, K = ids.shape
    _, inv = sort_slots(ids)
    h = out_perm[inv].reshape(T, K, out_perm.shape[-1])
    return (weights.unsqueeze(-1) * h).sum(dim=1).to(out_perm.dtype)


def block_forward(x, gate_w, w_gate, w_up, w_down, top_k: int, norm_topk_prob: bool = True, bias=None,
                  expert_fn=None):
    """The per-expert loop of Qwen3MoEBlock.forward (mini_qwen/model/layers/moe.py:49-68).

    w_gate/w_up/w_down are indexable by expert ([E, I, H], [E, I, H], [E, H, I] or lists).
    ``expert_fn(e, x_e)`` overrides the dense expert (used for the W4A16 variant).
    Returns (out, ids, weights, offsets).
    """
    shape = x.shape
    x2d = x.reshape(-1, shape[-1])
    E = gate_w.shape[0]
    ids, wts = router(x2d, gate_w, top_k, bias)
    if norm_topk_prob:
        wts = renormalise(wts)
    permuted, off = permute(x2d, ids, E)
    out_perm = torch.zeros_like(permuted)
    for e in range(E):
        s, t = int(off[e]), int(off[e + 1])
        if t == s:
            continue
        if expert_fn is not None:
            out_perm[s:t] = expert_fn(e, permuted[s:t])
        else:
            out_perm[s:t] = expert_mlp(permuted[s:t], w_gate[e], w_up[e], w_down[e])
    out = unpermute(out_perm, wts, ids, x2d.shape[0])
    return out.reshape(shape), ids, wts, off


# --------------------------------------------------------------------------- decoder-layer glue
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """RMSNorm as the reference computes it (mini_qwen/model/layers/rms_norm.py:11-18): normalise in fp32,
    cast back to the input dtype, THEN multiply by the weight (a product of two tensors of the model dtype)."""
    xf = x.float()
    rms = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return weight * (xf * rms).to(x.dtype)


def moe_half_layer(h, norm_weight, eps, gate_w, w_gate, w_up, w_down, top_k: int, norm_topk_prob: bool = True,
                   bias=None, expert_fn=None):
    """Second half of the reference's MoE decoder layer (mini_qwen/model/qwen3_moe.py:63-66):
    ``h + mlp(post_attention_layernorm(h))``.  Returns (out, normalised input, ids)."""
    xn = rms_norm(h, norm_weight, eps)
    out, ids, _, _ = block_forward(xn, gate_w, w_gate, w_up, w_down, top_k, norm_topk_prob, bias, expert_fn)
    return h + out, xn, ids


# --------------------------------------------------------------------------- int4 format
def pack_int4(x: torch.Tensor) -> torch.Tensor:
    """8 values of 4 bits -> one int32 along the last axis, value i in bits [4i, 4i+4)
    (mini_qwen/quantization/packing.py:11-24)."""
    assert x.shape[-1] % 8 == 0
    v = x.to(torch.int64).reshape(*x.shape[:-1], -1, 8) & 0xF
    word = torch.zeros(v.shape[:-1], dtype=torch.int64)
    for i, sh in enumerate(_NIBBLE_SHIFTS):
        word |= v[..., i] << sh
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word)  # two's complement wrap
    return word.to(torch.int32)


def unpack_int4(p: torch.Tensor) -> torch.Tensor:
    """Inverse of pack_int4 (mini_qwen/quantization/packing.py:27-39)."""
    u = p.to(torch.int64) & 0xFFFFFFFF
    cols = [(u >> sh) & 0xF for sh in _NIBBLE_SHIFTS]
    return torch.stack(cols, dim=-1).reshape(*p.shape[:-1], -1).to(torch.int32)


def minmax_quantize(w: torch.Tensor, group_size: int = 128):
    """Per-group asymmetric 4-bit quantisation of w [K, N]
    (mini_qwen/quantization/awq.py:14-58). Returns (qweight [K/8,N] int32,
    scales [K/g,N] bf16, qzeros [K/g,N/8] int32)."""
    K, N = w.shape
    assert K % group_size == 0 and N % 8 == 0
    g = w.float().reshape(K // group_size, group_size, N)
    hi, lo = g.amax(dim=1), g.amin(dim=1)
    scale = ((hi - lo) / 15.0).clamp(min=1e-8)
    zero = (-lo / scale).round().clamp(0, 15).to(torch.int32)
    q = (g / scale[:, None, :] + zero[:, None, :].float()).round().clamp(0, 15).to(torch.int32).reshape(K, N)
    return pack_int4(q.T).T, scale.to(torch.bfloat16), pack_int4(zero)


def gptq_buffers(qweight, qzeros, scales, zero_plus_one: bool = True):
    """What LinearW4A16.from_gptq stores (mini_qwen/model/layers/linear_w4a16.py:92-101):
    scales rounded to bf16; stored zero + 1 clamped to [0, 15] (15 stays 15)."""
    z = unpack_int4(qzeros.to(torch.int32))
    if zero_plus_one:
        z = (z + 1).clamp(0, 15)
    return qweight.to(torch.int32), scales.to(torch.bfloat16), pack_int4(z)


def dequantise(qweight, scales, qzeros, group_size: int = 128) -> torch.Tensor:
    """fp32 weight [K, N] = (q - z[group]) * s[group]  (tests/test_w4a16_gemm.py:19-44)."""
    q = unpack_int4(qweight.T.contiguous()).T.float()            # [K, N]
    z = unpack_int4(qzeros).float()                               # [G, N]
    s = scales.float()                                            # [G, N]
    return (q - z.repeat_interleave(group_size, 0)) * s.repeat_interleave(group_size, 0)


def w4a16_linear(x, qweight, scales, qzeros, group_size: int = 128, accumulate=torch.float32) -> torch.Tensor:
    """x @ dequantised weight in fp32, result rounded to bf16
    (contract of mini_qwen/kernels/w4a16_gemm.py:8-15, checked the way
    tests/test_w4a16_gemm.py:89-125 checks it).  ``accumulate=torch.float64`` evaluates the same
    product with exact sums (the dequantised weight is still the fp32 one): the yardstick for how far
    the fp32 summation order alone moves the bf16 result."""
    w = dequantise(qweight, scales, qzeros, group_size)
    return (x.to(accumulate) @ w.to(accumulate)).to(torch.bfloat16)


def w4a16_expert(x_e, gate, up, down, group_size: int = 128, accumulate=torch.float32):
    """SwiGLU expert whose three projections are W4A16 linears; activations between them are
    bf16 as LinearW4A16.forward returns bf16 (linear_w4a16.py:31-36, moe.py:24-25).
    gate/up/down are (qweight, scales, qzeros) triples."""
    g = w4a16_linear(x_e, *gate, group_size, accumulate)
    u = w4a16_linear(x_e, *up, group_size, accumulate)
    return w4a16_linear(F.silu(g) * u, *down, group_size, accumulate)
