"""Unpermute + weighted combine. Same call as ``mini_qwen/kernels/moe_unpermute.py:9-31``."""
from __future__ import annotations

import torch

from .. import _cabi
from .moe_permute import moe_permute_plan

_MAX_EXPERTS = 1024   # largest expert count the permute plan supports


def unpermute_combine(permuted_output: torch.Tensor, topk_weights: torch.Tensor, inv: torch.Tensor,
                      num_tokens: int, top_k: int, residual: torch.Tensor | None = None) -> torch.Tensor:
    """``out[t] = cast(sum_k topk_weights[t,k] * float(permuted_output[inv[t*K+k]]))`` in fp32, k ascending.
    With ``residual`` [T,H] the decoder layer's add (``mini_qwen/model/qwen3_moe.py:66``) runs in the same kernel:
    ``out[t] = residual[t] + out[t]`` as an add of two tensors of the model dtype."""
    rows = permuted_output.contiguous()
    w = topk_weights.to(torch.float32).contiguous()
    H = rows.shape[1]
    out = torch.empty(num_tokens, H, dtype=rows.dtype, device=rows.device)
    if residual is not None:
        assert residual.shape == out.shape and residual.dtype == out.dtype and residual.is_contiguous()
        _cabi.require_cuda(residual)
    rc = _cabi.load().mq_unpermute_combine_residual(
        _cabi.ptr(rows), _cabi.dtype_code(rows), _cabi.ptr(w), _cabi.ptr(inv),
        _cabi.ptr(residual) if residual is not None else None,
        num_tokens, top_k, H, _cabi.ptr(out), _cabi.stream_ptr(rows.device))
    _cabi.check(rc, "mq_unpermute_combine_residual")
    _cabi.count_launches(1 if num_tokens else 0)
    return out


def moe_unpermute(
    permuted_output: torch.Tensor,  # [num_tokens * top_k, hidden_dim]
    topk_weights: torch.Tensor,     # [num_tokens, top_k] float32
    topk_ids: torch.Tensor,         # [num_tokens, top_k]
    num_tokens: int,
) -> torch.Tensor:
    """Restores token order and sums each token's K expert outputs weighted by ``topk_weights``.
    The slot order is rebuilt from ``topk_ids`` exactly as :func:`moe_permute` builds it."""
    _cabi.require_cuda(permuted_output, topk_weights, topk_ids)
    T, K = topk_ids.shape
    assert T == num_tokens and permuted_output.shape[0] == T * K
    # the signature carries no expert count; the plan's upper bound avoids reading ids on the host
    _, inv, _, _ = moe_permute_plan(topk_ids, _MAX_EXPERTS, want_int64_offsets=False)
    return unpermute_combine(permuted_output, topk_weights, inv, T, K)
