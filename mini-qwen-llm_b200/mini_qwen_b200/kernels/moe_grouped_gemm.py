"""Grouped expert GEMM. Same call as ``mini_qwen/kernels/moe_grouped_gemm.py:115-156``."""
from __future__ import annotations

import torch

from .. import _cabi


def _status_word(dev) -> torch.Tensor:
    return torch.zeros(1, dtype=torch.int32, device=dev)


def _offsets32(expert_offsets: torch.Tensor) -> torch.Tensor:
    return expert_offsets if expert_offsets.dtype == torch.int32 else expert_offsets.to(torch.int32)


def moe_grouped_gemm(
    permuted_hidden: torch.Tensor,   # [num_tokens * top_k, hidden_dim]
    expert_weights: torch.Tensor,    # [num_experts, out_dim, hidden_dim]
    expert_offsets: torch.Tensor,    # [num_experts + 1]
    status: torch.Tensor | None = None,
    zero_init: bool = True,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """``out[s:t] = permuted_hidden[s:t] @ expert_weights[e].T`` per expert, fp32 accumulation.

    Unlike the reference there is no CPU branch (``moe_grouped_gemm.py:124-125``): CPU tensors
    are an error.  Rows covered by no expert are zero, as in the reference's oracle.
    ``expert_offsets`` may hold a multiple G of E groups (+1): group g then uses ``expert_weights[g % E]``
    (rows received under expert parallelism are grouped by source rank, then local expert).
    ``status`` (int32 [1], optional) receives device-side error bits (a bounded wait that ran out).
    ``zero_init=False`` skips the zero fill when the offsets are known to cover every row."""
    _cabi.require_cuda(permuted_hidden, expert_weights, expert_offsets)
    assert permuted_hidden.dim() == 2 and expert_weights.dim() == 3
    assert permuted_hidden.dtype == expert_weights.dtype, "activations and weights must share a dtype"
    E, D, H = expert_weights.shape
    groups = expert_offsets.numel() - 1       # == E, or G * E under expert parallelism (group g -> weight g % E)
    assert permuted_hidden.shape[1] == H and groups >= E and groups % E == 0
    a = permuted_hidden.contiguous()
    w = expert_weights.contiguous()
    S = a.shape[0]
    if out is None:
        out = (torch.zeros if zero_init else torch.empty)(S, D, dtype=a.dtype, device=a.device)
    assert out.is_contiguous() and tuple(out.shape) == (S, D) and out.dtype == a.dtype
    if status is None:
        status = _status_word(a.device)
    rc = _cabi.load().mq_grouped_gemm(_cabi.ptr(a), _cabi.ptr(w), _cabi.ptr(_offsets32(expert_offsets)), S, groups, E, D, H,
                                      _cabi.dtype_code(a), _cabi.ptr(out), _cabi.ptr(status),
                                      _cabi.stream_ptr(a.device))
    _cabi.check(rc, "mq_grouped_gemm")
    _cabi.count_launches(1 if S else 0)
    return out


def moe_grouped_swiglu(permuted_hidden: torch.Tensor, gate_up_weights: torch.Tensor,
                       expert_offsets: torch.Tensor, status: torch.Tensor | None = None,
                       zero_init: bool = True) -> torch.Tensor:
    """``h[s:t] = silu(x @ Wg[e].T) * (x @ Wu[e].T)`` with a rounding to the tensor dtype after
    every op, as the per-expert module path rounds.  ``gate_up_weights`` is [E, 2I, H]: gate
    rows first, then up rows."""
    _cabi.require_cuda(permuted_hidden, gate_up_weights, expert_offsets)
    E, I2, H = gate_up_weights.shape
    groups = expert_offsets.numel() - 1
    assert I2 % 2 == 0 and permuted_hidden.shape[1] == H and groups >= E and groups % E == 0
    a = permuted_hidden.contiguous()
    gate_up_weights = gate_up_weights.contiguous()
    S = a.shape[0]
    h = (torch.zeros if zero_init else torch.empty)(S, I2 // 2, dtype=a.dtype, device=a.device)
    if status is None:
        status = _status_word(a.device)
    rc = _cabi.load().mq_grouped_swiglu(_cabi.ptr(a), _cabi.ptr(gate_up_weights), _cabi.ptr(_offsets32(expert_offsets)),
                                        S, groups, E, I2 // 2, H, _cabi.dtype_code(a), _cabi.ptr(h), _cabi.ptr(status),
                                        _cabi.stream_ptr(a.device))
    _cabi.check(rc, "mq_grouped_swiglu")
    _cabi.count_launches(1 if S else 0)
    return h


def gather_swiglu_supported(hidden_states: torch.Tensor, gate_up_weights: torch.Tensor) -> bool:
    """True when :func:`moe_grouped_swiglu_gather` covers these tensors (bf16, H % 64 == 0, I % 128 == 0)."""
    E, I2, H = gate_up_weights.shape
    return (hidden_states.dtype == torch.bfloat16 and gate_up_weights.dtype == torch.bfloat16
            and H % 64 == 0 and (I2 // 2) % 128 == 0 and hidden_states.numel() < 2 ** 32)


def moe_grouped_swiglu_gather(hidden_states: torch.Tensor, perm: torch.Tensor, top_k: int,
                              gate_up_weights: torch.Tensor, expert_offsets: torch.Tensor,
                              status: torch.Tensor | None = None) -> torch.Tensor:
    """:func:`moe_grouped_swiglu` on ``hidden_states[perm // top_k]`` without materialising the
    permuted rows: the kernel gathers them itself.  ``hidden_states`` is the unpermuted [T, H].
    ``perm`` may be longer than the slots ``expert_offsets`` covers (a slot table sized for the worst
    case); the result has one row per entry of ``perm``."""
    _cabi.require_cuda(hidden_states, perm, gate_up_weights, expert_offsets)
    E, I2, H = gate_up_weights.shape
    x = hidden_states.contiguous()
    gate_up_weights = gate_up_weights.contiguous()
    T = x.shape[0]
    S = perm.numel()
    assert x.shape[1] == H
    groups = expert_offsets.numel() - 1
    h = torch.empty(S, I2 // 2, dtype=x.dtype, device=x.device)
    if status is None:
        status = _status_word(x.device)
    rc = _cabi.load().mq_grouped_swiglu_gather(_cabi.ptr(x), _cabi.ptr(perm), _cabi.ptr(gate_up_weights),
                                               _cabi.ptr(_offsets32(expert_offsets)), T, top_k, groups, E, I2 // 2, H,
                                               _cabi.dtype_code(x), _cabi.ptr(h), _cabi.ptr(status),
                                               _cabi.stream_ptr(x.device))
    _cabi.check(rc, "mq_grouped_swiglu_gather")
    _cabi.count_launches(1 if S else 0)
    return h


def scatter_gemm_supported(rows: torch.Tensor, expert_weights: torch.Tensor) -> bool:
    """True when :func:`moe_grouped_gemm_scatter` covers these tensors (bf16, K % 64 == 0, N % 128 == 0)."""
    E, N, Kd = expert_weights.shape
    return (rows.dtype == torch.bfloat16 and expert_weights.dtype == torch.bfloat16
            and Kd % 64 == 0 and N % 128 == 0)


def moe_grouped_gemm_scatter(rows: torch.Tensor, expert_weights: torch.Tensor, expert_offsets: torch.Tensor,
                             row_dst: torch.Tensor, dst_bases: torch.Tensor,
                             status: torch.Tensor | None = None) -> None:
    """:func:`moe_grouped_gemm` whose output rows go to one destination each: row r is written to row
    ``row_dst[r] & 0x3FFFFFF`` of the ``[*, N]`` buffer at address ``dst_bases[row_dst[r] >> 26]`` (int64
    device addresses, possibly in a peer GPU's memory).  Nothing is returned; the caller owns the
    destination buffers and the ordering with their readers."""
    _cabi.require_cuda(rows, expert_weights, expert_offsets, row_dst, dst_bases)
    E, N, Kd = expert_weights.shape
    a = rows.contiguous()
    S = a.shape[0]
    groups = expert_offsets.numel() - 1
    assert row_dst.dtype == torch.int32 and row_dst.numel() >= S and dst_bases.dtype == torch.int64
    assert a.shape[1] == Kd
    if status is None:
        status = _status_word(a.device)
    rc = _cabi.load().mq_grouped_gemm_scatter(_cabi.ptr(a), _cabi.ptr(expert_weights),
                                              _cabi.ptr(_offsets32(expert_offsets)), _cabi.ptr(row_dst),
                                              _cabi.ptr(dst_bases), S, groups, E, N, Kd, _cabi.dtype_code(a),
                                              _cabi.ptr(status), _cabi.stream_ptr(a.device))
    _cabi.check(rc, "mq_grouped_gemm_scatter")
    _cabi.count_launches(1 if S else 0)
