"""Expert-sorted permute. Same call as the reference's ``mini_qwen/kernels/moe_permute.py:10-33``."""
from __future__ import annotations

from typing import Tuple

import torch

from .. import _cabi


def moe_permute_plan(topk_ids: torch.Tensor, num_experts: int, want_int64_offsets: bool = True):
    """Stable counting sort of the T*K slots by expert id.

    Returns ``(perm int32 [S], inv int32 [S], offsets32 int32 [E+1], offsets64 int64 [E+1] | None)``:
    ``perm[p]`` is the flat slot ``t*K+k`` stored at sorted position ``p``, ``inv`` its inverse.
    """
    _cabi.require_cuda(topk_ids)
    assert topk_ids.dim() == 2, "topk_ids must be [T, K]"
    assert topk_ids.dtype in (torch.int64, torch.int32), "topk_ids must be int64 or int32"
    T, K = topk_ids.shape
    S = T * K
    ids = topk_ids.contiguous()
    dev = ids.device
    lib = _cabi.load()
    perm = torch.empty(S, dtype=torch.int32, device=dev)
    inv = torch.empty(S, dtype=torch.int32, device=dev)
    off32 = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
    off64 = torch.empty(num_experts + 1, dtype=torch.int64, device=dev) if want_int64_offsets else None
    ws_bytes = lib.mq_permute_workspace_bytes(S, num_experts)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    rc = lib.mq_permute_plan(_cabi.ptr(ids), int(ids.dtype == torch.int64), T, K, num_experts, _cabi.ptr(perm),
                             _cabi.ptr(inv), _cabi.ptr(off64), _cabi.ptr(off32), _cabi.ptr(ws), ws_bytes,
                             _cabi.stream_ptr(dev))
    _cabi.check(rc, "mq_permute_plan")
    _cabi.count_launches(1 if S <= 2048 else 3)
    return perm, inv, off32, off64


def gather_rows(hidden_states: torch.Tensor, perm: torch.Tensor, top_k: int) -> torch.Tensor:
    """``out[p] = hidden_states[perm[p] // top_k]``."""
    x = hidden_states.contiguous()
    S, H = perm.numel(), x.shape[1]
    out = torch.empty(S, H, dtype=x.dtype, device=x.device)
    rc = _cabi.load().mq_gather_rows(_cabi.ptr(x), _cabi.dtype_code(x), _cabi.ptr(perm), S, top_k, H,
                                     _cabi.ptr(out), _cabi.stream_ptr(x.device))
    _cabi.check(rc, "mq_gather_rows")
    _cabi.count_launches(1 if S else 0)
    return out


def moe_permute(
    hidden_states: torch.Tensor,  # [num_tokens, hidden_dim]
    topk_ids: torch.Tensor,       # [num_tokens, top_k]
    num_experts: int,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(permuted_hidden [T*K, H], expert_offsets int64 [E+1])``; rows
    ``expert_offsets[e]:expert_offsets[e+1]`` belong to expert ``e`` in ascending slot order."""
    _cabi.require_cuda(hidden_states, topk_ids)
    assert hidden_states.dim() == 2 and hidden_states.shape[0] == topk_ids.shape[0]
    perm, _, _, off64 = moe_permute_plan(topk_ids, num_experts)
    return gather_rows(hidden_states, perm, topk_ids.shape[1]), off64
