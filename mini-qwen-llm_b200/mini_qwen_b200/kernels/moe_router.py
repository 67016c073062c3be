"""Top-k router. Same call as the reference's ``mini_qwen/kernels/moe_router.py:7-22``."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _cabi


def moe_router(
    hidden_states: torch.Tensor,   # [num_tokens, hidden_dim]
    router_weight: torch.Tensor,   # [num_experts, hidden_dim]
    top_k: int = 8,
    bias: Optional[torch.Tensor] = None,
    renormalize: bool = False,
    return_int32_ids: bool = False,
) -> Tuple[torch.Tensor, ...]:
    """fp32 logits, fp32 softmax, the ``top_k`` largest scores in descending order; equal
    scores go to the lower expert id.

    Returns ``(topk_ids int64 [T, K], topk_weights fp32 [T, K])``.  The weights are the raw
    softmax scores unless ``renormalize`` (the block divides by their sum, as the reference's
    ``layers/moe.py:55-56`` does).  ``bias`` (fp32 [E]) is added to the logits.  With
    ``return_int32_ids`` a third tensor with the ids as int32 is returned as well.
    """
    _cabi.require_cuda(hidden_states, router_weight, bias)
    assert hidden_states.dim() == 2 and router_weight.dim() == 2, "expected [T, H] and [E, H]"
    T, H = hidden_states.shape
    E = router_weight.shape[0]
    assert router_weight.shape[1] == H, "hidden size of states and router weight differ"
    assert 1 <= top_k <= E, f"top_k={top_k} must be in [1, num_experts={E}]"
    x = hidden_states.contiguous()
    w = router_weight.contiguous()
    if bias is not None:
        bias = bias.to(torch.float32).contiguous()
        assert bias.numel() == E
    dev = x.device
    ids = torch.empty(T, top_k, dtype=torch.int64, device=dev)
    ids32 = torch.empty(T, top_k, dtype=torch.int32, device=dev) if return_int32_ids else None
    wts = torch.empty(T, top_k, dtype=torch.float32, device=dev)
    lib = _cabi.load()
    ws_bytes = lib.mq_router_workspace_bytes(T, H, E)
    logits = torch.empty(ws_bytes // 4, dtype=torch.float32, device=dev)
    rc = lib.mq_router_topk(_cabi.ptr(x), _cabi.dtype_code(x), _cabi.ptr(w), _cabi.dtype_code(w), _cabi.ptr(bias),
                            T, H, E, top_k, int(renormalize), _cabi.ptr(logits), ws_bytes, _cabi.ptr(ids), _cabi.ptr(ids32),
                            _cabi.ptr(wts), _cabi.stream_ptr(dev))
    _cabi.check(rc, "mq_router_topk")
    _cabi.count_launches(2 if T else 0)
    return (ids, wts, ids32) if return_int32_ids else (ids, wts)
