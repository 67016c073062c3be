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


ROUTE_SMALL_MAX_TOKENS, ROUTE_SMALL_MAX_EXPERTS = 64, 256


def route_small_workspace(num_experts: int, device) -> torch.Tensor:
    """A zero-filled workspace for :func:`moe_route_small` (any batch up to 64 tokens).  The kernel leaves it
    ready for the next call, so it is filled once; calls that share one must be stream-ordered."""
    nbytes = _cabi.load().mq_route_small_workspace_bytes(ROUTE_SMALL_MAX_TOKENS, num_experts)
    return torch.zeros(nbytes, dtype=torch.uint8, device=device)


def route_small_supported(num_tokens: int, num_experts: int, top_k: int) -> bool:
    return (0 < num_tokens <= ROUTE_SMALL_MAX_TOKENS and num_experts <= ROUTE_SMALL_MAX_EXPERTS and top_k <= 32
            and num_tokens * top_k <= 2048)


def moe_route_small(hidden_states: torch.Tensor, router_weight: torch.Tensor, top_k: int = 8,
                    bias: Optional[torch.Tensor] = None, renormalize: bool = False, prepare: bool = False,
                    workspace: Optional[torch.Tensor] = None):
    """Router, top-k, permute plan and (``prepare``) the W4A16 kernels' activation preparation in one launch,
    for at most 64 tokens: what ``moe_router`` + ``moe_permute_plan`` (+ ``w4a16_tc_prep``) do in three or four.

    Returns ``(ids32 [T,K], weights fp32 [T,K], perm int32 [S], inv int32 [S], offsets32 int32 [E+1], xp, xs)``;
    ``xp`` ([T,H], token rows in the k order the W4A16 kernels multiply in) and ``xs`` (fp32 [T,32], their
    sums over every 128 k) are None unless ``prepare``: True or "bf16" for bf16 rows, "f16" for fp16 rows scaled
    by their power of two (the stream kernels' faster format, H <= 3968).  ``workspace``: a tensor from
    :func:`route_small_workspace` to reuse across calls (a fresh one is made otherwise)."""
    _cabi.require_cuda(hidden_states, router_weight, bias)
    T, H = hidden_states.shape
    E = router_weight.shape[0]
    assert router_weight.shape[1] == H and route_small_supported(T, E, top_k)
    x, w = hidden_states.contiguous(), router_weight.contiguous()
    if bias is not None:
        bias = bias.to(torch.float32).contiguous()
    dev = x.device
    lib = _cabi.load()
    ws = workspace if workspace is not None else route_small_workspace(E, dev)
    ws_bytes = ws.numel()
    assert ws.is_cuda and ws.dtype == torch.uint8 and ws_bytes >= lib.mq_route_small_workspace_bytes(T, E)
    S = T * top_k
    ids32 = torch.empty(T, top_k, dtype=torch.int32, device=dev)
    wts = torch.empty(T, top_k, dtype=torch.float32, device=dev)
    perm = torch.empty(S, dtype=torch.int32, device=dev)
    inv = torch.empty(S, dtype=torch.int32, device=dev)
    off32 = torch.empty(E + 1, dtype=torch.int32, device=dev)
    xp = xs = None
    fmt = 0
    if prepare:
        fmt = 2 if prepare == "f16" else 1
        assert x.dtype == torch.bfloat16 and H % 128 == 0 and H <= (3968 if fmt == 2 else 4096)
        xp = torch.empty(T, H, dtype=torch.float16 if fmt == 2 else torch.bfloat16, device=dev)
        xs = torch.empty(T, 32, dtype=torch.float32, device=dev)
    rc = lib.mq_route_small(_cabi.ptr(x), _cabi.dtype_code(x), _cabi.ptr(w), _cabi.dtype_code(w), _cabi.ptr(bias),
                            T, H, E, top_k, int(renormalize), _cabi.ptr(ws), ws_bytes, None, _cabi.ptr(ids32),
                            _cabi.ptr(wts), _cabi.ptr(perm), _cabi.ptr(inv), None, _cabi.ptr(off32),
                            _cabi.ptr(xp), _cabi.ptr(xs), fmt, _cabi.stream_ptr(dev))
    _cabi.check(rc, "mq_route_small")
    _cabi.count_launches(1)
    return ids32, wts, perm, inv, off32, xp, xs
