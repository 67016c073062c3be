"""RMSNorm on the CUDA kernel.  Same module as ``mini_qwen/model/layers/rms_norm.py:5-18``: one ``weight``
parameter of ``hidden_size`` ones, ``forward`` normalises in fp32, casts to the input dtype, then scales."""
from __future__ import annotations

import torch
import torch.nn as nn

from ... import _cabi


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``weight * (x.float() * rsqrt(mean(x.float()**2, -1) + eps)).to(x.dtype)`` over the last dimension."""
    _cabi.require_cuda(x, weight)
    H = x.shape[-1]
    if weight.shape != (H,) or weight.dtype != x.dtype:
        raise ValueError("weight must be [hidden] of the input's dtype")
    rows = x.reshape(-1, H)
    if not rows.is_contiguous():
        rows = rows.contiguous()
    out = torch.empty_like(rows)
    T = rows.shape[0]
    rc = _cabi.load().mq_rms_norm(_cabi.ptr(rows), _cabi.dtype_code(rows), _cabi.ptr(weight.contiguous()), float(eps),
                                  T, H, _cabi.ptr(out), _cabi.stream_ptr(x.device))
    _cabi.check(rc, "mq_rms_norm")
    _cabi.count_launches(1 if T else 0)
    return out.reshape(x.shape)


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return rms_norm(x, self.weight.data, self.eps)
