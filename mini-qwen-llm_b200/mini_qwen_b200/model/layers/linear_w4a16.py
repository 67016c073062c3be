"""W4A16 linear layer with the interface of the reference's
``mini_qwen/model/layers/linear_w4a16.py:8-106`` (buffers ``qweight/scales/qzeros``,
``from_float``, ``from_gptq``)."""
from __future__ import annotations

import torch
import torch.nn as nn

from ...kernels.w4a16_gemm import w4a16_gemm
from ...quantization.awq import _per_group_minmax_quantize
from ...quantization.packing import pack_int4, unpack_int4


class LinearW4A16(nn.Module):
    """``y = x @ W`` with ``W[k, n] = (q[k, n] - z[k // g, n]) * s[k // g, n]``, x and y bf16.

    Buffers: ``qweight`` int32 [K/8, N] (8 values per word along K), ``scales`` bf16 [K/g, N],
    ``qzeros`` int32 [K/g, N/8] (8 values per word along N).
    """

    def __init__(self, in_features: int, out_features: int, group_size: int = 128):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.group_size = group_size
        groups = in_features // group_size
        self.register_buffer("qweight", torch.zeros(in_features // 8, out_features, dtype=torch.int32))
        self.register_buffer("scales", torch.zeros(groups, out_features, dtype=torch.bfloat16))
        self.register_buffer("qzeros", torch.zeros(groups, out_features // 8, dtype=torch.int32))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        y = w4a16_gemm(x.reshape(-1, self.in_features), self.qweight, self.scales, self.qzeros, self.group_size)
        return y.reshape(*lead, self.out_features)

    @classmethod
    def from_float(cls, linear: nn.Linear, group_size: int = 128) -> "LinearW4A16":
        """Min-max quantise an ``nn.Linear`` (weight [N, K]); the new layer lives on the CPU/device
        of the quantiser's outputs, as in the reference (callers move it)."""
        w = linear.weight.data.float().T.contiguous()      # [K, N]
        K, N = w.shape
        assert K % group_size == 0, f"K={K} is not divisible by group_size={group_size}"
        assert N % 8 == 0, f"N={N} is not a multiple of 8"
        qweight, scales, qzeros = _per_group_minmax_quantize(w, group_size)
        layer = cls(K, N, group_size)
        layer.qweight.copy_(qweight)
        layer.scales.copy_(scales)
        layer.qzeros.copy_(qzeros)
        return layer

    @classmethod
    def from_gptq(cls, qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor,
                  group_size: int = 128, zero_plus_one: bool = True) -> "LinearW4A16":
        """Adopt GPTQ (v1) tensors: ``qweight`` [K/8, N], ``qzeros`` [G, N/8], ``scales`` [G, N].

        GPTQ v1 stores the zero point minus one.  With ``zero_plus_one`` the stored value is
        incremented and clamped to 0..15 (a stored 15 stays 15, it does not wrap), then
        repacked; scales are rounded to bf16.
        """
        K, N = qweight.shape[0] * 8, qweight.shape[1]
        layer = cls(K, N, group_size)
        layer.qweight.copy_(qweight.to(torch.int32))
        layer.scales.copy_(scales.to(torch.bfloat16))
        zeros = qzeros.to(torch.int32)
        if zero_plus_one:
            zeros = pack_int4((unpack_int4(zeros) + 1).clamp(0, 15))
        layer.qzeros.copy_(zeros)
        return layer

    def extra_repr(self) -> str:
        return f"in={self.in_features}, out={self.out_features}, group_size={self.group_size}"
