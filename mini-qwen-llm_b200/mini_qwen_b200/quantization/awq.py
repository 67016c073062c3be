"""Per-group min-max 4-bit quantiser (the reference's ``mini_qwen/quantization/awq.py:14-58``).

It is what ``LinearW4A16.from_float`` and ``Qwen3MoEBlock.quantize_to_w4a16`` use, and the
generator of test data for the W4A16 kernels.  Activation-aware AWQ needs calibration
passes and is a placeholder in the reference too (``awq.py:61-77``).
"""
from __future__ import annotations

import torch
from torch import Tensor

from .packing import pack_int4


def _per_group_minmax_quantize(w: Tensor, group_size: int = 128) -> tuple[Tensor, Tensor, Tensor]:
    """w [K, N] -> (qweight [K//8, N] int32 packed along K, scales [K//g, N] bf16,
    qzeros [K//g, N//8] int32 packed along N).

    Per (group, column): scale = (max - min) / 15 floored at 1e-8, zero = round(-min / scale)
    in 0..15, q = round(w / scale + zero) in 0..15.
    """
    K, N = w.shape
    assert K % group_size == 0, f"K={K} must be divisible by group_size={group_size}"
    assert N % 8 == 0, f"N={N} must be a multiple of 8 (qzeros are packed along N)"
    grp = w.float().reshape(K // group_size, group_size, N)
    w_hi, w_lo = grp.amax(dim=1), grp.amin(dim=1)
    scales = ((w_hi - w_lo) / 15.0).clamp(min=1e-8)
    zeros = (-w_lo / scales).round().clamp(0, 15).to(torch.int32)
    q = (grp / scales.unsqueeze(1) + zeros.unsqueeze(1).float()).round().clamp(0, 15).to(torch.int32)
    qweight = pack_int4(q.reshape(K, N).T).T
    return qweight, scales.to(torch.bfloat16), pack_int4(zeros)


def quantize_awq(model, calibration_data, group_size: int = 128):
    """Activation-aware quantisation is not part of this path (the reference raises too)."""
    raise NotImplementedError(
        "activation-aware AWQ needs calibration forward passes; use _per_group_minmax_quantize "
        "or load offline-quantised GPTQ tensors with LinearW4A16.from_gptq")
