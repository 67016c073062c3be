"""Int4 <-> int32 packing, the storage format of W4A16 weights and zero points.

Eight unsigned 4-bit values share one int32 along the LAST axis; value ``i`` of a word sits
in bits ``[4i, 4i+4)``, so the lowest index is the lowest nibble.  Same format as the
reference's ``mini_qwen/quantization/packing.py:11-39`` (a word whose top nibble is >= 8
is a negative int32).  These are load-time format helpers; they run on whatever device the
tensor lives on.
"""
from __future__ import annotations

import torch
from torch import Tensor


def pack_int4(x: Tensor) -> Tensor:
    """[..., K] integers in 0..15 -> [..., K // 8] int32."""
    assert x.shape[-1] % 8 == 0, f"last dimension must be a multiple of 8, got {x.shape[-1]}"
    nib = x.to(torch.int64).reshape(*x.shape[:-1], x.shape[-1] // 8, 8) & 0xF
    word = nib[..., 0].clone()
    for i in range(1, 8):
        word |= nib[..., i] << (4 * i)
    # bit 31 is the sign bit of the stored int32
    return torch.where(word >= 2 ** 31, word - 2 ** 32, word).to(torch.int32)


def unpack_int4(packed: Tensor) -> Tensor:
    """[..., K // 8] int32 -> [..., K] int32 in 0..15 (inverse of :func:`pack_int4`)."""
    p = packed.to(torch.int32)
    nib = torch.stack([(p >> (4 * i)) & 0xF for i in range(8)], dim=-1)
    return nib.reshape(*packed.shape[:-1], packed.shape[-1] * 8)
