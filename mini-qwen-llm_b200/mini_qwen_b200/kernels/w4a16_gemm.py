"""W4A16 GEMM. Same call as the reference's ``mini_qwen/kernels/w4a16_gemm.py:194-247``.

# === FROZEN SIGNATURE (the reference's, kept) ===
# def w4a16_gemm(
#     x:          [M, K], bf16
#     qweight:    [K // 8, N], int32 (packed int4, nibble i of qweight[j,n] = weight[8j+i,n])
#     scales:     [K // group_size, N], bf16
#     qzeros:     [K // group_size, N // 8], int32 (packed int4 along N)
#     group_size: int = 128
# ) -> [M, N], bf16
"""
from __future__ import annotations

import torch

from .. import _cabi


_single_offsets: dict = {}   # (M, device) -> int32 [0, M]; a single linear is a one-expert group


def _offsets32(expert_offsets: torch.Tensor) -> torch.Tensor:
    """The kernels read int32 offsets; ``moe_permute`` returns int64 ones, as the reference does."""
    assert expert_offsets.is_cuda, "w4a16 kernels run on CUDA tensors only"
    off = expert_offsets if expert_offsets.dtype == torch.int32 else expert_offsets.to(torch.int32)
    return off.contiguous()


def _check_w4(x, qweight, scales, qzeros, group_size, E, prepared_f16=False):
    assert x.is_cuda and qweight.is_cuda, "w4a16 kernels run on CUDA tensors only"
    assert qweight.is_contiguous() and scales.is_contiguous() and qzeros.is_contiguous(), \
        "qweight, scales and qzeros must be contiguous (the kernels index them as dense expert-major stacks)"
    assert x.dtype == (torch.float16 if prepared_f16 else torch.bfloat16), "activations must be bfloat16"
    assert qweight.dtype == torch.int32 and qzeros.dtype == torch.int32 and scales.dtype == torch.bfloat16
    K = x.shape[-1]
    N = qweight.shape[-1]
    assert qweight.shape[-2] * 8 == K, "qweight must be [K // 8, N]"
    assert K % group_size == 0, f"K={K} must be divisible by group_size={group_size}"
    assert N % 8 == 0, f"N={N} must be a multiple of 8"
    assert group_size % 32 == 0, "group_size must be a multiple of 32"
    G = K // group_size
    assert tuple(scales.shape[-2:]) == (G, N) and tuple(qzeros.shape[-2:]) == (G, N // 8)
    return K, N


def w4a16_grouped_gemm(x, qweight, scales, qzeros, expert_offsets, group_size: int = 128,
                       zero_init: bool = True, out: torch.Tensor | None = None) -> torch.Tensor:
    """Rows ``offsets[e]:offsets[e+1]`` of x times the dequantised weight of expert e.
    qweight [E, K/8, N], scales [E, K/g, N], qzeros [E, K/g, N/8], offsets int32 [E+1]."""
    E = qweight.shape[0]
    K, N = _check_w4(x, qweight, scales, qzeros, group_size, E)
    expert_offsets = _offsets32(expert_offsets)
    groups = expert_offsets.numel() - 1       # E, or G * E (group g -> weight set g % E)
    assert groups >= E and groups % E == 0
    x = x.contiguous()
    S = x.shape[0]
    if out is None:
        out = (torch.zeros if zero_init else torch.empty)(S, N, dtype=torch.bfloat16, device=x.device)
    assert out.is_contiguous() and tuple(out.shape) == (S, N) and out.dtype == torch.bfloat16
    rc = _cabi.load().mq_w4a16_grouped_gemm(_cabi.ptr(x), _cabi.ptr(qweight), _cabi.ptr(scales), _cabi.ptr(qzeros),
                                            _cabi.ptr(expert_offsets), S, groups, E, N, K, group_size, _cabi.ptr(out),
                                            _cabi.stream_ptr(x.device))
    _cabi.check(rc, "mq_w4a16_grouped_gemm")
    _cabi.count_launches(1 if S else 0)
    return out


def w4a16_grouped_swiglu(x, gate, up, expert_offsets, group_size: int = 128, zero_init: bool = True) -> torch.Tensor:
    """Fused gate/up W4A16 projections + SwiGLU; gate and up are (qweight, scales, qzeros) stacks."""
    E = gate[0].shape[0]
    K, N = _check_w4(x, *gate, group_size, E)
    _check_w4(x, *up, group_size, E)
    expert_offsets = _offsets32(expert_offsets)
    groups = expert_offsets.numel() - 1
    assert groups >= E and groups % E == 0
    x = x.contiguous()
    S = x.shape[0]
    h = (torch.zeros if zero_init else torch.empty)(S, N, dtype=torch.bfloat16, device=x.device)
    rc = _cabi.load().mq_w4a16_grouped_swiglu(_cabi.ptr(x), _cabi.ptr(gate[0]), _cabi.ptr(gate[1]), _cabi.ptr(gate[2]),
                                              _cabi.ptr(up[0]), _cabi.ptr(up[1]), _cabi.ptr(up[2]),
                                              _cabi.ptr(expert_offsets), S, groups, E, N, K, group_size, _cabi.ptr(h),
                                              _cabi.stream_ptr(x.device))
    _cabi.check(rc, "mq_w4a16_grouped_swiglu")
    _cabi.count_launches(1 if S else 0)
    return h


def w4a16_gemm(
    x: torch.Tensor,
    qweight: torch.Tensor,
    scales: torch.Tensor,
    qzeros: torch.Tensor,
    group_size: int = 128,
) -> torch.Tensor:
    """``x @ dequant(qweight)`` with ``W[k,n] = (q[k,n] - z[k//g,n]) * s[k//g,n]``; returns bf16 [M, N]."""
    assert x.dim() == 2 and qweight.dim() == 2
    M = x.shape[0]
    key = (M, x.device)
    offsets = _single_offsets.get(key)
    if offsets is None:
        if len(_single_offsets) > 256:
            _single_offsets.clear()
        offsets = _single_offsets[key] = torch.tensor([0, M], dtype=torch.int32, device=x.device)
    return w4a16_grouped_gemm(x, qweight.contiguous().unsqueeze(0), scales.contiguous().unsqueeze(0),
                              qzeros.contiguous().unsqueeze(0), offsets, group_size, zero_init=False)


# ---- prepared-activation forms of the stream kernel (the block's decode path) ------------------

def w4a16_stream_supported(hidden: int, out_features: int, group_size: int, groups: int) -> bool:
    """Shapes the TMA-staged stream kernel covers with prepared activations."""
    return (group_size == 128 and hidden % 128 == 0 and hidden <= 4096 and out_features % 32 == 0
            and groups <= 384)


def w4a16_stream_swiglu(xp, xs, gate, up, expert_offsets, group_size: int = 128, x_shuffled: bool = True,
                        shuffle_out: bool = True, status: torch.Tensor | None = None,
                        perm: torch.Tensor | None = None, top_k: int = 1) -> torch.Tensor:
    """Fused gate/up + SwiGLU on prepared activations (``w4a16_tc_prep``): ``xp`` the expert-sorted rows in the
    shuffled k order, ``xs`` their group sums (or None).  With ``shuffle_out`` the result's columns are in the
    shuffled order, ready for :func:`w4a16_stream_gemm` with ``x_shuffled=True``.  With ``perm`` (int32 [S]),
    ``xp``/``xs`` hold one row per token and sorted row p is row ``perm[p] // top_k`` (``moe_route_small``).
    ``xp`` of dtype float16 is the row-scaled fp16 format (``w4a16_tc_prep(..., f16=True)``)."""
    E = gate[0].shape[0]
    f16 = xp.dtype == torch.float16
    assert not f16 or (x_shuffled and xs is not None)
    K, N = _check_w4(xp, *gate, group_size, E, f16)
    _check_w4(xp, *up, group_size, E, f16)
    expert_offsets = _offsets32(expert_offsets)
    groups = expert_offsets.numel() - 1
    assert xp.is_contiguous() and (xs is None or (xs.is_contiguous() and xs.dtype == torch.float32))
    S = xp.shape[0] if perm is None else perm.numel()
    if perm is not None:
        assert perm.dtype == torch.int32 and perm.is_contiguous() and top_k >= 1
    h = torch.empty(S, N, dtype=torch.bfloat16, device=xp.device)
    rc = _cabi.load().mq_w4a16_stream_swiglu(
        _cabi.ptr(xp), _cabi.ptr(xs), 2 if f16 else (1 if x_shuffled else 0), _cabi.ptr(perm), top_k,
        _cabi.ptr(gate[0]), _cabi.ptr(gate[1]), _cabi.ptr(gate[2]),
        _cabi.ptr(up[0]), _cabi.ptr(up[1]), _cabi.ptr(up[2]), _cabi.ptr(expert_offsets), S, groups, E, N, K, group_size,
        1 if shuffle_out else 0, _cabi.ptr(h), _cabi.ptr(status), _cabi.stream_ptr(xp.device))
    _cabi.check(rc, "mq_w4a16_stream_swiglu")
    _cabi.count_launches(1 if S else 0)
    return h


def w4a16_stream_gemm(xp, xs, qweight, scales, qzeros, expert_offsets, group_size: int = 128, x_shuffled: bool = True,
                      status: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """One W4A16 projection per group on prepared activations; natural column order."""
    E = qweight.shape[0]
    f16 = xp.dtype == torch.float16
    assert not f16 or (x_shuffled and xs is not None)
    K, N = _check_w4(xp, qweight, scales, qzeros, group_size, E, f16)
    expert_offsets = _offsets32(expert_offsets)
    groups = expert_offsets.numel() - 1
    assert xp.is_contiguous() and (xs is None or (xs.is_contiguous() and xs.dtype == torch.float32))
    S = xp.shape[0]
    if out is None:
        out = torch.empty(S, N, dtype=torch.bfloat16, device=xp.device)
    assert out.is_contiguous() and tuple(out.shape) == (S, N) and out.dtype == torch.bfloat16
    rc = _cabi.load().mq_w4a16_stream_gemm(
        _cabi.ptr(xp), _cabi.ptr(xs), 2 if f16 else (1 if x_shuffled else 0), _cabi.ptr(qweight), _cabi.ptr(scales),
        _cabi.ptr(qzeros),
        _cabi.ptr(expert_offsets), S, groups, E, N, K, group_size, _cabi.ptr(out), _cabi.ptr(status),
        _cabi.stream_ptr(xp.device))
    _cabi.check(rc, "mq_w4a16_stream_gemm")
    _cabi.count_launches(1 if S else 0)
    return out


# ---- tcgen05 path for decode-size groups ------------------------------------------------------

def w4a16_tc_supported(hidden: int, out_features: int, group_size: int) -> bool:
    """Shapes the tensor-memory kernel covers: group 128, K a multiple of 128 up to 4096, N a multiple of 128."""
    return group_size == 128 and hidden % 128 == 0 and hidden <= 4096 and out_features % 128 == 0


def w4a16_tc_prep(x: torch.Tensor, perm: torch.Tensor | None = None, top_k: int = 1, shuffle: bool = True,
                  want_rows: bool = True, f16: bool = False):
    """Prepared activations for the stream and tensor-memory kernels: (xp, xs).  xp [S, K] = the (optionally
    gathered) rows with the k order 0,4,1,5,2,6,3,7 inside every 8; xs fp32 [S, 32] = per-row sums over every
    128 k.  ``f16`` (stream kernels only, K <= 3968): xp is float16, every row scaled by the power of two that
    puts its largest magnitude into [2^14, 2^15); xs holds the sums of the scaled values and, in column 31, the
    inverse of the row's factor."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2
    x = x.contiguous()
    S = perm.numel() if perm is not None else x.shape[0]
    K = x.shape[1]
    assert not f16 or (shuffle and K <= 3968)
    xp = torch.empty(S, K, dtype=torch.float16 if f16 else torch.bfloat16, device=x.device) if want_rows else None
    xs = torch.empty(S, 32, dtype=torch.float32, device=x.device)
    rc = _cabi.load().mq_w4a16_tc_prep(_cabi.ptr(x), _cabi.ptr(perm) if perm is not None else None, top_k, S, K,
                                       2 if f16 else (1 if shuffle else 0), _cabi.ptr(xp) if want_rows else None,
                                       _cabi.ptr(xs),
                                       _cabi.stream_ptr(x.device))
    _cabi.check(rc, "mq_w4a16_tc_prep")
    _cabi.count_launches(1 if S else 0)
    return xp, xs


def w4a16_tc_swiglu(xp, xs, gate, up, expert_offsets, group_size: int = 128, status: torch.Tensor | None = None):
    """Fused gate/up + SwiGLU on prepared activations; the result's columns are in the shuffled k order
    (it is the ``xp`` of the down projection)."""
    E = gate[0].shape[0]
    K, N = _check_w4(xp, *gate, group_size, E)
    _check_w4(xp, *up, group_size, E)
    expert_offsets = _offsets32(expert_offsets)
    groups = expert_offsets.numel() - 1
    S = xp.shape[0]
    h = torch.empty(S, N, dtype=torch.bfloat16, device=xp.device)
    rc = _cabi.load().mq_w4a16_tc_swiglu(_cabi.ptr(xp), _cabi.ptr(xs), _cabi.ptr(gate[0]), _cabi.ptr(gate[1]),
                                         _cabi.ptr(gate[2]), _cabi.ptr(up[0]), _cabi.ptr(up[1]), _cabi.ptr(up[2]),
                                         _cabi.ptr(expert_offsets), S, groups, E, N, K, group_size, _cabi.ptr(h),
                                         _cabi.ptr(status) if status is not None else None,
                                         _cabi.stream_ptr(xp.device))
    _cabi.check(rc, "mq_w4a16_tc_swiglu")
    _cabi.count_launches(1 if S else 0)
    return h


def w4a16_tc_gemm(xp, xs, qweight, scales, qzeros, expert_offsets, group_size: int = 128,
                  status: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """One W4A16 projection per group on prepared activations; natural column order."""
    E = qweight.shape[0]
    K, N = _check_w4(xp, qweight, scales, qzeros, group_size, E)
    expert_offsets = _offsets32(expert_offsets)
    groups = expert_offsets.numel() - 1
    S = xp.shape[0]
    if out is None:
        out = torch.empty(S, N, dtype=torch.bfloat16, device=xp.device)
    assert out.is_contiguous() and tuple(out.shape) == (S, N) and out.dtype == torch.bfloat16
    rc = _cabi.load().mq_w4a16_tc_gemm(_cabi.ptr(xp), _cabi.ptr(xs), _cabi.ptr(qweight), _cabi.ptr(scales),
                                       _cabi.ptr(qzeros), _cabi.ptr(expert_offsets), S, groups, E, N, K, group_size,
                                       _cabi.ptr(out), _cabi.ptr(status) if status is not None else None,
                                       _cabi.stream_ptr(xp.device))
    _cabi.check(rc, "mq_w4a16_tc_gemm")
    _cabi.count_launches(1 if S else 0)
    return out
