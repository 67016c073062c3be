"""ctypes binding of libmqmoe.so (the C ABI declared in include/mqmoe.h).

There is no fallback: if the library is missing or a call returns a non-zero status, a
RuntimeError / ValueError is raised.  torch only supplies device memory and the stream.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libmqmoe.so"

MQ_F32, MQ_BF16, MQ_F16 = 0, 1, 2
_DTYPES = {torch.float32: MQ_F32, torch.bfloat16: MQ_BF16, torch.float16: MQ_F16}

# name -> (restype, argtypes); kept in the order of include/mqmoe.h
_P, _I, _L = c_void_p, c_int, c_int64
PROTOTYPES = {
    "mq_version": (c_int, []),
    "mq_status_string": (c_char_p, [c_int]),
    "mq_last_cuda_error": (c_char_p, []),
    "mq_router_workspace_bytes": (c_size_t, [_L, _L, _L]),
    "mq_router_topk": (c_int, [_P, _I, _P, _I, _P, _L, _L, _L, _L, _I, _P, c_size_t, _P, _P, _P, _P]),
    "mq_router_topk_static": (c_int, [_P, _I, _P, _I, _P, _L, _L, _L, _L, _I, _P, _P, _P, _P]),
    "mq_route_small_workspace_bytes": (c_size_t, [_L, _L]),
    "mq_route_small": (c_int, [_P, _I, _P, _I, _P, _L, _L, _L, _L, _I, _P, c_size_t, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _P]),
    "mq_permute_workspace_bytes": (c_size_t, [_L, _L]),
    "mq_permute_plan": (c_int, [_P, _I, _L, _L, _L, _P, _P, _P, _P, _P, c_size_t, _P]),
    "mq_gather_rows": (c_int, [_P, _I, _P, _L, _L, _L, _P, _P]),
    "mq_unpermute_combine": (c_int, [_P, _I, _P, _P, _L, _L, _L, _P, _P]),
    "mq_unpermute_combine_residual": (c_int, [_P, _I, _P, _P, _P, _L, _L, _L, _P, _P]),
    "mq_rms_norm": (c_int, [_P, _I, _P, c_float, _L, _L, _P, _P]),
    "mq_grouped_gemm": (c_int, [_P, _P, _P, _L, _L, _L, _L, _L, _I, _P, _P, _P]),
    "mq_grouped_swiglu": (c_int, [_P, _P, _P, _L, _L, _L, _L, _L, _I, _P, _P, _P]),
    "mq_grouped_gemm_scatter": (c_int, [_P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _I, _P, _P]),
    "mq_grouped_swiglu_gather": (c_int, [_P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _I, _P, _P, _P]),
    "mq_stack_tensors": (c_int, [_P, _L, _L, _I, _P, _P]),
    "mq_w4a16_grouped_gemm": (c_int, [_P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _P, _P]),
    "mq_w4a16_grouped_swiglu": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _P, _P]),
    "mq_w4a16_stream_swiglu": (c_int, [_P, _P, _I, _P, _L, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _I, _P, _P, _P]),
    "mq_w4a16_stream_gemm": (c_int, [_P, _P, _I, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _P, _P, _P]),
    "mq_w4a16_tc_prep": (c_int, [_P, _P, _L, _L, _L, _I, _P, _P, _P]),
    "mq_w4a16_tc_gemm": (c_int, [_P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _P, _P, _P]),
    "mq_w4a16_tc_swiglu": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _P, _P, _P]),
    "mq_ep_share_counts": (c_int, [_P, _L, _L, _L, _P, _P]),
    "mq_ep_barrier": (c_int, [_P, _P, _L, _L, _L, _P, _P]),
    "mq_ep_plan": (c_int, [_P, _L, _L, _L, _P, _P, _P]),
    "mq_ep_exchange_plan": (c_int, [_P, _L, _L, _L, _P, _P, _P, _P, _P, _L, _P, _P]),
    "mq_ep_dispatch": (c_int, [_P, _I, _P, _P, _P, _L, _L, _L, _L, _L, _L, _P, _P, _L, _P, _P, _P]),
    "mq_ep_unique_rows": (c_int, [_P, _L, _L, _L, _L, _P, _P]),
    "mq_ep_dispatch_unique": (c_int, [_P, _I, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _L, _P, _P, _P, _L, _P, _P, _P]),
    "mq_ep_combine": (c_int, [_P, _I, _P, _P, _P, _P, _L, _L, _L, _L, _P, _P]),
    "mq_ep_gather_tokens": (c_int, [_P, _I, _L, _L, _L, _L, _P, _P, _P, _L, _P, _P]),
    "mq_ep_send_partials": (c_int, [_P, _I, _P, _P, _P, _L, _L, _L, _L, _L, _L, _L, _P, _P, _P, _P, _L, _P, _P]),
    "mq_ep_sum_partials": (c_int, [_P, _I, _P, _L, _L, _L, _P, _P]),
}

_lib = None
launch_count = 0   # kernels launched through this binding (each wrapper adds what it launched)


def count_launches(n: int) -> None:
    global launch_count
    launch_count += n


def lib_path() -> Path:
    return Path(os.environ.get("MQMOE_LIB", _LIB_PATH))


def load() -> ctypes.CDLL:
    """Loads the library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        path = lib_path()
        if not path.exists():
            raise RuntimeError(
                f"{path} is missing: build it with `python mini-qwen-llm_b200/build.py` "
                "(there is no CPU or PyTorch fallback for these kernels)")
        lib = ctypes.CDLL(str(path))
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(lib, name)   # AttributeError if the symbol is not exported
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {t.dtype}; expected float32, bfloat16 or float16") from None


def ptr(t: torch.Tensor | None):
    return None if t is None else c_void_p(t.data_ptr())


def stream_ptr(device) -> c_void_p:
    return c_void_p(torch.cuda.current_stream(device).cuda_stream)


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("these kernels run on CUDA tensors only; there is no CPU path")


def check(status: int, what: str) -> None:
    if status == 0:
        return
    lib = load()
    msg = lib.mq_status_string(status).decode()
    if status == 4:
        msg += ": " + lib.mq_last_cuda_error().decode()
    exc = ValueError if status in (1, 2, 3, 6) else RuntimeError
    raise exc(f"{what}: {msg} (mq_status {status})")
