"""The router entry point that allocates nothing (mq_router_topk_static), called through the C ABI.

It exists for callers that cannot allocate device memory when they call: code running where the
CUDA allocator is off limits, a host runtime that owns only its input/output buffers, a process
whose pool already holds the device.  Its scratch is an array inside the library image, so this
test checks that the built-in array really is what the kernels use: results must equal those of
the entry point with a caller-provided workspace, bit for bit, on two calls in a row (the second
call finds the first call's leftovers in the shared array).

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes

import pytest
import torch

from mini_qwen_b200 import _cabi

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _route(lib, static, x, w, K, renorm):
    T, H = x.shape
    E = w.shape[0]
    ids = torch.full((T, K), -1, dtype=torch.int64, device=DEV)
    ids32 = torch.full((T, K), -1, dtype=torch.int32, device=DEV)
    wts = torch.full((T, K), float("nan"), dtype=torch.float32, device=DEV)
    stream = _cabi.stream_ptr(x.device)
    args = (_cabi.ptr(x), _cabi.dtype_code(x), _cabi.ptr(w), _cabi.dtype_code(w), None, T, H, E, K, int(renorm))
    if static:
        rc = lib.mq_router_topk_static(*args, _cabi.ptr(ids), _cabi.ptr(ids32), _cabi.ptr(wts), stream)
    else:
        nbytes = lib.mq_router_workspace_bytes(T, H, E)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
        rc = lib.mq_router_topk(*args, _cabi.ptr(ws), nbytes, _cabi.ptr(ids), _cabi.ptr(ids32), _cabi.ptr(wts), stream)
    assert rc == 0, lib.mq_status_string(rc).decode()
    torch.cuda.synchronize()
    return ids, ids32, wts


def test_static_router_matches_workspace_router_twice_in_a_row():
    lib = _cabi.load()
    g = torch.Generator().manual_seed(123)
    # first call: a prefill-sized batch (tiled kernel, several K slices); second: a decode batch (other
    # kernel, smaller footprint) that finds the first call's logits still in the array
    # third: 9000 tokens, inside the range (8193..9440) where the logits are kept in two K slices and take
    # more room than at 16384 tokens
    shapes = [(4096, 2048, 128, 8, torch.bfloat16, True), (7, 2048, 128, 8, torch.bfloat16, False),
              (9000, 2048, 128, 8, torch.bfloat16, True)]
    for T, H, E, K, dt, renorm in shapes:
        x = torch.randn(T, H, generator=g).to(dt).to(DEV)
        w = (torch.randn(E, H, generator=g) * 0.02).to(dt).to(DEV)
        got = _route(lib, True, x, w, K, renorm)
        want = _route(lib, False, x, w, K, renorm)
        assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])   # ids: bit-exact
        assert torch.equal(got[2], want[2])                                     # same kernels, same bits
        assert int(got[0].min()) >= 0 and bool(torch.isfinite(got[2]).all())


def test_static_router_rejects_oversized_requests():
    lib = _cabi.load()
    # 32768 tokens x 128 experts x 4 bytes is beyond the 10 MiB array: refused before any launch
    rc = lib.mq_router_topk_static(None, 1, None, 1, None, 32768, 2048, 128, 8, 0, None, None, None, None)
    assert rc == 6
    assert "10 MiB" in lib.mq_status_string(rc).decode()
