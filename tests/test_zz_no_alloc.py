"""The allocation-free decode entry point, called through the C ABI.

Some callers can hand the library nothing but their inputs and outputs: inside a
compiler-planned custom call every buffer is fixed ahead of time and cudaMalloc is
off limits, and the same holds while a device allocator is locked or out of
memory.  ``pjx_attn_decode_splitkv_static`` keeps its per-split partials in a
fixed array inside the library for them.  This file checks it against the
workspace-taking entry point on two calls in a row (the second with other inputs,
shorter sequences and a different split length, so that leftovers of the first
call sit in the shared array), and that oversized calls are refused.

It is collected last on purpose: a run that stops at the first failure has then
already run every other test.
"""

import ctypes as C
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _call_pair(L, q, k, v, lens, sc, split_len):
    """(static entry point, workspace entry point) results for the same inputs."""
    from probjax_b200 import _lib

    dev = q.device
    B, Lq, Hq, D = q.shape
    cap, Hkv, Dv = k.shape[1], k.shape[2], v.shape[3]
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    o_s = torch.empty(B, Lq, Hq, Dv, dtype=q.dtype, device=dev)
    lse_s = torch.empty(B, Hq, Lq, dtype=torch.float32, device=dev)
    rc = L.pjx_attn_decode_splitkv_static(_ptr(q), _ptr(k), _ptr(v), _ptr(lens), _ptr(o_s), _ptr(lse_s),
                                          B, Lq, Hq, Hkv, D, Dv, cap, _lib.PJX_BF16, sc, split_len, stream)
    _lib.check(rc)
    o_w = torch.empty_like(o_s)
    lse_w = torch.empty_like(lse_s)
    need = L.pjx_attn_decode_workspace_bytes(B, Lq, Hq, Hkv, Dv, cap, split_len)
    ws = torch.empty(need, dtype=torch.uint8, device=dev)
    rc = L.pjx_attn_decode_splitkv(_ptr(q), _ptr(k), _ptr(v), _ptr(lens), _ptr(o_w), _ptr(lse_w),
                                   B, Lq, Hq, Hkv, D, Dv, cap, _lib.PJX_BF16, sc, split_len, 0, _ptr(ws), need, stream)
    _lib.check(rc)
    torch.cuda.synchronize(dev)
    return (o_s, lse_s), (o_w, lse_w)


def test_static_scratch_decode_matches_workspace_decode_twice():
    from probjax_b200 import _lib

    L = _lib.lib()
    dev = torch.device("cuda", 0)
    assert L.pjx_attn_decode_static_scratch_bytes() == 16 * 1024 * 1024
    g = torch.Generator().manual_seed(123)
    B, Hq, Hkv, D = 4, 32, 8, 128
    sc = 1 / math.sqrt(D)
    calls = [
        (4096, torch.tensor([4096, 1000, 2500, 77], dtype=torch.int32), 256),
        (4096, torch.tensor([300, 4096, 1, 0], dtype=torch.int32), 0),  # shorter: stale partials stay behind
    ]
    for cap, lens, split_len in calls:
        q = torch.randn(B, 1, Hq, D, generator=g).bfloat16().to(dev)
        k = torch.randn(B, cap, Hkv, D, generator=g).bfloat16().to(dev)
        v = torch.randn(B, cap, Hkv, D, generator=g).bfloat16().to(dev)
        (o_s, lse_s), (o_w, lse_w) = _call_pair(L, q, k, v, lens.to(dev), sc, split_len)
        # same kernels, same split geometry: 16-bit outputs within 2e-2, LSE within 1e-3 (they are in fact equal)
        assert float((o_s.float() - o_w.float()).abs().max()) <= 2e-2
        fin = torch.isfinite(lse_w)
        assert torch.equal(torch.isinf(lse_s), torch.isinf(lse_w))
        assert float((lse_s[fin] - lse_w[fin]).abs().max()) <= 1e-3
        assert (o_s[lens.to(dev) == 0] == 0).all()


def test_static_scratch_decode_rejects_what_it_cannot_hold():
    from probjax_b200 import _lib

    L = _lib.lib()
    dev = torch.device("cuda", 0)
    B, Hq, Hkv, D, cap = 64, 32, 8, 128, 32768
    q = torch.zeros(B, 1, Hq, D, dtype=torch.bfloat16, device=dev)
    o = torch.empty_like(q)
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    # 64 x 8 x 512 splits x 4 rows x 129 floats is far beyond 16 MiB; the caches are never touched
    rc = L.pjx_attn_decode_splitkv_static(_ptr(q), _ptr(q), _ptr(q), None, _ptr(o), None,
                                          B, 1, Hq, Hkv, D, D, cap, _lib.PJX_BF16, 0.1, 64, stream)
    assert rc == _lib.PJX_ERR_WORKSPACE and "split_len" in _lib.last_error()
    # fp32 is not a streaming-kernel case
    rc = L.pjx_attn_decode_splitkv_static(_ptr(q), _ptr(q), _ptr(q), None, _ptr(o), None,
                                          1, 1, Hq, Hkv, D, D, 64, _lib.PJX_F32, 0.1, 64, stream)
    assert rc == _lib.PJX_ERR_UNSUPPORTED
