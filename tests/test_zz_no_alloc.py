"""The allocation-free RMSNorm backward (``kwu_rmsnorm_bwd_noalloc``) against the regular entry point.

Some users of the native library cannot allocate device memory at the point where they call it (a
plugin inside a runtime that owns the memory pool, code under a fixed memory budget). For them the
library carries its temporary inside its own image. This test calls the exported C symbol directly,
twice in a row with different shapes and data, and checks both results against ``kwu_rmsnorm_bwd``
given an ordinary scratch buffer. The second call also shows that nothing left in the shared scratch
by the first call leaks into the next result. The file sorts last so a run that stops at the first
failure has already run every other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

c_int = ctypes.c_int


def _ptr(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _case(rows, cols, seed, with_res):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, cols, device="cuda", generator=g).to(torch.bfloat16)
    dy = torch.randn(rows, cols, device="cuda", generator=g).to(torch.bfloat16)
    dres = torch.randn(rows, cols, device="cuda", generator=g).to(torch.bfloat16) if with_res else None
    w = torch.rand(cols, device="cuda", generator=g) + 0.5
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6).contiguous()
    return x, w, rstd, dy, dres


def test_noalloc_rmsnorm_bwd_matches_regular_entry_point_twice():
    from kohakuwullm_b200.ops import native

    L = native.require()
    L.kwu_rmsnorm_bwd_noalloc.restype = ctypes.c_int
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for rows, cols, seed, with_res in ((1000, 1280, 1, False), (333, 4096, 2, True)):
        x, w, rstd, dy, dres = _case(rows, cols, seed, with_res)
        # regular entry point with a caller-provided scratch buffer
        dx_ref = torch.empty_like(x)
        dw_ref = torch.empty(cols, dtype=torch.float32, device="cuda")
        nblocks = L.kwu_rmsnorm_bwd_blocks(c_int(rows))
        scratch = torch.empty(nblocks, cols, dtype=torch.float32, device="cuda")
        rc = L.kwu_rmsnorm_bwd(_ptr(x), _ptr(w), _ptr(rstd), _ptr(dy), _ptr(dres), _ptr(dx_ref), _ptr(dw_ref),
                               _ptr(scratch), c_int(rows), c_int(cols), c_int(0), c_int(0), stream)
        assert rc == 0, L.kwu_last_error()
        # allocation-free entry point: inputs and outputs only
        dx = torch.empty_like(x)
        dw = torch.empty(cols, dtype=torch.float32, device="cuda")
        rc = L.kwu_rmsnorm_bwd_noalloc(_ptr(x), _ptr(w), _ptr(rstd), _ptr(dy), _ptr(dres), _ptr(dx), _ptr(dw),
                                       c_int(rows), c_int(cols), c_int(0), c_int(0), stream)
        assert rc == 0, L.kwu_last_error()
        torch.cuda.synchronize()
        assert torch.equal(dx, dx_ref)
        # the partial sums are grouped differently (fewer blocks), so dw agrees to rounding only
        err = (dw - dw_ref).abs().max().item()
        assert err <= 2e-2 * dw_ref.abs().max().item(), f"dw differs by {err}"


def test_noalloc_rejects_oversized_rows_of_columns():
    from kohakuwullm_b200.ops import native

    L = native.require()
    L.kwu_rmsnorm_bwd_noalloc.restype = ctypes.c_int
    cols = 4096 + 8
    x, w, rstd, dy, _ = _case(4, cols, 3, False)
    dx = torch.empty_like(x)
    dw = torch.empty(cols, dtype=torch.float32, device="cuda")
    rc = L.kwu_rmsnorm_bwd_noalloc(_ptr(x), _ptr(w), _ptr(rstd), _ptr(dy), _ptr(None), _ptr(dx), _ptr(dw),
                                   c_int(4), c_int(cols), c_int(0), c_int(0),
                                   ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc != 0
    assert b"exceeds" in L.kwu_last_error()
