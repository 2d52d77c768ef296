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


def _both(L, rows, cols, seed, with_res, accumulate, stream, with_w=True, with_dw=True):
    """Run the regular and the allocation-free entry point on the same inputs; returns (dx, dw) of each."""
    x, w, rstd, dy, dres = _case(rows, cols, seed, with_res)
    base = torch.full((cols,), 0.25, dtype=torch.float32, device="cuda")   # what dw holds before an accumulating call
    nblocks = L.kwu_rmsnorm_bwd_blocks(c_int(rows))
    scratch = torch.empty(nblocks, cols, dtype=torch.float32, device="cuda")
    dx_ref, dw_ref = torch.empty_like(x), base.clone()
    rc = L.kwu_rmsnorm_bwd(_ptr(x), _ptr(w if with_w else None), _ptr(rstd), _ptr(dy), _ptr(dres), _ptr(dx_ref),
                           _ptr(dw_ref if with_dw else None), _ptr(scratch), c_int(rows), c_int(cols), c_int(0),
                           c_int(int(accumulate)), stream)
    assert rc == 0, L.kwu_last_error()
    dx, dw = torch.empty_like(x), base.clone()
    rc = L.kwu_rmsnorm_bwd_noalloc(_ptr(x), _ptr(w if with_w else None), _ptr(rstd), _ptr(dy), _ptr(dres), _ptr(dx),
                                   _ptr(dw if with_dw else None), c_int(rows), c_int(cols), c_int(0),
                                   c_int(int(accumulate)), stream)
    assert rc == 0, L.kwu_last_error()
    torch.cuda.synchronize()
    return (dx_ref, dw_ref), (dx, dw), base


@pytest.mark.parametrize("rows,cols", [(4096, 4096), (32768, 1280), (2000, 2048), (1500, 3072)])
@pytest.mark.parametrize("accumulate", [False, True])
def test_noalloc_with_the_block_cap_active_and_with_accumulation(rows, cols, accumulate):
    """Row counts for which the regular entry point would use more blocks than the built-in scratch has rows
    (the cap must keep every partial sum inside the array), both ways of forming dw (register-resident rows up
    to 2048 columns add to dw directly, wider rows go through the column sum of the partials), and dw += ."""
    from kohakuwullm_b200.ops import native

    L = native.require()
    L.kwu_rmsnorm_bwd_noalloc.restype = ctypes.c_int
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    (dx_ref, dw_ref), (dx, dw), base = _both(L, rows, cols, 7, True, accumulate, stream)
    assert torch.equal(dx, dx_ref)
    scale = max((dw_ref - (base if accumulate else 0)).abs().max().item(), 1e-6)
    assert (dw - dw_ref).abs().max().item() <= 2e-2 * scale
    if accumulate:   # the previous contents of dw were kept
        assert (dw_ref - base).abs().max().item() > 0


def test_noalloc_without_weight_or_without_dw_writes_dx_only():
    from kohakuwullm_b200.ops import native

    L = native.require()
    L.kwu_rmsnorm_bwd_noalloc.restype = ctypes.c_int
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for with_w, with_dw in ((False, False), (True, False)):
        (dx_ref, _), (dx, dw), base = _both(L, 700, 1280, 9, False, False, stream, with_w=with_w, with_dw=with_dw)
        assert torch.equal(dx, dx_ref)
        assert torch.equal(dw, base)      # dw was not passed: untouched


def test_noalloc_narrow_call_after_a_wide_one_ignores_stale_partials():
    """The shared scratch keeps the last call's contents: a call with fewer columns behind a wide one (same
    stream) must not read partial sums beyond its own columns."""
    from kohakuwullm_b200.ops import native

    L = native.require()
    L.kwu_rmsnorm_bwd_noalloc.restype = ctypes.c_int
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _both(L, 3000, 4096, 21, False, False, stream)
    (dx_ref, dw_ref), (dx, dw), _ = _both(L, 3000, 2560, 22, False, False, stream)
    assert torch.equal(dx, dx_ref)
    assert (dw - dw_ref).abs().max().item() <= 2e-2 * dw_ref.abs().max().item()


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
