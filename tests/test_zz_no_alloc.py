"""The allocation-free short-convolution backward (``kda_short_conv_bwd_static``).

Some hosts of this library cannot create device memory when they call it -- their memory
plan is fixed at start-up, or an allocator call is forbidden inside their latency-critical
loop.  For them the filter-gradient partial sums live in an array inside the library image.
This test calls that entry point through the C ABI twice in a row (the second call finds the
first call's leftovers in the shared array) and checks both against the ordinary entry point,
which must agree bit for bit because the kernels and the reduction order are the same."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _run(lib, static, x, w, dy, cu):
    dx = torch.empty_like(x)
    dw = torch.full((x.shape[-1], w.shape[-1]), float("nan"), device=x.device)
    B, T, Cc = x.shape
    dtype = 1 if x.dtype == torch.bfloat16 else 0
    n = 0 if cu is None else cu.numel() - 1
    if static:
        rc = lib.kda_short_conv_bwd_static(_ptr(x), _ptr(w), _ptr(dy), _ptr(dx), _ptr(dw), B, T, Cc, w.shape[-1], dtype,
                                           _ptr(cu), n, None)
    else:
        part = torch.empty(64, Cc, w.shape[-1], device=x.device)
        rc = lib.kda_short_conv_bwd(_ptr(x), _ptr(w), _ptr(dy), _ptr(dx), _ptr(dw), _ptr(part), 64, B, T, Cc,
                                    w.shape[-1], dtype, _ptr(cu), n, None)
    torch.cuda.synchronize()
    assert rc == 0
    return dx, dw


def test_static_scratch_matches_regular_entry_point_twice():
    from openkimi_b200 import _lib

    lib = _lib.load()
    gen = torch.Generator().manual_seed(0)
    cases = [  # the second case is smaller than the first, so stale partial sums lie beyond its footprint
        (torch.randn(2, 300, 768, generator=gen).bfloat16().cuda(), torch.randn(768, 1, 4, generator=gen).cuda(), None),
        (torch.randn(1, 129, 96, generator=gen).cuda(), torch.randn(96, 1, 3, generator=gen).cuda(),
         torch.tensor([0, 5, 70, 129], device="cuda")),
    ]
    for x, w, cu in cases:
        dy = torch.randn(x.shape, generator=gen).to(x.dtype).cuda()
        w2 = w.reshape(w.shape[0], w.shape[-1]).contiguous()
        dx_ref, dw_ref = _run(lib, False, x, w2, dy, cu)
        dx_new, dw_new = _run(lib, True, x, w2, dy, cu)
        assert torch.isfinite(dw_new).all()
        assert torch.equal(dx_new, dx_ref) and torch.equal(dw_new, dw_ref)


def test_static_scratch_rejects_oversize():
    from openkimi_b200 import _lib

    lib = _lib.load()
    z = torch.zeros(16, device="cuda")
    rc = lib.kda_short_conv_bwd_static(_ptr(z), _ptr(z), _ptr(z), _ptr(z), _ptr(z), 1, 1, 4096, 4, 0, None, 0, None)
    assert rc == 9
    assert b"8192" in lib.kda_status_string(rc)
