"""GPU parity of the sublayer companions (short conv + SiLU, gated RMSNorm) against their CPU
oracles and the reference-generated golden vectors (k3mini/model.py:76-98).  The whole sublayer is
covered by tests/test_sublayer_gpu.py."""
import os

import pytest
import torch

from oracle import kda_oracle as O
from tests.kda_testlib import max_rel, rel_l2

pytestmark = pytest.mark.gpu


def _check(a, r, tol):
    assert torch.isfinite(a.float()).all()
    assert max_rel(a, r) <= tol and rel_l2(a, r) <= tol, (max_rel(a, r), rel_l2(a, r))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1.5e-2)])
@pytest.mark.parametrize("B,T,Cc,cu", [(2, 37, 96, None), (1, 300, 768, [0, 1, 5, 130, 300]), (3, 64, 128, None)])
def test_short_conv(dtype, tol, B, T, Cc, cu):
    from openkimi_b200 import ShortConvolution

    gen = torch.Generator().manual_seed(0)
    x = torch.randn(B, T, Cc, generator=gen).to(dtype)
    dy = torch.randn(B, T, Cc, generator=gen).to(dtype)
    mod = ShortConvolution(Cc, 4).cuda()
    w = mod.weight.detach().cpu().clone()
    cu_t = None if cu is None else torch.tensor(cu)
    xr = x.float().clone().requires_grad_(True)
    wr = w.clone().requires_grad_(True)
    yr = O.short_conv_oracle(xr, wr, cu_t)
    yr.backward(dy.float())
    xd = x.detach().cuda().requires_grad_(True)
    yd, _ = mod(xd, cu_seqlens=None if cu is None else cu_t.cuda())
    yd.backward(dy.cuda())
    _check(yd, yr.detach(), tol)
    _check(xd.grad, xr.grad, tol)
    _check(mod.weight.grad, wr.grad, tol)


def test_short_conv_golden(golden_dir):
    from openkimi_b200 import ShortConvolution

    c = torch.load(os.path.join(golden_dir, "misc.pt"), weights_only=False)["conv"]
    mod = ShortConvolution(96, 4).cuda()
    with torch.no_grad():
        mod.weight.copy_(c["weight"])
    _check(mod(c["x"].cuda())[0], c["out"], 1e-5)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1.5e-2)])
def test_norm_gate(dtype, tol):
    from openkimi_b200 import FusedRMSNormGated

    gen = torch.Generator().manual_seed(1)
    x = torch.randn(2, 50, 6, 128, generator=gen).to(dtype)
    g = torch.randn(2, 50, 6, 128, generator=gen).to(dtype)
    dy = torch.randn(2, 50, 6, 128, generator=gen).to(dtype)
    mod = FusedRMSNormGated(128).cuda()
    with torch.no_grad():
        mod.weight.uniform_(0.5, 1.5)
    w = mod.weight.detach().cpu().clone().requires_grad_(True)
    xr, gr = x.float().clone().requires_grad_(True), g.float().clone().requires_grad_(True)
    yr = O.rms_norm_gate_oracle(xr, gr, w)
    yr.backward(dy.float())
    xd, gd = x.detach().cuda().requires_grad_(True), g.detach().cuda().requires_grad_(True)
    yd = mod(xd, gd)
    yd.backward(dy.cuda())
    _check(yd, yr.detach(), tol)
    _check(xd.grad, xr.grad, tol)
    _check(gd.grad, gr.grad, tol)
    _check(mod.weight.grad, w.grad, tol)


def test_norm_gate_golden(golden_dir):
    """Head width 128 against the reference module's own output and autograd gradients."""
    from openkimi_b200 import FusedRMSNormGated

    n = torch.load(os.path.join(golden_dir, "misc.pt"), weights_only=False)["norm_gate_128"]
    mod = FusedRMSNormGated(128).cuda()
    with torch.no_grad():
        mod.weight.copy_(n["weight"])
    xd, gd = n["x"].cuda().requires_grad_(True), n["gate"].cuda().requires_grad_(True)
    yd = mod(xd, gd)
    yd.backward(n["dy"].cuda())
    _check(yd, n["out"], 1e-5)
    _check(xd.grad, n["dx"], 1e-5)
    _check(gd.grad, n["dgate"], 1e-5)
    _check(mod.weight.grad, n["dweight"], 1e-5)
