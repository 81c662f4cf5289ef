"""The whole KimiDeltaAttention sublayer (k3mini/model.py:132-227; benchmark configuration 4) on the
GPU against (a) the golden vectors produced by the reference's own module on its reference branch
and (b) the CPU oracle composition  linear -> short_conv_oracle -> kda_oracle -> rms_norm_gate_oracle
-> linear  at the width of configuration 4, in FP32 and in BF16 under autocast exactly as bench.py
drives it; with the short convolution fused into the KDA load stage and not, and with packed
documents.  Compared: output, input gradient and the gradient of EVERY parameter (this also covers
the merged narrow projection GEMM and its slicing)."""
import os

import pytest
import torch

from oracle import kda_oracle as O
from tests.kda_testlib import max_rel, rel_l2

pytestmark = pytest.mark.gpu


def _module(d_model, heads, state, fuse, dtype=torch.float32):
    from openkimi_b200 import KimiDeltaAttention

    m = KimiDeltaAttention(d_model, heads, 128, conv_kernel=4, disable_recompute=True, fuse_short_conv=fuse)
    missing = m.load_state_dict(state, strict=True)   # same parameter names and shapes as the reference module
    assert not missing.missing_keys and not missing.unexpected_keys
    return m.cuda().to(dtype) if dtype != torch.float32 else m.cuda()


def _compare(named, tol_out, tol_grad):
    bad = []
    for name, a, r, is_out in named:
        assert torch.isfinite(a.float()).all(), name
        l2, mx = rel_l2(a, r), max_rel(a, r)
        if l2 > (tol_out if is_out else tol_grad):
            bad.append(f"{name}: rel_l2={l2:.2e} max_rel={mx:.2e}")
    assert not bad, "; ".join(bad)


@pytest.mark.parametrize("fuse", [False, True])
def test_sublayer_golden_fp32(golden_dir, fuse):
    """FP32 operands: <= 1e-4 on the output and the input gradient (the north-star FP32 bound), 2e-3 on
    the parameter gradients (sums over all 300 tokens)."""
    s = torch.load(os.path.join(golden_dir, "sublayer.pt"), weights_only=False)
    m = _module(256, 2, s["state"], fuse)
    x = s["x"].cuda().requires_grad_(True)
    y = m(x)
    y.backward(s["dy"].cuda())
    rows = [("out", y.detach(), s["out"], True), ("dx", x.grad, s["dx"], True)]
    rows += [(k, p.grad, s["grads"][k], False) for k, p in m.named_parameters()]
    assert len(rows) == 2 + len(s["grads"])
    _compare(rows, 1e-4, 2e-3)


def _config4_case(seed, B, T, cu=None):
    torch.manual_seed(seed)
    from openkimi_b200 import KimiDeltaAttention

    proto = KimiDeltaAttention(768, 6, 128, conv_kernel=4)
    with torch.no_grad():   # configuration 4: weights N(0, 0.02); a non-trivial dt_bias and norm weight
        for name, prm in proto.named_parameters():
            if name.endswith("proj.weight") or "out_gate" in name or name.endswith("conv.weight"):
                prm.normal_(0.0, 0.02)
        proto.dt_bias.normal_(0.0, 0.2)
        proto.out_norm_gate.weight.uniform_(0.5, 1.5)
        for name in ("q_conv", "k_conv", "v_conv"):   # taps large enough that the convolved rows are not ~0
            getattr(proto, name).weight.normal_(0.0, 0.5)
    state = {k: v.detach().clone() for k, v in proto.state_dict().items()}
    x = torch.randn(B, T, 768)
    dy = torch.randn(B, T, 768)
    params = {k: v.clone().requires_grad_(True) for k, v in state.items()}
    xr = x.clone().requires_grad_(True)
    yr = O.kda_sublayer_oracle(xr, params, n_heads=6, head_dim=128, cu_seqlens=cu)
    yr.backward(dy)
    return state, x, dy, yr.detach(), xr.grad, {k: v.grad for k, v in params.items()}


@pytest.mark.parametrize("fuse", [False, True])
@pytest.mark.parametrize("cu", [None, [0, 37, 200, 400]])
def test_sublayer_config4_width_bf16_autocast(fuse, cu):
    """d_model 768, 6 heads of 128, BF16 autocast as in bench.py: 2e-2 relative L2 on output, input
    gradient and every parameter gradient (BF16 operands throughout: the north-star BF16 bound)."""
    cu_t = None if cu is None else torch.tensor(cu)
    B, T = (2, 200) if cu is None else (1, 400)
    state, x, dy, yr, dxr, gr = _config4_case(21, B, T, cu_t)
    m = _module(768, 6, state, fuse)
    xd = x.cuda().requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = m(xd, cu_seqlens=None if cu is None else cu_t.cuda())
    y.backward(dy.cuda().to(y.dtype))
    rows = [("out", y.detach(), yr, True), ("dx", xd.grad, dxr, True)]
    rows += [(k, p.grad, gr[k], False) for k, p in m.named_parameters()]
    _compare(rows, 2e-2, 2e-2)


def test_sublayer_config4_width_fp32():
    state, x, dy, yr, dxr, gr = _config4_case(22, 2, 130)
    m = _module(768, 6, state, True)
    xd = x.cuda().requires_grad_(True)
    y = m(xd)
    y.backward(dy.cuda())
    rows = [("out", y.detach(), yr, True), ("dx", xd.grad, dxr, True)]
    rows += [(k, p.grad, gr[k], False) for k, p in m.named_parameters()]
    _compare(rows, 1e-4, 2e-3)
