"""Short convolution fused into the KDA kernels (k3mini/model.py:181-185 followed by
k3mini/model.py:200-216), forward in the load stage and backward inside the backward kernels: the
fused call must give the same bits as ShortConvolution followed by chunk_kda -- outputs, state and
every input / parameter gradient -- except the three filter gradients, whose sums run over chunks in
a different (fixed) order and must agree to FP32 summation accuracy; and both must agree with the
CPU oracle."""
import pytest
import torch

from oracle import kda_oracle as orc

pytestmark = pytest.mark.gpu


def _inputs(B, T, H, D, ks, seed, dtype=torch.bfloat16):
    gen = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=gen)
    t = dict(q=r(B, T, H, D), k=r(B, T, H, D), v=r(B, T, H, D), g=r(B, T, H, D), beta=r(B, T, H), do=r(B, T, H, D))
    t = {n: x.to(dtype) for n, x in t.items()}
    t["w"] = [(r(H * D, 1, ks) * 0.5).to(dtype) for _ in range(3)]
    t["A_log"] = torch.log(torch.empty(H).uniform_(1.0, 16.0, generator=gen))
    t["dt_bias"] = r(H * D) * 0.1
    return t


def _run(t, fused, cu=None, h0=None, **kw):
    from openkimi_b200 import chunk_kda
    from openkimi_b200.modules import short_convolution
    dev = "cuda"
    leaf = lambda x: x.to(dev).detach().clone().requires_grad_(True)
    q, k, v, g, beta = (leaf(t[n]) for n in ("q", "k", "v", "g", "beta"))
    w = [leaf(x) for x in t["w"]]
    A, bias = leaf(t["A_log"]), leaf(t["dt_bias"])
    h0d = leaf(h0) if h0 is not None else None
    cud = None if cu is None else cu.to(dev)
    B, T, H, D = q.shape
    if fused:
        qq, kk, vv, cw = q, k, v, tuple(w)
    else:
        qq, kk, vv = (short_convolution(x.view(B, T, H * D), wi, cud).view(B, T, H, D) for x, wi in zip((q, k, v), w))
        cw = None
    o, ht = chunk_kda(qq, kk, vv, g, beta, A_log=A, dt_bias=bias, use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True,
                      use_beta_sigmoid_in_kernel=True, output_final_state=True, initial_state=h0d, cu_seqlens=cud,
                      short_conv_weights=cw, **kw)
    loss = (o.float() * t["do"].to(dev).float()).sum() + (ht * 0.01).sum()
    loss.backward()
    out = dict(o=o, ht=ht, dq=q.grad, dk=k.grad, dv=v.grad, dg=g.grad, dbeta=beta.grad, dA=A.grad, dbias=bias.grad,
               dwq=w[0].grad, dwk=w[1].grad, dwv=w[2].grad)
    if h0d is not None:
        out["dh0"] = h0d.grad
    return {n: x.detach().cpu() for n, x in out.items()}


def _same(a, b):
    for n in a:
        if n in ("dwq", "dwk", "dwv"):  # same terms, another fixed summation order (then rounded to the filter's type)
            err = (a[n].float() - b[n].float()).norm() / b[n].float().norm().clamp_min(1e-20)
            assert torch.isfinite(a[n].float()).all() and err < 2e-3, (n, float(err))
        else:
            assert torch.equal(a[n], b[n]), (n, (a[n].float() - b[n].float()).abs().max())


@pytest.mark.parametrize("ks", [4, 3, 2, 1])
def test_fused_matches_unfused_bitwise(ks):
    t = _inputs(2, 200, 2, 128, ks, seed=31 + ks)
    _same(_run(t, True), _run(t, False))


@pytest.mark.parametrize("recompute", [False, True])
def test_fused_varlen_with_initial_state(recompute):
    t = _inputs(1, 389, 3, 128, 4, seed=77)
    cu = torch.tensor([0, 2, 70, 134, 135, 389])
    h0 = torch.randn(5, 3, 128, 128, generator=torch.Generator().manual_seed(5)) * 0.02
    a = _run(t, True, cu=cu, h0=h0, disable_recompute=not recompute)
    b = _run(t, False, cu=cu, h0=h0, disable_recompute=not recompute)
    _same(a, b)


@pytest.mark.parametrize("T", [1, 3, 4, 66])
def test_fused_tiny_sequences(T):
    """Fewer tokens than filter taps, and a chunk border with a one-row halo."""
    t = _inputs(2, T, 2, 128, 4, seed=90 + T)
    _same(_run(t, True), _run(t, False))


def test_fused_against_oracle():
    """Oracle: the reference's conv1d + SiLU (k3mini/model.py:76-88) in FP32 rounded to BF16 like the
    module's output, then the recurrent KDA oracle."""
    B, T, H, D = 1, 160, 2, 128
    t = _inputs(B, T, H, D, 4, seed=9)
    dev = _run(t, True)
    conv = [orc.short_conv_oracle(t[n].float().view(B, T, H * D), w.float()).to(torch.bfloat16).view(B, T, H, D)
            for n, w in zip(("q", "k", "v"), t["w"])]
    ref = orc.kda_oracle_fwd_bwd(conv[0], conv[1], conv[2], t["g"], t["beta"], t["do"], a_log=t["A_log"],
                                 dt_bias=t["dt_bias"], round_qk_to=torch.bfloat16)
    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30)).item()
    assert rel(dev["o"], ref["o"]) < 5e-3
    assert rel(dev["ht"], ref["ht"]) < 5e-3


def test_unsupported_sizes_take_the_separate_kernels():
    """d = 64 / FP32: the argument is honoured through the stand-alone convolution kernels."""
    t = _inputs(1, 100, 2, 64, 4, seed=3, dtype=torch.float32)
    a, b = _run(t, True), _run(t, False)
    _same(a, b)


def test_sublayer_fused_equals_unfused():
    from openkimi_b200.modules import KimiDeltaAttention
    torch.manual_seed(0)
    m = KimiDeltaAttention(256, 2).cuda().bfloat16()
    x = torch.randn(2, 130, 256, device="cuda", dtype=torch.bfloat16)
    outs = []
    for fuse in (True, False):
        m.fuse_short_conv = fuse
        m.zero_grad()
        xi = x.clone().requires_grad_(True)
        y = m(xi)
        y.float().square().mean().backward()
        outs.append([("y", y.detach()), ("dx", xi.grad)] + [(n, p.grad.clone()) for n, p in m.named_parameters()])
    for (n, a), (_, b) in zip(*outs):
        if n.endswith("conv.weight"):  # filter gradients: another fixed summation order
            assert (a.float() - b.float()).norm() / b.float().norm() < 2e-3, n
        else:
            assert torch.equal(a, b), n
