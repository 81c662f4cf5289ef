"""Generate the golden vectors under tests/golden/ by running the REFERENCE's own code.

Run once, in a container that has the reference checkout (read-only) next to this repo:

    python tests/golden/make_golden.py /path/to/reference

It imports ``k3mini.model`` (kda_recurrent_reference, CausalDepthwiseConv1d,
HeadwiseRMSNormGate), ``experiments.kda_sm90.guarded_diagonal_oracle`` and
``scripts.profile_kda_gate_spans`` from that checkout, feeds them seeded inputs and stores
inputs and outputs in ``tests/golden/*.pt``.  The reference holds no golden files of its
own (its fixtures are seeded-random and regenerated at run time), so these files are the
pin for ``oracle/kda_oracle.py``; nothing at test time reads the reference checkout.
"""

from __future__ import annotations

import math
import os
import sys

import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


def kda_case(ref, *, seed, shape, dtype, a_lo=1.0, a_hi=16.0, dt_bias_std=0.0):
    """The recipe of tests/test_h100_parity.py:72-96 (raw q,k,v,gate ~ N(0,1), beta logits,
    A_log = log U(a_lo,a_hi), prologue of model.py:218-223) on the CPU with ``do``~N(0,1)."""
    torch.manual_seed(seed)
    b, t, h, d = shape
    q = torch.randn(shape, dtype=dtype).requires_grad_()
    k = torch.randn(shape, dtype=dtype).requires_grad_()
    v = torch.randn(shape, dtype=dtype).requires_grad_()
    raw = torch.randn(shape, dtype=dtype).requires_grad_()
    bl = torch.randn(b, t, h, dtype=dtype).requires_grad_()
    a_log = torch.log(torch.empty(h).uniform_(a_lo, a_hi)).requires_grad_()
    dt_bias = (torch.randn(h, d) * dt_bias_std).requires_grad_()
    do = torch.randn(shape, dtype=dtype)
    qn = F.normalize(q.float(), dim=-1, eps=1e-6).to(q.dtype)
    kn = F.normalize(k.float(), dim=-1, eps=1e-6).to(k.dtype)
    log_alpha = -a_log.exp().view(1, 1, h, 1) * F.softplus(raw.float() + dt_bias.view(1, 1, h, d))
    out = ref.kda_recurrent_reference(qn, kn, v, log_alpha, bl.float().sigmoid(), scale=d ** -0.5)
    out.backward(do)
    leaves = dict(q=q, k=k, v=v, g=raw, beta=bl, a_log=a_log, dt_bias=dt_bias)
    rec = {n: x.detach().clone() for n, x in leaves.items()}
    rec["do"] = do
    rec["o"] = out.detach().clone()
    rec["qn"], rec["kn"], rec["log_alpha"] = qn.detach(), kn.detach(), log_alpha.detach()
    for n, x in leaves.items():
        rec["d" + n] = x.grad.detach().clone()
    return rec


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    import k3mini.model as ref
    from experiments.kda_sm90 import guarded_diagonal_oracle as gdo
    from scripts.profile_kda_gate_spans import gate_tile_spans

    gold = {}
    # the reference's only fast-path-vs-oracle pin: one 64-token chunk, H=1, d=128, BF16, seed 123
    gold["parity_1x64x1x128_bf16"] = kda_case(ref, seed=123, shape=(1, 64, 1, 128), dtype=torch.bfloat16)
    # multi-chunk, multi-head FP32 cases (ragged T exercises a partial last chunk)
    gold["fp32_2x150x2x64"] = kda_case(ref, seed=7, shape=(2, 150, 2, 64), dtype=torch.float32, dt_bias_std=0.3)
    gold["fp32_1x130x2x128"] = kda_case(ref, seed=11, shape=(1, 130, 2, 128), dtype=torch.float32)
    torch.save(gold, os.path.join(HERE, "kda_recurrent.pt"))

    # guarded diagonal: the three input sets of tests/test_kda_guarded_diagonal.py:12-27
    def diag_inputs(spans):
        torch.manual_seed(19)
        blocks = len(spans)
        inc = torch.rand(blocks, 16, 32)
        inc[:, 0] = 0.0
        for blk, span in enumerate(spans):
            inc[blk] *= span / inc[blk].sum(dim=0).amax().clamp_min(1e-6)
        gate = -inc.cumsum(dim=1)
        q = torch.randn_like(gate)
        k = torch.randn_like(gate)
        beta = torch.sigmoid(torch.randn(blocks, 16))
        return gate, q, k, beta, torch.randn(blocks, 16, 16), torch.randn(blocks, 16, 16)

    diag = {}
    for name, spans, thr, policy, poke in (
        ("small", [2.0, 8.0, 16.0], 20.0, "first", False),
        ("reject", [4.0, 200.0, 4.0], 20.0, "first", True),
        ("midpoint", [100.0, 200.0, 251.0], 240.0, "midpoint", False),
    ):
        inp = list(diag_inputs(spans))
        if poke:
            inp[0][2, 5, 0] = inp[0][2, 4, 0] + 1.0
        ex = gdo.exact_diagonal_backward(*inp)
        gd = gdo.guarded_diagonal_backward(*inp, max_log2_span=thr, reference_policy=policy)
        diag[name] = dict(inputs=inp, thr=thr, policy=policy,
                          exact=(ex.dq, ex.dk, ex.dkt), guarded=(gd.dq, gd.dk, gd.dkt), hits=gd.guard_hits)
    torch.save(diag, os.path.join(HERE, "guarded_diagonal.pt"))

    # gate-span closed form (tests/test_kda_gate_spans.py:10-19) and a random case
    misc = {}
    raw0 = torch.zeros(1, 64, 1, 32)
    a0 = torch.tensor([math.log(math.log(2.0))])
    b0 = torch.full((1, 32), math.log(math.expm1(1.0)))
    torch.manual_seed(5)
    raw1, a1, b1 = torch.randn(2, 128, 3, 64), torch.log(torch.empty(3).uniform_(1, 16)), torch.randn(3, 64) * 0.1
    misc["spans"] = [dict(raw=raw0, a_log=a0, dt_bias=b0, out=gate_tile_spans(raw0, a0, b0)),
                     dict(raw=raw1, a_log=a1, dt_bias=b1, out=gate_tile_spans(raw1, a1, b1))]
    # short conv + SiLU (model.py:76-88) and headwise RMSNorm gate (model.py:91-98)
    torch.manual_seed(6)
    conv = ref.CausalDepthwiseConv1d(96, 4)
    x = torch.randn(2, 37, 96)
    misc["conv"] = dict(x=x, weight=conv.weight.detach().clone(), out=conv(x).detach())
    ng = ref.HeadwiseRMSNormGate(32, 1e-6)
    with torch.no_grad():
        ng.weight.uniform_(0.5, 1.5)
    xo, go = torch.randn(2, 9, 3, 32), torch.randn(2, 9, 3, 32)
    misc["norm_gate"] = dict(x=xo, gate=go, weight=ng.weight.detach().clone(), out=ng(xo, go).detach())
    # the head width the kernels serve (128), with gradients from the reference module's autograd
    ng128 = ref.HeadwiseRMSNormGate(128, 1e-6)
    with torch.no_grad():
        ng128.weight.uniform_(0.5, 1.5)
    x128 = torch.randn(2, 9, 3, 128).requires_grad_()
    g128 = torch.randn(2, 9, 3, 128).requires_grad_()
    dy128 = torch.randn(2, 9, 3, 128)
    y128 = ng128(x128, g128)
    y128.backward(dy128)
    misc["norm_gate_128"] = dict(x=x128.detach().clone(), gate=g128.detach().clone(), weight=ng128.weight.detach().clone(),
                                 dy=dy128, out=y128.detach().clone(), dx=x128.grad.clone(), dgate=g128.grad.clone(),
                                 dweight=ng128.weight.grad.clone())
    torch.save(misc, os.path.join(HERE, "misc.pt"))

    # the whole KimiDeltaAttention sublayer (model.py:132-227) through the reference's own module on
    # its reference branch (recurrent FP32 oracle), FP32, two heads of 128: output, input gradient and
    # the gradient of every parameter
    from k3mini.backends import resolve_backend
    from k3mini.config import KernelBackend, ModelConfig

    torch.manual_seed(8)
    cfg = ModelConfig(d_model=256, n_heads=2, kda_head_dim=128, kda_conv_kernel=4, kernel_backend=KernelBackend.REFERENCE)
    mod = ref.KimiDeltaAttention(cfg, resolve_backend(KernelBackend.REFERENCE))
    with torch.no_grad():
        mod.dt_bias.normal_(0.0, 0.2)
        mod.out_norm_gate.weight.uniform_(0.5, 1.5)
    xs = torch.randn(2, 150, 256).requires_grad_()
    dys = torch.randn(2, 150, 256)
    ys = mod(xs)
    ys.backward(dys)
    torch.save(dict(state={k: v.detach().clone() for k, v in mod.state_dict().items()}, x=xs.detach().clone(), dy=dys,
                    out=ys.detach().clone(), dx=xs.grad.clone(),
                    grads={k: v.grad.clone() for k, v in mod.named_parameters()}),
               os.path.join(HERE, "sublayer.pt"))
    print("wrote", sorted(os.listdir(HERE)))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
