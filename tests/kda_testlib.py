"""Shared helpers of the GPU parity tests: run ``chunk_kda`` on the device and the CPU
oracle on the same seeded inputs, and compare with the error measures the tests state."""

import torch

from oracle import kda_oracle as O

GRADS = ("dq", "dk", "dv", "dg", "dbeta", "dA_log", "ddt_bias", "dh0")


def rel_l2(a, r):
    a, r = a.double().cpu(), r.double().cpu()
    return float((a - r).norm() / r.norm().clamp_min(1e-12))


def max_rel(a, r):
    """max |a - r| relative to the largest reference magnitude (the 'max-abs/rel' measure)."""
    a, r = a.double().cpu(), r.double().cpu()
    return float((a - r).abs().max() / r.abs().max().clamp_min(1e-12))


def run_device(inp, *, fused=True, h0=None, dht=None, cu=None, state_v_first=False, fp32_math=False,
               disable_recompute=True, device="cuda"):
    """chunk_kda forward + backward on the GPU; returns the same dict layout as the oracle."""
    from openkimi_b200 import chunk_kda

    dev = torch.device(device)
    leaves = {n: inp[n].to(dev).detach().clone().requires_grad_(True) for n in ("q", "k", "v", "g", "beta")}
    a_log = inp["a_log"].to(dev).detach().clone().requires_grad_(True) if fused else None
    dt_bias = inp["dt_bias"].to(dev).detach().clone().requires_grad_(True) if fused else None
    tr = (lambda s: s.transpose(-1, -2).contiguous()) if state_v_first else (lambda s: s)
    h0d = tr(h0.to(dev)).detach().clone().requires_grad_(True) if h0 is not None else None
    o, ht = chunk_kda(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"], A_log=a_log, dt_bias=dt_bias,
                      scale=inp.get("scale"), initial_state=h0d, output_final_state=True,
                      use_qk_l2norm_in_kernel=fused, use_gate_in_kernel=fused, use_beta_sigmoid_in_kernel=fused,
                      cu_seqlens=None if cu is None else cu.to(dev), cu_seqlens_cpu=cu, state_v_first=state_v_first,
                      fp32_math=fp32_math, disable_recompute=disable_recompute)
    grads_out = [inp["do"].to(dev)]
    outs = [o]
    if dht is not None:
        outs.append(ht)
        grads_out.append(tr(dht.to(dev)))
    torch.autograd.backward(outs, grads_out)
    torch.cuda.synchronize()
    res = {"o": o.detach(), "ht": tr(ht.detach())}
    for n in ("q", "k", "v", "g", "beta"):
        res["d" + n] = leaves[n].grad
    if fused:
        res["dA_log"], res["ddt_bias"] = a_log.grad, dt_bias.grad
    if h0d is not None:
        res["dh0"] = tr(h0d.grad)
    return res


def run_oracle(inp, *, fused=True, h0=None, dht=None, cu=None, dtype=torch.float32):
    # with BF16 activations the reference rounds the normalised q and k back to BF16 before
    # the recurrence (k3mini/model.py:218-219: ``.to(x.dtype)``); FP32 inputs stay FP32
    round_to = torch.bfloat16 if (fused and inp["q"].dtype == torch.bfloat16) else None
    return O.kda_oracle_fwd_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["do"],
                                a_log=inp["a_log"] if fused else None, dt_bias=inp["dt_bias"] if fused else None,
                                scale=inp.get("scale"), initial_state=h0, dht=dht, cu_seqlens=cu, use_qk_l2norm=fused,
                                use_gate=fused, use_beta_sigmoid=fused, dtype=dtype, round_qk_to=round_to)


def max_abs(a, r):
    return float((a.double().cpu() - r.double().cpu()).abs().max())


def compare(dev, ref, tol_max, tol_l2, names=None, abs_escape=0.0):
    """Returns a list of (name, max_rel, rel_l2, ok).  ``abs_escape`` is the reference's own
    rule for references that are numerically zero
    (experiments/kda_sm90/validate_fla_guarded_integration.py:24-25,40-48): a tensor whose
    largest absolute error is below it passes whatever the relative error."""
    rows = []
    for name in names or (("o", "ht") + GRADS):
        if name not in ref or name not in dev or dev[name] is None:
            continue
        r = ref[name].reshape(dev[name].shape)
        m, l = max_rel(dev[name], r), rel_l2(dev[name], r)
        finite = bool(torch.isfinite(dev[name].float()).all())
        ok = finite and ((m <= tol_max and l <= tol_l2) or max_abs(dev[name], r) <= abs_escape)
        rows.append((name, m, l, ok))
    return rows


def assert_rows(rows):
    bad = [r for r in rows if not r[3]]
    assert not bad, "parity failed: " + ", ".join(f"{n}: max_rel={m:.3e} rel_l2={l:.3e}" for n, m, l, _ in bad)
