"""The CPU oracle against the golden vectors produced by the reference's own code
(tests/golden/make_golden.py)."""
import os

import pytest
import torch

from oracle import kda_oracle as O


def _load(golden_dir, name):
    return torch.load(os.path.join(golden_dir, name), weights_only=False)


@pytest.mark.parametrize("case", ["parity_1x64x1x128_bf16", "fp32_2x150x2x64", "fp32_1x130x2x128"])
def test_recurrent_oracle_matches_reference(golden_dir, case):
    g = _load(golden_dir, "kda_recurrent.pt")[case]
    bf16 = g["q"].dtype == torch.bfloat16
    res = O.kda_oracle_fwd_bwd(g["q"], g["k"], g["v"], g["g"], g["beta"], g["do"], a_log=g["a_log"],
                               dt_bias=g["dt_bias"].reshape(-1), scale=g["q"].shape[-1] ** -0.5,
                               round_qk_to=torch.bfloat16 if bf16 else None)
    # the reference returns o in the input dtype (model.py:129)
    # (bit-equal for BF16; FP32 differs only by the einsum summation order of a batched call)
    otol = dict(atol=0, rtol=0) if bf16 else dict(atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(res["o"].to(g["o"].dtype), g["o"], **otol)
    tol = dict(atol=2e-2, rtol=2e-2) if bf16 else dict(atol=2e-5, rtol=2e-5)
    for name, key in (("dq", "dq"), ("dk", "dk"), ("dv", "dv"), ("dg", "dg"), ("dbeta", "dbeta"),
                      ("dA_log", "da_log"), ("ddt_bias", "ddt_bias")):
        want = g[key].float().reshape(res[name].shape)
        torch.testing.assert_close(res[name].float(), want, **tol)


def test_prologue_matches_reference(golden_dir):
    g = _load(golden_dir, "kda_recurrent.pt")["fp32_2x150x2x64"]
    qn, kn, la, b = O.kda_prologue(g["q"], g["k"], g["g"], g["beta"], a_log=g["a_log"], dt_bias=g["dt_bias"].reshape(-1))
    torch.testing.assert_close(qn, g["qn"], atol=0, rtol=0)
    torch.testing.assert_close(kn, g["kn"], atol=0, rtol=0)
    torch.testing.assert_close(la, g["log_alpha"], atol=0, rtol=0)


@pytest.mark.parametrize("case", ["small", "reject", "midpoint"])
def test_guarded_diagonal_matches_reference(golden_dir, case):
    g = _load(golden_dir, "guarded_diagonal.pt")[case]
    ex = O.diagonal_exact_oracle(*g["inputs"])
    for a, b in zip(ex, g["exact"]):
        torch.testing.assert_close(a, b, atol=1e-6, rtol=1e-6)
    if g["policy"] == "midpoint":
        dq, dk, dkt, hits = O.diagonal_guarded_oracle(*g["inputs"], max_log2_span=g["thr"])
        assert hits.tolist() == g["hits"].tolist()
        for a, b in zip((dq, dk, dkt), g["guarded"]):
            torch.testing.assert_close(a, b, atol=2e-5, rtol=2e-5)
    else:
        hits, _ = O.diagonal_guard_oracle(g["inputs"][0], g["thr"])
        assert hits.tolist() == g["hits"].tolist()


def test_guard_threshold_validation(golden_dir):
    g = _load(golden_dir, "guarded_diagonal.pt")["small"]
    for thr in (-1.0, 0.0, 252.0, float("inf")):
        with pytest.raises(ValueError):
            O.diagonal_guarded_oracle(*g["inputs"], max_log2_span=thr)


def test_gate_spans_conv_normgate(golden_dir):
    m = _load(golden_dir, "misc.pt")
    for s in m["spans"]:
        torch.testing.assert_close(O.gate_tile_spans_oracle(s["raw"], s["a_log"], s["dt_bias"]), s["out"])
    torch.testing.assert_close(m["spans"][0]["out"], torch.full((4,), 15.0))
    c = m["conv"]
    torch.testing.assert_close(O.short_conv_oracle(c["x"], c["weight"]), c["out"], atol=1e-6, rtol=1e-6)
    n = m["norm_gate"]
    torch.testing.assert_close(O.rms_norm_gate_oracle(n["x"], n["gate"], n["weight"]), n["out"], atol=1e-6, rtol=1e-6)


def test_norm_gate_128_and_sublayer_match_reference(golden_dir):
    """The head width the kernels serve, and the whole sublayer composition, against results of
    the reference's own modules (HeadwiseRMSNormGate, KimiDeltaAttention on its reference branch)."""
    n = _load(golden_dir, "misc.pt")["norm_gate_128"]
    x, g, w = (n[k].clone().requires_grad_(True) for k in ("x", "gate", "weight"))
    y = O.rms_norm_gate_oracle(x, g, w)
    y.backward(n["dy"])
    for a, b in ((y.detach(), n["out"]), (x.grad, n["dx"]), (g.grad, n["dgate"]), (w.grad, n["dweight"])):
        torch.testing.assert_close(a, b, atol=1e-6, rtol=1e-5)
    s = _load(golden_dir, "sublayer.pt")
    params = {k: v.clone().requires_grad_(True) for k, v in s["state"].items()}
    xs = s["x"].clone().requires_grad_(True)
    ys = O.kda_sublayer_oracle(xs, params, n_heads=2, head_dim=128)
    ys.backward(s["dy"])
    torch.testing.assert_close(ys.detach(), s["out"], atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(xs.grad, s["dx"], atol=1e-5, rtol=1e-4)
    for k, v in s["grads"].items():
        torch.testing.assert_close(params[k].grad, v, atol=1e-4, rtol=1e-4, msg=lambda m, k=k: f"{k}: {m}")


def test_state_extensions_against_fla_naive():
    """Secondary check of what the reference's oracle does not cover (initial state, final state):
    the third-party ``fla.ops.kda.naive.naive_recurrent_kda`` (upstream FLA, not the pinned fork),
    where it is installed.  Test-only; skipped if the package or its signature is unavailable."""
    naive = pytest.importorskip("fla.ops.kda.naive", reason="flash-linear-attention is not installed")
    fn = getattr(naive, "naive_recurrent_kda", None)
    if fn is None:
        pytest.skip("naive_recurrent_kda is not in this FLA version")
    d = O.make_inputs(2, 70, 2, 16, seed=9, fused=False)
    h0 = torch.randn(2, 2, 16, 16, generator=torch.Generator().manual_seed(10)) * 0.3
    o, s = O.kda_recurrent_oracle(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=h0, output_final_state=True,
                                  scale=16 ** -0.5)
    try:
        o2, s2 = fn(d["q"], d["k"], d["v"], d["g"], d["beta"], scale=16 ** -0.5, initial_state=h0, output_final_state=True)
    except TypeError as e:  # a different signature in another FLA version
        pytest.skip(f"naive_recurrent_kda signature differs: {e}")
    torch.testing.assert_close(o, o2.to(o.dtype), atol=2e-5, rtol=2e-5)
    torch.testing.assert_close(s, s2.to(s.dtype), atol=2e-5, rtol=2e-5)


def test_state_extensions_are_consistent():
    """h0 / final state / cu_seqlens have no reference counterpart: check them against the
    recurrence itself (running two halves with the carried state equals one run; packed
    documents equal separate runs)."""
    d = O.make_inputs(1, 96, 2, 16, seed=3, fused=False)
    o_full, s_full = O.kda_recurrent_oracle(d["q"], d["k"], d["v"], d["g"], d["beta"], output_final_state=True)
    sl = lambda t, a, b: t[:, a:b]
    o1, s1 = O.kda_recurrent_oracle(*(sl(d[n], 0, 40) for n in ("q", "k", "v", "g", "beta")), output_final_state=True)
    o2, s2 = O.kda_recurrent_oracle(*(sl(d[n], 40, 96) for n in ("q", "k", "v", "g", "beta")), initial_state=s1,
                                    output_final_state=True)
    torch.testing.assert_close(torch.cat([o1, o2], 1), o_full, atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(s2, s_full, atol=1e-6, rtol=1e-5)
    cu = torch.tensor([0, 40, 96])
    h0 = torch.randn(2, 2, 16, 16) * 0.1
    op, sp = O.kda_recurrent_oracle(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=h0, cu_seqlens=cu,
                                    output_final_state=True)
    oa, sa = O.kda_recurrent_oracle(*(sl(d[n], 0, 40) for n in ("q", "k", "v", "g", "beta")), initial_state=h0[:1],
                                    output_final_state=True)
    ob, sb = O.kda_recurrent_oracle(*(sl(d[n], 40, 96) for n in ("q", "k", "v", "g", "beta")), initial_state=h0[1:],
                                    output_final_state=True)
    torch.testing.assert_close(op, torch.cat([oa, ob], 1), atol=0, rtol=0)
    torch.testing.assert_close(sp, torch.cat([sa, sb], 0), atol=0, rtol=0)
