"""The recurrent decoding step (one token per (sequence, head), state in / state out) against the
CPU oracle of the recurrence (k3mini/model.py:121-128) and against ``chunk_kda`` over the same
tokens: T decode steps must reproduce the chunked op's outputs and final state."""
import pytest
import torch

from openkimi_b200.synthetic import make_inputs
from tests.kda_testlib import max_rel, rel_l2, run_oracle

pytestmark = pytest.mark.gpu


def _decode(inp, h0, vfirst, T0=0):
    from openkimi_b200 import fused_recurrent_kda

    tr = (lambda s: s.transpose(-1, -2).contiguous()) if vfirst else (lambda s: s)
    d = {k: v.cuda() for k, v in inp.items() if isinstance(v, torch.Tensor)}
    o, s = fused_recurrent_kda(d["q"][:, T0:], d["k"][:, T0:], d["v"][:, T0:], d["g"][:, T0:], d["beta"][:, T0:],
                               initial_state=None if h0 is None else tr(h0.cuda()), output_final_state=True,
                               A_log=d["a_log"], dt_bias=d["dt_bias"], use_qk_l2norm_in_kernel=True,
                               use_gate_in_kernel=True, use_beta_sigmoid_in_kernel=True, state_v_first=vfirst)
    return o, tr(s)


@pytest.mark.parametrize("dtype,d,tol", [(torch.float32, 64, 1e-4), (torch.float32, 128, 1e-4), (torch.bfloat16, 128, 2e-2)])
@pytest.mark.parametrize("vfirst", [False, True])
def test_decode_steps_match_the_oracle(dtype, d, tol, vfirst):
    inp = make_inputs(2, 24, 3, d, seed=41, dtype=dtype)
    h0 = torch.randn(2, 3, d, d, generator=torch.Generator().manual_seed(42)) * 0.1
    ref = run_oracle(inp, h0=h0)
    o, s = _decode(inp, h0, vfirst)
    assert torch.isfinite(o.float()).all()
    assert max_rel(o, ref["o"]) <= tol and rel_l2(o, ref["o"]) <= tol, (max_rel(o, ref["o"]), rel_l2(o, ref["o"]))
    assert max_rel(s, ref["ht"]) <= tol and rel_l2(s, ref["ht"]) <= tol


def test_prefill_with_chunk_kda_then_decode_equals_one_chunked_run():
    """chunk_kda over 150 prompt tokens, then 20 decode steps from its final state, against chunk_kda over
    all 170 tokens (BF16 operands: the two paths round differently, so the BF16 bound applies)."""
    from openkimi_b200 import chunk_kda

    inp = make_inputs(2, 170, 2, 128, seed=43, dtype=torch.bfloat16)
    d = {k: v.cuda() for k, v in inp.items() if isinstance(v, torch.Tensor)}
    kw = dict(A_log=d["a_log"], dt_bias=d["dt_bias"], use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True,
              use_beta_sigmoid_in_kernel=True, output_final_state=True, state_v_first=True)
    with torch.no_grad():
        o_all, s_all = chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], **kw)
        o_pre, s_pre = chunk_kda(*(d[n][:, :150] for n in ("q", "k", "v", "g", "beta")), **kw)
    o_dec, s_dec = _decode(inp, s_pre.transpose(-1, -2).cpu(), True, T0=150)
    assert torch.equal(o_pre, o_all[:, :150])
    assert rel_l2(o_dec, o_all[:, 150:]) < 7e-3 and max_rel(o_dec, o_all[:, 150:]) < 2e-2
    assert rel_l2(s_dec, s_all.transpose(-1, -2)) < 7e-3


def test_in_place_state_update_and_argument_checks():
    from openkimi_b200 import recurrent_kda_step

    from oracle.kda_oracle import make_inputs as oracle_inputs

    inp = oracle_inputs(3, 1, 2, 128, seed=44, dtype=torch.bfloat16, fused=False)  # normalised q/k, log decay, beta
    a = [inp[n][:, 0].cuda() for n in ("q", "k", "v", "g", "beta")]
    s = torch.randn(3, 2, 128, 128, device="cuda") * 0.1
    o1, s1 = recurrent_kda_step(*a, s)
    s2 = s.clone()
    o2, s3 = recurrent_kda_step(*a, s2, inplace=True)
    assert s3.data_ptr() == s2.data_ptr() and torch.equal(s1, s2) and torch.equal(o1, o2)
    with pytest.raises(ValueError):
        recurrent_kda_step(*a, s[:, :, :64])
    with pytest.raises(RuntimeError):
        recurrent_kda_step(*(t.cpu() for t in a), s.cpu())
