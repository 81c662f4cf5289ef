"""The benchmark configurations at their full sizes, checked through properties that do not
need the (slow) CPU oracle: the op is linear in v, a sequence cut in two with the state
carried over equals the uncut run, packed documents equal separate runs, two runs are
bit-identical, and rejected guard tiles give the same bits with the guard on or off.  One
full-length sequence is also compared with the oracle directly."""
import pytest
import torch

from openkimi_b200.synthetic import make_inputs, random_cu_seqlens
from tests.kda_testlib import assert_rows, compare, rel_l2, run_device, run_oracle

pytestmark = pytest.mark.gpu

C1 = dict(batch=16, time=2048, heads=6, dim=128)


def _fwd(inp, **kw):
    from openkimi_b200 import chunk_kda

    d = {k: v.cuda() for k, v in inp.items() if isinstance(v, torch.Tensor)}
    with torch.no_grad():
        return chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], A_log=d["a_log"], dt_bias=d["dt_bias"],
                         use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, use_beta_sigmoid_in_kernel=True,
                         output_final_state=True, **kw)


def test_c1_linear_in_v():
    """o and the final state are linear in v for fixed q, k, g, beta (the delta rule's
    correction k (beta (v - k^T S)) is affine in v and the state starts at zero)."""
    inp = make_inputs(**C1, seed=0, dtype=torch.bfloat16)
    gen = torch.Generator().manual_seed(5)
    v2 = torch.randn(inp["v"].shape, generator=gen).bfloat16()
    o1, s1 = _fwd(inp)
    o2, s2 = _fwd(dict(inp, v=v2))
    o12, s12 = _fwd(dict(inp, v=(inp["v"].float() + v2.float()).bfloat16()))
    assert rel_l2(o12, o1.float() + o2.float()) < 8e-3
    assert rel_l2(s12, s1 + s2) < 8e-3


def test_c1_split_sequence_with_carried_state_is_bit_identical():
    inp = make_inputs(**C1, seed=1, dtype=torch.bfloat16)
    o, s = _fwd(inp)
    cut = 1024
    first = {k: (v[:, :cut] if v.dim() >= 3 else v) for k, v in inp.items()}
    second = {k: (v[:, cut:] if v.dim() >= 3 else v) for k, v in inp.items()}
    oa, sa = _fwd(first)
    ob, sb = _fwd(second, initial_state=sa)
    assert torch.equal(torch.cat([oa, ob], 1), o)
    assert torch.equal(sb, s)


def test_c1_two_runs_bit_identical_forward_and_backward():
    inp = make_inputs(**C1, seed=2, dtype=torch.bfloat16)
    a = run_device(inp)
    b = run_device(inp)
    for n in a:
        if a[n] is not None:
            assert torch.isfinite(a[n].float()).all(), n
            assert torch.equal(a[n], b[n]), n


def test_c3_packed_documents_equal_separate_runs():
    """65 536 packed tokens, 16 documents of ragged length with their own initial states:
    every document must come out exactly as if it had been run alone."""
    total, docs, H, d = 65536, 16, 6, 128
    inp = make_inputs(1, total, H, d, seed=3, dtype=torch.bfloat16)
    cu = random_cu_seqlens(total, docs, seed=3)
    gen = torch.Generator().manual_seed(4)
    h0 = torch.randn(docs, H, d, d, generator=gen) * 0.02
    dht = torch.randn(docs, H, d, d, generator=gen) * 0.02
    packed = run_device(inp, h0=h0, dht=dht, cu=cu, state_v_first=True)
    for n in (0, 7, 15):
        a, b = int(cu[n]), int(cu[n + 1])
        one = {k: (v[:, a:b] if v.dim() >= 3 else v) for k, v in inp.items()}
        alone = run_device(one, h0=h0[n:n + 1], dht=dht[n:n + 1], state_v_first=True)
        for name in ("o", "dq", "dk", "dv", "dg", "dbeta"):
            assert torch.equal(packed[name][:, a:b], alone[name]), (n, name)
        assert torch.equal(packed["ht"][n:n + 1], alone["ht"])
        assert torch.equal(packed["dh0"][n:n + 1], alone["dh0"])
    for name in ("dA_log", "ddt_bias"):
        assert torch.isfinite(packed[name]).all()


def test_c2_adversarial_span_guard_on_and_off_bit_identical():
    """x ~ N(3,1), A_log ~ U(ln 8, ln 64): every diagonal tile exceeds the 232 span, so the
    guarded run must take the exact path everywhere and reproduce the unguarded bits."""
    from openkimi_b200 import chunk_intra

    inp = make_inputs(4, 4096, 6, 128, seed=6, dtype=torch.bfloat16, x_mean=3.0, a_lo=8.0, a_hi=64.0, beta_mean=2.0)
    old = chunk_intra._OPENKIMI_GUARD_MAX_LOG2_SPAN
    try:
        chunk_intra._OPENKIMI_GUARD_MAX_LOG2_SPAN = 232.0
        a = run_device(inp)
        chunk_intra._OPENKIMI_GUARD_MAX_LOG2_SPAN = -1.0
        b = run_device(inp)
    finally:
        chunk_intra._OPENKIMI_GUARD_MAX_LOG2_SPAN = old
    for n in a:
        if a[n] is not None:
            assert torch.isfinite(a[n].float()).all(), n
            assert torch.equal(a[n], b[n]), n


def test_full_length_sequence_against_oracle():
    """One sequence of the primary profile's length (T = 2048, d = 128, 2 heads) against the
    recurrent oracle: 32 chunks of state carry-over in both directions."""
    inp = make_inputs(1, 2048, 2, 128, seed=7, dtype=torch.bfloat16)
    ref = run_oracle(inp)
    dev = run_device(inp)
    rows = compare(dev, ref, tol_max=2e-2, tol_l2=7e-3)
    assert_rows(rows)
    assert dict((r[0], r[2]) for r in rows)["o"] < 5e-3


def test_c1_shape_two_sequences_six_heads_against_oracle():
    """Configuration 1's head count and length, two of its sixteen sequences ([2,2048,6,128], BF16) against
    the recurrent oracle; the oracle runs one sequence at a time (its autograd graph holds ~3 GB each)."""
    inp = make_inputs(2, 2048, 6, 128, seed=8, dtype=torch.bfloat16)
    dev = run_device(inp)
    refs = []
    for b in range(2):
        one = {k: (v[b:b + 1] if v.dim() >= 3 else v) for k, v in inp.items()}
        refs.append(run_oracle(one))
    ref = {k: (refs[0][k] + refs[1][k] if k in ("dA_log", "ddt_bias") else torch.cat([refs[0][k], refs[1][k]], 0))
           for k in refs[0]}
    rows = compare(dev, ref, tol_max=2e-2, tol_l2=7e-3)
    assert_rows(rows)
    assert dict((r[0], r[2]) for r in rows)["o"] < 5e-3


@pytest.mark.parametrize("B,T,H", [(3, 512, 7), (7, 320, 5)])
def test_more_units_than_sms_with_odd_head_counts_against_oracle(B, T, H):
    """The per-unit kernels run one CTA per SM that walks units first, first + #SMs, ...; with head counts that
    share no factor with the SM count (and more units than SMs: 168 and 175 chunk-head pairs) every CTA
    meets several heads and several sequences, and some CTAs get one unit more than others."""
    inp = make_inputs(B, T, H, 128, seed=60 + H, dtype=torch.bfloat16)
    dev = run_device(inp)
    refs = []
    for b in range(B):
        one = {k: (v[b:b + 1] if v.dim() >= 3 else v) for k, v in inp.items()}
        refs.append(run_oracle(one))
    ref = {k: (sum(r[k] for r in refs) if k in ("dA_log", "ddt_bias") else torch.cat([r[k] for r in refs], 0)) for k in refs[0]}
    assert_rows(compare(dev, ref, tol_max=2e-2, tol_l2=7e-3))
