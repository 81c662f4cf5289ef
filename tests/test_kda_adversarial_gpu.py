"""The reference's adversarial KDA fixtures (experiments/kda_sm90/validate_fla_guarded_integration.py:
149-254) against the CPU oracle and against the exact (guard off) run of the same kernels.

The fixture recipes are the reference's: constant raw gate softplus^-1(decay/16) with A_log = log 16
(so the per-token natural-log decay is ``decay``), random BF16 q, k, v, beta logits and output
gradient; seeds 2401-2405.  Sizes are reduced where the CPU oracle would take minutes (2 heads instead
of 6); the tile structure ([16 rows x 32 channels] guard tiles, 64-token chunks) is unchanged.
Acceptance rule of the reference: rel-L2 <= 5e-3, or max-abs <= 5e-5 for numerically-zero tensors."""
import math

import pytest
import torch

from tests.kda_testlib import assert_rows, compare, run_device, run_oracle

pytestmark = pytest.mark.gpu
H, D = 2, 128
LOG2E = 1.0 / math.log(2.0)


def _base(batch, T, seed, per_token_decay):
    gen = torch.Generator().manual_seed(seed)
    shape = (batch, T, H, D)
    rnd = lambda s: torch.randn(s, generator=gen).bfloat16()
    q, k, v = rnd(shape), rnd(shape), rnd(shape)
    raw = torch.full(shape, math.log(math.expm1(per_token_decay / 16.0))).bfloat16()
    beta = rnd(shape[:-1])
    return dict(q=q, k=k, v=v, g=raw, beta=beta, a_log=torch.full((H,), math.log(16.0)), dt_bias=torch.zeros(H * D),
                do=rnd(shape))


def _guard(span):
    from openkimi_b200 import chunk_intra

    class _Ctx:
        def __enter__(self):
            self.old = chunk_intra._OPENKIMI_GUARD_MAX_LOG2_SPAN
            chunk_intra._OPENKIMI_GUARD_MAX_LOG2_SPAN = span

        def __exit__(self, *a):
            chunk_intra._OPENKIMI_GUARD_MAX_LOG2_SPAN = self.old
    return _Ctx()


def _check(inp, expect_bit_identical, fused=True):
    ref = run_oracle(inp, fused=fused)
    with _guard(232.0):
        guarded = run_device(inp, fused=fused)
    with _guard(-1.0):
        exact = run_device(inp, fused=fused)
    assert_rows(compare(guarded, ref, tol_max=2e-2, tol_l2=7e-3, abs_escape=5e-5))
    assert_rows(compare(exact, ref, tol_max=2e-2, tol_l2=7e-3, abs_escape=5e-5))
    # guarded vs exact: the reference's self-consistency rule
    assert_rows(compare(guarded, exact, tol_max=2e-2, tol_l2=5e-3, abs_escape=5e-5))
    if expect_bit_identical:
        for n in guarded:
            if guarded[n] is not None:
                assert torch.equal(guarded[n], exact[n]), n


def test_near_threshold_accepted():
    """15.2 log2 units per token -> 228 over the 16 rows of a tile: accepted, close to 232."""
    inp = _base(2, 256, 2401, 15.2 / LOG2E)
    _check(inp, expect_bit_identical=False)


def test_high_decay_falls_back_bit_identically():
    """32 per token -> 480 per tile: far beyond the guard, every tile takes the exact path."""
    inp = _base(2, 256, 2402, 32.0 / LOG2E)
    _check(inp, expect_bit_identical=True)


def test_cancellation_heavy():
    inp = _base(2, 1024, 2403, 2.0)
    inp["q"][..., 1::2] = -inp["q"][..., 0::2]
    inp["k"][..., 1::2] = inp["k"][..., 0::2]
    sign = torch.where(torch.arange(1024) % 2 == 0, 1.0, -1.0).bfloat16()
    inp["v"] = inp["v"] * sign[None, :, None, None]
    inp["do"] = inp["do"] * (-sign[None, :, None, None])
    _check(inp, expect_bit_identical=False)


def test_partial_chunk_4103():
    """T = 4103: a final 7-token chunk and a partial 16-row tile."""
    inp = _base(1, 4103, 2404, 4.0)
    _check(inp, expect_bit_identical=False)


def test_nonmonotonic_gate_falls_back_bit_identically():
    """Precomputed gate with a +0.5 step every 16 rows (use_gate_in_kernel=False): not monotone,
    so every tile must be rejected although all decays stay bounded."""
    gen = torch.Generator().manual_seed(2405)
    shape = (2, 256, H, D)
    rnd = lambda s: torch.randn(s, generator=gen).bfloat16()
    q, k, v = rnd(shape), rnd(shape), rnd(shape)
    q = torch.nn.functional.normalize(q.float(), dim=-1).bfloat16()
    k = torch.nn.functional.normalize(k.float(), dim=-1).bfloat16()
    gate = torch.full(shape, -0.25).bfloat16()
    gate[:, 8::16] = 0.5
    beta = torch.sigmoid(rnd(shape[:-1]).float()).bfloat16()
    inp = dict(q=q, k=k, v=v, g=gate, beta=beta, a_log=torch.zeros(H), dt_bias=torch.zeros(H * D), do=rnd(shape))
    _check(inp, expect_bit_identical=True, fused=False)
