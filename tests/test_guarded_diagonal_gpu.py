"""The reference's guarded-diagonal tests (tests/test_kda_guarded_diagonal.py) against the CUDA
tile kernel, on the golden inputs/outputs produced by the reference's own oracle."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _gold(golden_dir):
    return torch.load(os.path.join(golden_dir, "guarded_diagonal.pt"), weights_only=False)


def _run(inputs, span):
    from openkimi_b200 import guarded_diagonal_backward

    return guarded_diagonal_backward(*(t.cuda() for t in inputs), max_log2_span=span)


def test_factorisation_matches_pairwise_oracle(golden_dir):
    g = _gold(golden_dir)["small"]                       # spans 2, 8, 16 at threshold 20
    res = _run(g["inputs"], g["thr"])
    assert res.guard_hits.tolist() == [True, True, True]
    for a, b in zip((res.dq, res.dk, res.dkt), g["exact"]):
        torch.testing.assert_close(a.cpu(), b, atol=2e-4, rtol=2e-4)


def test_rejected_tiles_are_bit_identical_to_the_exact_path(golden_dir):
    g = _gold(golden_dir)["reject"]                      # span 200 and a non-monotone tile at threshold 20
    res = _run(g["inputs"], g["thr"])
    exact = _run(g["inputs"], -1.0)
    assert res.guard_hits.tolist() == [True, False, False]
    assert exact.guard_hits.tolist() == [False, False, False]
    for a, b in zip((res.dq, res.dk, res.dkt), (exact.dq, exact.dk, exact.dkt)):
        assert torch.equal(a[1:], b[1:])
    for a, b in zip((exact.dq, exact.dk, exact.dkt), g["exact"]):
        torch.testing.assert_close(a.cpu(), b, atol=2e-4, rtol=2e-4)


def test_midpoint_supports_large_spans(golden_dir):
    g = _gold(golden_dir)["midpoint"]                    # spans 100, 200, 251 at threshold 240
    res = _run(g["inputs"], g["thr"])
    assert res.guard_hits.tolist() == g["hits"].tolist() == [True, True, False]
    for a, b in zip((res.dq, res.dk, res.dkt), g["guarded"]):
        torch.testing.assert_close(a.cpu(), b, atol=2e-4, rtol=2e-4)


@pytest.mark.parametrize("threshold", [252.0, float("inf"), float("nan")])
def test_threshold_validation(golden_dir, threshold):
    g = _gold(golden_dir)["small"]
    with pytest.raises(ValueError):
        _run(g["inputs"], threshold)


def test_gate_tile_spans_closed_form_and_golden(golden_dir):
    from openkimi_b200 import gate_tile_spans

    m = torch.load(os.path.join(golden_dir, "misc.pt"), weights_only=False)
    for s in m["spans"]:
        out = gate_tile_spans(s["raw"].cuda(), s["a_log"].cuda(), s["dt_bias"].cuda())
        torch.testing.assert_close(out.cpu(), s["out"], atol=1e-4, rtol=1e-5)
    torch.testing.assert_close(m["spans"][0]["out"], torch.full((4,), 15.0))
