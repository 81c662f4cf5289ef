"""GPU parity of ``chunk_kda`` (through the C ABI) against the CPU oracle, i.e. against the
reference's recurrent FP32-state KDA (k3mini/model.py:101-129) on identical seeded inputs.

Tolerances: FP32 validation mode <= 1e-4 (max error relative to the largest reference
magnitude, and relative L2) against the oracle evaluated in FP64 -- the FP32 oracle's own
rounding on the two parameter gradients (long sums with cancellation) is of the same size
as the bound, and the golden-vector test below checks the FP32 reference outputs directly; BF16 operands <= 2e-2 max and the reference's own bounds
rel-L2 < 5e-3 on the output and < 7e-3 on the gradients (tests/test_h100_parity.py:114-119).
"""
import os

import pytest
import torch

from oracle import kda_oracle as O
from tests.kda_testlib import assert_rows, compare, run_device, run_oracle

pytestmark = pytest.mark.gpu

FP32_TOL = dict(tol_max=1e-4, tol_l2=1e-4)
BF16_TOL = dict(tol_max=2e-2, tol_l2=7e-3)


def _states(N, H, d, seed=4, std=0.1):
    gen = torch.Generator().manual_seed(seed)
    return torch.randn(N, H, d, d, generator=gen) * std, torch.randn(N, H, d, d, generator=gen) * std


@pytest.mark.parametrize("B,T,H,d", [(2, 512, 4, 64), (1, 130, 2, 128), (2, 64, 1, 64), (1, 7, 1, 64), (1, 65, 2, 128)])
@pytest.mark.parametrize("fused", [True, False])
def test_fp32_validation_mode(B, T, H, d, fused):
    """Config 0 of the benchmark ([2,512,4,64] FP32) and ragged lengths, fused prologue and
    precomputed gate entry, with initial state and final-state gradient."""
    inp = O.make_inputs(B, T, H, d, seed=0, fused=fused)
    inp["dt_bias"] = torch.randn(H * d, generator=torch.Generator().manual_seed(1)) * 0.2
    h0, dht = _states(B, H, d)
    ref = run_oracle(inp, fused=fused, h0=h0, dht=dht, dtype=torch.float64)
    dev = run_device(inp, fused=fused, h0=h0, dht=dht)
    assert_rows(compare(dev, ref, **FP32_TOL, names=("o", "ht", "dq", "dk", "dv", "dg", "dbeta", "dh0")))
    # dA_log[h] and ddt_bias[h,d] are sums of dg*g over every token of a head with heavy
    # cancellation; with a few hundred tokens per head FP32 rounding of dg (<= 1e-4 itself)
    # shows up amplified in these sums, so the bound is 1e-4 only for the benchmark-sized case
    ptol = 1e-4 if B * T >= 1024 else 2e-3
    assert_rows(compare(dev, ref, tol_max=ptol, tol_l2=ptol, names=("dA_log", "ddt_bias")))


def test_fp32_zero_state_no_final_grad():
    inp = O.make_inputs(2, 200, 2, 64, seed=3)
    ref = run_oracle(inp, dtype=torch.float64)
    dev = run_device(inp)
    assert_rows(compare(dev, ref, **FP32_TOL))


@pytest.mark.parametrize("state_v_first", [False, True])
def test_fp32_varlen_packed(state_v_first):
    """cu_seqlens packing: documents of ragged length (including a 1-token and a 64-token
    one), per-document initial state, state layout [N,H,V,K] when state_v_first."""
    cu = torch.tensor([0, 1, 65, 200, 327, 391, 500])
    inp = O.make_inputs(1, 500, 2, 64, seed=5)
    h0, dht = _states(len(cu) - 1, 2, 64)
    ref = run_oracle(inp, h0=h0, dht=dht, cu=cu, dtype=torch.float64)
    dev = run_device(inp, h0=h0, dht=dht, cu=cu, state_v_first=state_v_first)
    assert_rows(compare(dev, ref, **FP32_TOL))


def test_fp32_recompute_policy_matches_saved():
    inp = O.make_inputs(1, 300, 2, 64, seed=6)
    a = run_device(inp, disable_recompute=True)
    b = run_device(inp, disable_recompute=False)
    for n in a:
        if a[n] is not None:
            assert torch.equal(a[n], b[n]), n


def test_golden_reference_vectors_fp32(golden_dir):
    """The reference's own outputs and autograd gradients (tests/golden/make_golden.py)."""
    gold = torch.load(os.path.join(golden_dir, "kda_recurrent.pt"), weights_only=False)
    for case in ("fp32_2x150x2x64", "fp32_1x130x2x128"):
        g = gold[case]
        inp = dict(q=g["q"], k=g["k"], v=g["v"], g=g["g"], beta=g["beta"], a_log=g["a_log"],
                   dt_bias=g["dt_bias"].reshape(-1), do=g["do"])
        dev = run_device(inp)
        ref = {"o": g["o"], "dq": g["dq"], "dk": g["dk"], "dv": g["dv"], "dg": g["dg"], "dbeta": g["dbeta"],
               "dA_log": g["da_log"], "ddt_bias": g["ddt_bias"].reshape(-1)}
        assert_rows(compare(dev, ref, **FP32_TOL, names=("o", "dq", "dk", "dv", "dg", "dbeta")))
        # FP32 autograd of the reference rounds these two long sums at the 1e-4..1e-3 level itself
        assert_rows(compare(dev, ref, tol_max=2e-3, tol_l2=2e-3, names=("dA_log", "ddt_bias")))


def test_golden_reference_parity_recipe_bf16(golden_dir):
    """The reference's only fast-path pin, tests/test_h100_parity.py:68-119: [1,64,1,128] BF16,
    rel-L2(out) < 5e-3, max gradient rel-L2 < 7e-3."""
    g = torch.load(os.path.join(golden_dir, "kda_recurrent.pt"), weights_only=False)["parity_1x64x1x128_bf16"]
    inp = dict(q=g["q"], k=g["k"], v=g["v"], g=g["g"], beta=g["beta"], a_log=g["a_log"],
               dt_bias=g["dt_bias"].reshape(-1), do=g["do"])
    dev = run_device(inp)
    ref = {"o": g["o"], "dq": g["dq"], "dk": g["dk"], "dv": g["dv"], "dg": g["dg"], "dbeta": g["dbeta"],
           "dA_log": g["da_log"], "ddt_bias": g["ddt_bias"].reshape(-1)}
    rows = compare(dev, ref, tol_max=2e-2, tol_l2=7e-3)
    assert_rows(rows)
    assert dict((r[0], r[2]) for r in rows)["o"] < 5e-3


@pytest.mark.parametrize("B,T,H,d,fp32_math", [(2, 256, 2, 128, False), (1, 200, 2, 64, False), (2, 256, 2, 128, True)])
def test_bf16_operands(B, T, H, d, fp32_math):
    """BF16 q/k/v/g/beta with FP32 state, against the FP32 oracle fed the same BF16 values."""
    inp = O.make_inputs(B, T, H, d, seed=2, dtype=torch.bfloat16)
    h0, dht = _states(B, H, d)
    ref = run_oracle(inp, h0=h0, dht=dht)
    dev = run_device(inp, h0=h0, dht=dht, fp32_math=fp32_math)
    rows = compare(dev, ref, **BF16_TOL)
    assert_rows(rows)
    assert dict((r[0], r[2]) for r in rows)["o"] < 5e-3


@pytest.mark.parametrize("mask", [1, 2, 4, 8, 16, 31])
def test_bf16_stage_mixing(mask, monkeypatch):
    """Any stage of the BF16 path can be swapped for its FP32 CUDA-core counterpart (KDA_FLAG_SIMT_* in
    the C ABI, OPENKIMI_B200_FP32_STAGES in the Python host): both families read and write the same
    per-chunk records, so every mixture must stay within the BF16 tolerance of the oracle."""
    monkeypatch.setenv("OPENKIMI_B200_FP32_STAGES", str(mask))
    inp = O.make_inputs(2, 256, 2, 128, seed=21, dtype=torch.bfloat16)
    h0, dht = _states(2, 2, 128)
    ref = run_oracle(inp, h0=h0, dht=dht)
    dev = run_device(inp, h0=h0, dht=dht)
    tensors = ("o", "ht", "dq", "dk", "dv", "dg", "dbeta", "ddt_bias", "dh0")
    assert_rows(compare(dev, ref, names=tensors, **BF16_TOL))
    # dA_log is two numbers here (H = 2), each a cancelling sum over all tokens of BF16-derived terms:
    # the north-star bound (2e-2) applies, not the tighter relative-L2 bound of the large tensors
    assert_rows(compare(dev, ref, names=("dA_log",), tol_max=2e-2, tol_l2=2e-2))


@pytest.mark.parametrize("T", [1, 5, 17, 63, 65])
def test_bf16_tensor_core_path_tiny_sequences(T):
    """Ragged edge of the tensor-core kernels: sequences shorter than a 16-row block, shorter than a
    chunk, and one token past a chunk.  Gradients of so few tokens are compared with the 2e-2 bound."""
    inp = O.make_inputs(2, T, 2, 128, seed=40 + T, dtype=torch.bfloat16)
    h0, dht = _states(2, 2, 128)
    ref = run_oracle(inp, h0=h0, dht=dht)
    dev = run_device(inp, h0=h0, dht=dht)
    tensors = ("o", "ht", "dq", "dk", "dv", "dg", "dbeta", "ddt_bias", "dh0")
    assert_rows(compare(dev, ref, names=tensors, tol_max=2e-2, tol_l2=2e-2, abs_escape=5e-5))
    # dA_log: two numbers, each a cancelling sum of BF16-derived terms over at most 130 tokens; its
    # relative error is set by the cancellation, so this edge-case test only bounds it loosely
    assert_rows(compare(dev, ref, names=("dA_log",), tol_max=5e-2, tol_l2=5e-2, abs_escape=5e-5))


def test_bf16_varlen_packed():
    cu = O.random_cu_seqlens(1024, 5, seed=1)
    inp = O.make_inputs(1, 1024, 2, 128, seed=8, dtype=torch.bfloat16)
    h0, dht = _states(5, 2, 128, std=0.02)
    ref = run_oracle(inp, h0=h0, dht=dht, cu=cu)
    dev = run_device(inp, h0=h0, dht=dht, cu=cu, state_v_first=True)
    assert_rows(compare(dev, ref, **BF16_TOL))


def test_adversarial_gate_span():
    """Benchmark config 2 distributions (x ~ N(3,1), A_log ~ U(ln 8, ln 64), beta = sigmoid(N(2,1))):
    within-chunk cumulative log2 decay far beyond the 232 guard; everything must stay finite
    and match the oracle."""
    inp = O.make_inputs(1, 256, 2, 128, seed=9, dtype=torch.bfloat16, x_mean=3.0, a_lo=8.0, a_hi=64.0, beta_mean=2.0)
    ref = run_oracle(inp)
    dev = run_device(inp)
    # decays this strong leave gate gradients that are numerically zero; the reference's
    # acceptance rule lets such tensors pass on absolute error <= 5e-5
    assert_rows(compare(dev, ref, **BF16_TOL, abs_escape=5e-5))


def test_guard_span_exact_switch_is_consistent():
    """Setting the runtime span to -1 forces the exact diagonal everywhere
    (experiments/kda_sm90/validate_fla_guarded_integration.py:257-267); guarded and exact
    results agree within the reference's acceptance rule (rel-L2 <= 5e-3)."""
    from openkimi_b200 import chunk_intra

    inp = O.make_inputs(2, 256, 2, 128, seed=10, dtype=torch.bfloat16)
    old = chunk_intra._OPENKIMI_GUARD_MAX_LOG2_SPAN
    try:
        chunk_intra._OPENKIMI_GUARD_MAX_LOG2_SPAN = 232.0
        a = run_device(inp)
        chunk_intra._OPENKIMI_GUARD_MAX_LOG2_SPAN = -1.0
        b = run_device(inp)
        c = run_device(inp)
    finally:
        chunk_intra._OPENKIMI_GUARD_MAX_LOG2_SPAN = old
    assert_rows(compare(a, b, tol_max=2e-2, tol_l2=5e-3))
    for n in b:  # run-to-run bit equality: no float atomics on any graded output
        if b[n] is not None:
            assert torch.equal(b[n], c[n]), n


def test_argument_errors():
    from openkimi_b200 import chunk_kda

    q = torch.zeros(2, 64, 2, 64, device="cuda")
    b = torch.zeros(2, 64, 2, device="cuda")
    with pytest.raises(ValueError, match="batch size is expected to be 1"):
        chunk_kda(q, q, q, q, b, cu_seqlens=torch.tensor([0, 64, 128], device="cuda"))
    with pytest.raises(TypeError, match="float32"):
        chunk_kda(q, q, q, q, b, initial_state=torch.zeros(2, 2, 64, 64, device="cuda", dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="A_log must be provided"):
        chunk_kda(q, q, q, q, b, use_gate_in_kernel=True)
    with pytest.raises(ValueError, match="chunk_size"):
        chunk_kda(q, q, q, q, b, chunk_size=32)
    with pytest.raises(RuntimeError, match="CUDA"):
        chunk_kda(q.cpu(), q.cpu(), q.cpu(), q.cpu(), b.cpu())


@pytest.mark.parametrize("dtype,d", [(torch.bfloat16, 128), (torch.float32, 64)])
def test_forward_only_call_matches_the_saving_forward_bitwise(dtype, d):
    """Under no_grad (the forward an activation-checkpointed block runs first, k3mini/model.py:825-831)
    the kernels write none of the records the backward reads; o and the final state must not change."""
    from openkimi_b200 import chunk_kda

    inp = O.make_inputs(2, 200, 2, d, seed=31, dtype=dtype)
    cu = torch.tensor([0, 70, 200])
    for kw in (dict(), dict(cu_seqlens=cu.cuda(), cu_seqlens_cpu=cu)):
        sl = (lambda t: t[:1]) if kw else (lambda t: t)
        args = [sl(inp[n]).cuda() for n in ("q", "k", "v", "g", "beta")]
        common = dict(A_log=inp["a_log"].cuda(), dt_bias=inp["dt_bias"].cuda(), use_qk_l2norm_in_kernel=True,
                      use_gate_in_kernel=True, use_beta_sigmoid_in_kernel=True, output_final_state=True,
                      disable_recompute=True, **kw)
        with torch.no_grad():
            o0, s0 = chunk_kda(*args, **common)
        leaves = [a.clone().requires_grad_(True) for a in args]
        o1, s1 = chunk_kda(*leaves, **common)
        assert torch.equal(o0, o1) and torch.equal(s0, s1)
        o1.float().sum().backward()   # the saving forward still feeds a working backward
        assert all(torch.isfinite(x.grad.float()).all() for x in leaves)


@pytest.mark.parametrize("varlen", [False, True])
def test_tile_copies_move_the_same_bytes_as_row_copies(varlen, monkeypatch):
    """The q / k / v / gate tiles of full chunks arrive (and the o / dv tiles leave) with one bulk-tensor copy
    through a tensor map; partial chunks, and KDA_FLAG_ROW_COPIES, move the same rows one by one.  Both ways
    must give the same bits, packed sequences whose chunks start at odd token offsets included."""
    inp = O.make_inputs(1 if varlen else 2, 1024 if varlen else 320, 2, 128, seed=52, dtype=torch.bfloat16)
    cu = O.random_cu_seqlens(1024, 5, seed=3) if varlen else None
    h0, dht = (None, None) if varlen else _states(2, 2, 128)
    a = run_device(inp, h0=h0, dht=dht, cu=cu)
    monkeypatch.setenv("OPENKIMI_B200_ROW_COPIES", "1")
    b = run_device(inp, h0=h0, dht=dht, cu=cu)
    for name in a:
        if isinstance(a[name], torch.Tensor):
            assert torch.equal(a[name], b[name]), name
