"""Pins the tcgen05 operand conventions the tensor-core kernels rely on: the core-matrix
shared-memory layout read as a K-major or MN-major operand, the A operand taken from tensor
memory, operand negation, and where the rows of an M=64 accumulator land in tensor memory."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(N, K, a_mode, b_mode, neg=0, M=128):
    from openkimi_b200 import _lib

    lib = _lib.load()
    gen = torch.Generator().manual_seed(N * 1000 + K * 10 + a_mode * 2 + b_mode)
    A = torch.randn(128, K, generator=gen).cuda()
    B = torch.randn(K, N, generator=gen).cuda()
    if M == 64:
        A[64:] = 0
    D = torch.zeros(128, N, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    if a_mode == 0:      # K-major: next 8 k = 128 B, next 8 rows = (K/8)*128 B, one K=16 step = 256 B
        lbo_a, sbo_a, step_a = 128, (K // 8) * 128, 256
    else:                # MN-major: next 8 rows = 128 B, next 8 k = (128/8)*128 B
        sbo_a, lbo_a = 128, 2048
        step_a = 2 * lbo_a
    if b_mode == 0:
        lbo_b, sbo_b, step_b = 128, (K // 8) * 128, 256
    else:
        sbo_b, lbo_b = 128, (N // 8) * 128
        step_b = 2 * lbo_b
    rc = lib.kda_selftest_mma(A.data_ptr(), B.data_ptr(), D.data_ptr(), N, K, a_mode, b_mode, lbo_a, sbo_a, step_a,
                              lbo_b, sbo_b, step_b, neg, M, st.data_ptr(), None)
    torch.cuda.synchronize()
    assert rc == 0 and int(st.item()) == 0
    ref = (A.bfloat16().float() @ B.bfloat16().float()) * (-1 if neg else 1)
    return D, ref


@pytest.mark.parametrize("N,K", [(64, 64), (128, 128), (64, 128), (128, 64), (16, 48), (32, 64)])
@pytest.mark.parametrize("a_mode", [0, 1, 2])
@pytest.mark.parametrize("b_mode", [0, 1])
def test_operand_views(N, K, a_mode, b_mode):
    D, ref = _run(N, K, a_mode, b_mode)
    assert float((D - ref).abs().max() / ref.abs().max()) < 1e-5


@pytest.mark.parametrize("a_mode", [0, 2])
def test_negated_operand(a_mode):
    D, ref = _run(64, 64, a_mode, 0, neg=1)
    assert float((D - ref).abs().max() / ref.abs().max()) < 1e-5


def test_m64_accumulator_rows():
    """Row r of an M=64 accumulator lives in TMEM lane 32*(r/16) + r%16; other lanes untouched."""
    D, ref = _run(64, 64, 0, 0, M=64)
    lanes = [32 * (r // 16) + r % 16 for r in range(64)]
    assert float((D[lanes] - ref[:64]).abs().max() / ref.abs().max()) < 1e-5
    others = [l for l in range(128) if l not in lanes]
    assert float(D[others].abs().max()) == 0.0


def test_rejects_strides_outside_the_tile():
    from openkimi_b200 import _lib

    lib = _lib.load()
    z = torch.zeros(128 * 128, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert lib.kda_selftest_mma(z.data_ptr(), z.data_ptr(), z.data_ptr(), 64, 64, 0, 0, 128, 8192, 256, 128, 1024, 256,
                                0, 128, st.data_ptr(), None) == 2
