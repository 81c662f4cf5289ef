"""A bounded device-side wait that gives up must be audible and must leave the device usable.

The wait is made to run out in the permitted way only: a self-test kernel whose mbarrier is
armed for twice the bytes its single bulk copy delivers, with a short poll limit passed as an
argument.  The kernel records its code in the status word, waits for the copy that is in
flight, frees its tensor memory and returns; nothing hangs, traps or faults."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_that_runs_out_sets_the_status_word_and_the_device_stays_usable():
    from openkimi_b200 import _lib
    from openkimi_b200.synthetic import make_inputs
    from tests.kda_testlib import run_device

    lib = _lib.load()
    src = torch.arange(64, dtype=torch.float32, device="cuda")
    dst = torch.zeros(64, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.kda_selftest_wait(src.data_ptr(), dst.data_ptr(), 64, 5, st.data_ptr(), None)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(st.item()) == 5              # the short wait gave up and said so
    assert torch.equal(dst, src)            # the copy in flight was waited for before the exit
    # tensor memory was freed and the context is healthy: an ordinary call still works
    inp = make_inputs(1, 130, 2, 128, seed=11, dtype=torch.bfloat16)
    a = run_device(inp)
    b = run_device(inp)
    assert torch.isfinite(a["o"].float()).all() and torch.equal(a["o"], b["o"])


def test_status_word_of_the_op_surfaces_as_an_error():
    """The host passes one status word per device in KdaParams.status; a non-zero word raises
    RuntimeError(kda_status_string(KDA_ERR_DEVICE_WAIT)) at the next poll and is cleared."""
    from openkimi_b200 import check_device_status
    from openkimi_b200.ops import _DeviceStatus
    from openkimi_b200.synthetic import make_inputs
    from tests.kda_testlib import run_device

    inp = make_inputs(1, 64, 1, 128, seed=12, dtype=torch.bfloat16)
    run_device(inp)
    check_device_status()                                   # clean after an ordinary call
    st = _DeviceStatus.get(torch.device("cuda", torch.cuda.current_device()))
    st.dev.fill_(32)                                        # what a kernel's atomicOr would leave
    with pytest.raises(RuntimeError, match="bounded device-side wait gave up"):
        check_device_status()
    check_device_status()                                   # cleared by the report
    run_device(inp)


def test_selftest_wait_rejects_bad_arguments():
    from openkimi_b200 import _lib

    lib = _lib.load()
    t = torch.zeros(64, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert lib.kda_selftest_wait(t.data_ptr(), t.data_ptr(), 0, 5, st.data_ptr(), None) == 2
    assert lib.kda_selftest_wait(t.data_ptr(), t.data_ptr(), 64, 0, st.data_ptr(), None) == 2
    assert lib.kda_selftest_wait(None, t.data_ptr(), 64, 5, st.data_ptr(), None) == 1
