"""Failure detection on the device without faulting it (-m gpu): a bounded wait that runs out is reported through the
status word, the kernel returns, and the next kernels run normally."""
import pytest
import torch

from oracle import tables as otab

pytestmark = pytest.mark.gpu


def test_expired_wait_sets_status_and_context_stays_usable():
    import neuralattentionsearchlinear_b200 as nat
    from neuralattentionsearchlinear_b200 import _lib
    lib = _lib.load()
    assert lib.natsl_device_status() == 0
    _lib.call("natsl_bounded_wait_selftest", 2000, torch.cuda.current_stream().cuda_stream)
    assert lib.natsl_device_status() == 1                      # the wait gave up and said so
    assert b"bounded wait" in lib.natsl_last_error()
    assert lib.natsl_device_status() == 0                      # reading clears the word
    # the context is intact: a regular kernel runs and is bit-exact against the oracle
    types = otab.synth_types(2, 8, 2, 0.4, seed=1)
    tb = nat.build_selection_tables(types.cuda(), 512, 64)
    assert torch.equal(tb.indices.cpu().long(), otab.build_tables(types, 512, 64)["indices"])
    assert lib.natsl_device_status() == 0


def test_status_check_switch_surfaces_an_expired_wait_on_the_op_path(monkeypatch):
    """With the debugging switch (NATSL_CHECK_STATUS=1) every entry point reads the status word after its kernels have
    run: a wait that ran out in an earlier kernel makes the next op raise instead of passing unnoticed."""
    import neuralattentionsearchlinear_b200 as nat
    from neuralattentionsearchlinear_b200 import _lib
    lib = _lib.load()
    assert lib.natsl_device_status() == 0
    monkeypatch.setattr(_lib, "CHECK_STATUS", True)
    types = otab.synth_types(1, 8, 2, 0.4, seed=2).cuda()
    nat.build_selection_tables(types, 512, 64)                 # a healthy op passes the check
    _lib.call("natsl_bounded_wait_selftest", 2000, torch.cuda.current_stream().cuda_stream)
    with pytest.raises(_lib.NatslError, match="device status 1"):
        nat.build_selection_tables(types, 512, 64)
    assert lib.natsl_device_status() == 0                      # read and cleared by the check
    nat.build_selection_tables(types, 512, 64)
