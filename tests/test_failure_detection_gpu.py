"""The bounded-wait convention of the pipelined kernels, exercised without any GPU fault.

Every mbarrier wait in the library's kernels gives up after a limit, writes its site into a host-visible word
and lets the kernel return; the next synchronising call reports it through the usual error convention. The
self-test entry makes a wait run out on purpose (a barrier nothing arrives on, a limit of a millisecond): the
kernel returns normally, the error is reported, and the context keeps working.
"""
import numpy as np
import pytest
import torch

from kutacc_b200 import api, runner
from kutacc_b200 import workloads as W
from tests import helpers

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_and_the_context_survives(kutacc_lib):
    w = W.random_gating_case(seed=5, B=2, S=128, H=4, D=32)
    case = runner.DeviceCase(w)
    want = runner.out_to_f32(case.run()).copy()
    assert api.lib().kutacc_b200_selftest_wait_timeout(1000) == 0          # 1 ms
    assert api.error_set()
    msg = api.last_error()
    assert "device-side wait ran out of time" in msg and str(0x5e1f) in msg
    api.clear_error()
    # the same context still computes, bit for bit
    got = runner.out_to_f32(case.run())
    torch.cuda.synchronize()
    assert not api.error_set()
    assert np.array_equal(got, want)
    assert helpers.rel_err(got, helpers.oracle_faithful(w)) <= helpers.BF16_TOL


def test_in_enqueue_only_mode_the_report_comes_at_synchronize(kutacc_lib):
    api.set_async(True)
    try:
        assert api.lib().kutacc_b200_selftest_wait_timeout(500) == 0
        assert not api.error_set()                 # nothing has been waited for yet
        api.synchronize()
        assert api.error_set() and "ran out of time" in api.last_error()
    finally:
        api.clear_error()
        api.set_async(False)
