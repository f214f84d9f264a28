"""The allocation-free global-attention entry point against the regular operator.

Collected last on purpose (file name): if it fails, a run that stops at the first failure has already
executed every other test. It must also pass alone in a fresh process, where its first call is the one
that resolves the static scratch's device address.

The entry point serves hosts that may not allocate device memory inside an operator call - for
instance a server whose own pool owns all of HBM, or a loop that cannot take the synchronisation that
cudaMalloc and cudaFree imply. Here torch owns the tensors; the library call itself must not grow the
library's workspace.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from kutacc_b200 import api, runner
from kutacc_b200 import workloads as W
from tests import helpers

pytestmark = pytest.mark.gpu


def _noalloc(case, out, stream=0):
    w = case.w
    rc = api.lib().kutacc_b200_global_attention_noalloc(
        case.x.data_ptr(), case.mask.data_ptr(), case.wq.data_ptr(), case.wk.data_ptr(), case.wv.data_ptr(),
        case.wg.data_ptr(), case.bg.data_ptr(), case.wo.data_ptr(), case.bo.data_ptr(), out.data_ptr(), w.C,
        w.B, w.S, w.H, w.D, C.c_void_p(stream))
    return rc


def test_noalloc_entry_matches_regular_operator_twice_in_a_row(kutacc_lib):
    w1 = W.random_global_case(seed=31, B=5, S=700, H=8, D=8, zero_mask_rows=1)
    w2 = W.random_global_case(seed=32, B=3, S=333, H=4, D=16)
    for w in (w1, w2):                      # two calls in a row share the static scratch
        case = runner.DeviceCase(w)
        want = runner.out_to_f32(case.run()).copy()          # kutacc_af2_global_attention
        held = api.lib().kutacc_b200_workspace_bytes()
        out = torch.full((w.B, w.S, w.C), float("nan"), dtype=torch.bfloat16, device="cuda:0")
        assert _noalloc(case, out) == 0
        torch.cuda.synchronize()
        api.raise_if_error()
        got = out.float().cpu().numpy()
        # the parity tolerance of the other tests (1e-2 relative) is the formal bound; where the regular
        # operator runs the same three kernels with the same split plan (every shape but 8 heads x 8, which
        # it computes in one cluster kernel) the results agree to the last bit
        assert np.isfinite(got).all()
        assert np.abs(got - want).max() <= 1e-2 * np.abs(want).max()
        if (w.H, w.D) != (8, 8):
            assert np.array_equal(got, want)
        assert api.lib().kutacc_b200_workspace_bytes() == held      # the library's pool did not grow


def test_noalloc_entry_matches_the_oracle_on_split_columns_and_on_a_stream(kutacc_lib):
    """The entry point's own kernels against the CPU oracle (the regular operator runs a different kernel for
    8 heads x 8): a column long enough to be cut into several row splits, a length that is not a multiple of
    16, one column with every row masked, and the call made on a stream of the caller's."""
    w = W.random_global_case(seed=34, B=3, S=1000 + 13, H=8, D=8, zero_mask_rows=1)
    case = runner.DeviceCase(w)
    ref = helpers.oracle_faithful(w)
    stream = torch.cuda.Stream()
    for _ in range(2):
        out = torch.full((w.B, w.S, w.C), float("nan"), dtype=torch.bfloat16, device="cuda:0")
        stream.wait_stream(torch.cuda.current_stream())
        assert _noalloc(case, out, stream.cuda_stream) == 0
        stream.synchronize()
        api.raise_if_error()
        got = out.float().cpu().numpy()
        assert np.isfinite(got).all()
        assert helpers.rel_err(got, ref) <= helpers.BF16_TOL


def test_noalloc_entry_refuses_unaligned_weights(kutacc_lib):
    # the kernels read the weights with vector loads: a view that starts on an odd element is refused, not launched
    w = W.random_global_case(seed=35, B=2, S=64)
    case = runner.DeviceCase(w)
    out = torch.zeros((w.B, w.S, w.C), dtype=torch.bfloat16, device="cuda:0")
    shifted = torch.zeros(w.D * w.C + 8, dtype=torch.bfloat16, device="cuda:0")
    before = api.launch_count()
    rc = api.lib().kutacc_b200_global_attention_noalloc(
        case.x.data_ptr(), case.mask.data_ptr(), case.wq.data_ptr(), shifted.data_ptr() + 2, case.wv.data_ptr(),
        case.wg.data_ptr(), case.bg.data_ptr(), case.wo.data_ptr(), case.bo.data_ptr(), out.data_ptr(), w.C,
        w.B, w.S, w.H, w.D, C.c_void_p(0))
    assert rc == -1 and "16-byte aligned" in api.last_error()
    assert api.launch_count() == before
    api.clear_error()


def test_noalloc_entry_refuses_shapes_beyond_the_static_scratch(kutacc_lib):
    w = W.random_global_case(seed=33, B=2, S=64)
    case = runner.DeviceCase(w)
    out = torch.zeros((w.B, w.S, w.C), dtype=torch.bfloat16, device="cuda:0")
    rc = api.lib().kutacc_b200_global_attention_noalloc(
        case.x.data_ptr(), case.mask.data_ptr(), case.wq.data_ptr(), case.wk.data_ptr(), case.wv.data_ptr(),
        case.wg.data_ptr(), case.bg.data_ptr(), case.wo.data_ptr(), case.bo.data_ptr(), out.data_ptr(), w.C,
        60000, 4096, w.H, w.D, C.c_void_p(0))              # far more scratch than 4 MiB; nothing is launched
    assert rc == -1 and api.error_set()
    assert "static scratch holds" in api.last_error()
    api.clear_error()
    assert _noalloc(case, out) == 0                          # the entry point still works afterwards
    torch.cuda.synchronize()
