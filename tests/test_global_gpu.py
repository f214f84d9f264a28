"""Parity of kutacc_af2_global_attention (CUDA, through the C ABI) with the CPU oracle."""
import numpy as np
import pytest
import torch

from kutacc_b200 import api, runner
from kutacc_b200 import workloads as W
from tests import helpers

pytestmark = pytest.mark.gpu


def _run(w, device=True):
    case = runner.DeviceCase(w) if device else runner.HostCase(w)
    out = case.run()
    torch.cuda.synchronize()
    return runner.out_to_f32(out)


@pytest.mark.parametrize("B,S,H,D", [(2, 48, 8, 8), (3, 130, 8, 8), (1, 1000, 8, 8), (2, 1500, 8, 8), (1, 5300, 8, 8),
                                     (1, 14100, 8, 8), (2, 257, 4, 16), (2, 64, 2, 32),
                                     (1, 96, 16, 4), (1, 70, 1, 64)])
def test_matches_faithful_oracle(kutacc_lib, B, S, H, D):
    w = W.random_global_case(seed=400 + S, B=B, S=S, H=H, D=D, zero_mask_rows=1 if B > 1 else 0)
    got = _run(w)
    assert np.isfinite(got).all()
    assert helpers.rel_err(got, helpers.oracle_faithful(w)) <= helpers.BF16_TOL
    assert helpers.rel_err(got, helpers.oracle_exact(w)) <= helpers.BF16_TOL


def test_all_rows_masked_still_gives_gate_times_uniform_average(kutacc_lib):
    # sum(mask) == 0: q_avg is 0 by the 1e-10 guard, softmax uniform over ALL rows; masked query
    # rows still receive an output (global_attention.cpp:64, :134-156)
    w = W.random_global_case(seed=21, B=1, S=80, zero_mask_rows=1)
    got = _run(w)
    assert helpers.rel_err(got, helpers.oracle_faithful(w)) <= helpers.BF16_TOL


def test_extra_msa_shape_subsampled_columns(kutacc_lib):
    w = W.make("extra_msa_global", rows=6)       # full 5120 rows, 6 of the 384 columns
    got = _run(w)
    assert helpers.rel_err(got, helpers.oracle_faithful(w)) <= helpers.BF16_TOL


def test_extra_msa_shape_full_size_columns_spread_over_the_batch(kutacc_lib):
    """The extra-MSA shape at FULL size on the GPU; the oracle checks columns at the start, in the middle and at
    the end of the 384."""
    w = W.make("extra_msa_global")
    full = _run(w)
    assert np.isfinite(full).all()
    cols = [0, 1, 191, 192, 382, 383]
    pick = W.Workload(name="pick", kind="global", dtype="bf16", B=len(cols), S=w.S, H=w.H, D=w.D, seed=0)
    pick.arrays = dict(w.arrays)
    pick.arrays["x"] = w.arrays["x"][cols]
    pick.arrays["mask"] = w.arrays["mask"][cols]
    assert helpers.rel_err(full[cols], helpers.oracle_faithful(pick)) <= helpers.BF16_TOL


def test_host_pointers_match_device_pointers(kutacc_lib):
    w = W.random_global_case(seed=22, B=2, S=200)
    assert np.array_equal(_run(w, True), _run(w, False))


def test_columns_are_independent_at_full_size(kutacc_lib):
    w = W.make("extra_msa_global", rows=40)
    full = _run(w)
    sub = W.make("extra_msa_global", rows=3)
    assert np.array_equal(_run(sub), full[:3])


def test_many_short_columns_wrap_the_shared_memory_ring(kutacc_lib):
    # more columns than resident clusters: every CTA walks several columns and reuses its slots
    w = W.random_global_case(seed=23, B=700, S=300, zero_mask_rows=3)
    got = _run(w)
    assert np.isfinite(got).all()
    assert helpers.rel_err(got, helpers.oracle_faithful(w)) <= helpers.BF16_TOL


def test_strided_output_rows(kutacc_lib):
    w = W.random_global_case(seed=24, B=3, S=333)
    want = _run(w)
    case = runner.DeviceCase(w)
    wide = torch.full((w.B, w.S, 96), 7.0, dtype=torch.bfloat16, device="cuda:0")
    out_t = api.Tensor(wide.data_ptr(), [w.B, w.S, w.C], [w.S * 96, 96, 1], api.DTYPE_BF16, keep=wide)
    api.global_attention(case.inputs, case.t_x, case.t_mask, case.weights, out_t)
    torch.cuda.synchronize()
    api.raise_if_error()
    got = wide.float().cpu().numpy()
    assert np.array_equal(got[:, :, :w.C], want)
    assert (got[:, :, w.C:] == 7.0).all()                   # the gap between rows is left alone


def test_pipelined_host_call_matches_device_call(kutacc_lib):
    # 16 columns x 2048 rows = 4 MiB of activations in pinned host memory: the library uploads, computes and
    # downloads the columns in chunks on three streams; the result must not change by a bit
    w = W.random_global_case(seed=25, B=16, S=2048, zero_mask_rows=2)
    assert np.array_equal(_run(w, True), _run(w, False))
