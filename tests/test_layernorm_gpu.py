"""kutacc_af2_layernorm / kutacc_b200_layernorm_rows (CUDA, through the C ABI) against the CPU oracle."""
import ctypes as C

import numpy as np
import pytest
import torch

from kutacc_b200 import api
from kutacc_b200.workloads import as_f32, bf16_bits
from oracle import cpu_oracle as O

pytestmark = pytest.mark.gpu


def _case(rows, size, seed, offset=0.0):
    rng = np.random.default_rng(seed)
    x = bf16_bits(rng.standard_normal((rows, size), dtype=np.float32) * 2 + offset)
    g = rng.standard_normal(size).astype(np.float32)
    b = rng.standard_normal(size).astype(np.float32)
    return x, g, b


def _dev(a, dtype=None):
    t = torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).cuda()
    return t


def _ulp_close(got_bits, want_bits):
    # the fp32 partial sums are added in another order than in the oracle: results may differ by one bf16 ulp
    got, want = as_f32(got_bits).astype(np.float64), as_f32(want_bits).astype(np.float64)
    ulp = np.maximum(np.abs(want), 2.0 ** -126) * 2.0 ** -7
    return bool((np.abs(got - want) <= 1.01 * ulp).all())


@pytest.mark.parametrize("rows,size,offset", [(1000, 128, 0.0), (37, 64, 20.0), (5, 256, -3.0), (3, 1024, 0.0),
                                              (7, 384, 1.0), (4, 100, 0.0), (2, 2048, 0.5)])
def test_rows_match_oracle(kutacc_lib, rows, size, offset):
    x, g, b = _case(rows, size, 7 * rows + size, offset)
    dx, dg, db = _dev(x), _dev(g), _dev(b)
    out = torch.zeros((rows, size), dtype=torch.int16, device="cuda")
    api.layernorm_rows(dx.data_ptr(), dg.data_ptr(), db.data_ptr(), rows, size, 1e-5, out.data_ptr())
    torch.cuda.synchronize()
    got = out.cpu().numpy().view(np.uint16)
    want = O.layernorm_bf16(x, g, b, 1e-5)
    assert _ulp_close(got, want)
    exact = O.layernorm_exact(as_f32(x), g, b, 1e-5)
    assert np.abs(as_f32(got) - exact).max() <= 1e-2 * np.abs(exact).max()


def test_one_row_entry_with_host_pointers(kutacc_lib):
    x, g, b = _case(1, 128, 3)
    out = np.zeros((1, 128), dtype=np.uint16)
    api.layernorm(x.ctypes.data, g.ctypes.data, b.ctypes.data, 128, 1e-5, out.ctypes.data)
    assert _ulp_close(out, O.layernorm_bf16(x, g, b, 1e-5))


def test_strided_rows_and_in_place(kutacc_lib):
    rows, size, pitch = 33, 128, 160
    x, g, b = _case(rows, size, 5)
    wide = np.full((rows, pitch), 0x4049, dtype=np.uint16)         # filler between the rows
    wide[:, :size] = x
    d = _dev(wide)
    dg, db = _dev(g), _dev(b)
    api.layernorm_rows(d.data_ptr(), dg.data_ptr(), db.data_ptr(), rows, size, 1e-5, d.data_ptr(), pitch, pitch)
    torch.cuda.synchronize()
    got = d.cpu().numpy().view(np.uint16)
    assert _ulp_close(got[:, :size], O.layernorm_bf16(x, g, b, 1e-5))
    assert (got[:, size:] == 0x4049).all()


def test_bad_arguments_are_reported(kutacc_lib):
    x, g, b = _case(2, 64, 9)
    out = np.zeros_like(x)
    api.layernorm_rows(0, g.ctypes.data, b.ctypes.data, 2, 64, 1e-5, out.ctypes.data, check=False)
    assert api.error_set() and "nullptr" in api.last_error()
    api.clear_error()
    api.layernorm_rows(x.ctypes.data, g.ctypes.data, b.ctypes.data, 2, 0, 1e-5, out.ctypes.data, check=False)
    assert api.error_set()
    api.clear_error()
