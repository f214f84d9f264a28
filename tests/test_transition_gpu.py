"""kutacc_af2_transition (CUDA, through the C ABI) against the CPU oracle."""
import numpy as np
import pytest
import torch

from kutacc_b200 import api
from kutacc_b200.workloads import as_f32, bf16_bits
from oracle import cpu_oracle as O
from tests import helpers

pytestmark = pytest.mark.gpu


def _case(batch, n_res, c_o, c_i, seed):
    rng = np.random.default_rng(seed)
    x = bf16_bits(rng.standard_normal((batch * n_res, c_o), dtype=np.float32))
    w1 = bf16_bits(rng.standard_normal((c_i, c_o), dtype=np.float32) / np.sqrt(c_o))
    w2 = bf16_bits(rng.standard_normal((c_o, c_i), dtype=np.float32) / np.sqrt(c_i))
    b1 = rng.standard_normal(c_i).astype(np.float32) * 0.5
    b2 = rng.standard_normal(c_o).astype(np.float32) * 0.5
    return x, w1, b1, w2, b2


def _bf(a):
    return torch.from_numpy(a.view(np.int16)).view(torch.bfloat16)


def _run(batch, n_res, c_o, c_i, arrays, device=True):
    x, w1, b1, w2, b2 = arrays
    f = (lambda t: t.cuda()) if device else (lambda t: t.pin_memory())
    tx, tw1, tw2 = f(_bf(x).view(batch, n_res, c_o)), f(_bf(w1)), f(_bf(w2))
    tb1, tb2 = f(torch.from_numpy(b1)), f(torch.from_numpy(b2))
    out = f(torch.zeros((batch, n_res, c_o), dtype=torch.bfloat16))
    api.transition(batch, n_res, c_o, c_i, api.tensor(tx), api.tensor(tw1), api.tensor(tb1), api.tensor(tw2),
                   api.tensor(tb2), api.tensor(out))
    torch.cuda.synchronize()
    return out.float().cpu().numpy().reshape(batch * n_res, c_o)


@pytest.mark.parametrize("batch,n_res,c_o,c_i", [(3, 130, 128, 512), (2, 64, 256, 1024), (1, 37, 64, 256), (2, 20, 48, 100)])
def test_matches_oracle(kutacc_lib, batch, n_res, c_o, c_i):
    arrays = _case(batch, n_res, c_o, c_i, 100 + c_o + n_res)
    got = _run(batch, n_res, c_o, c_i, arrays)
    want = as_f32(O.transition_bf16(*arrays))
    exact = O.transition_exact(as_f32(arrays[0]), as_f32(arrays[1]), arrays[2], as_f32(arrays[3]), arrays[4])
    assert np.isfinite(got).all()
    assert helpers.rel_err(got, want) <= helpers.BF16_TOL
    assert helpers.rel_err(got, exact) <= helpers.BF16_TOL


def test_host_pointers_match_device_pointers(kutacc_lib):
    arrays = _case(2, 96, 128, 512, 7)
    assert np.array_equal(_run(2, 96, 128, 512, arrays, True), _run(2, 96, 128, 512, arrays, False))


def test_bad_arguments_are_reported(kutacc_lib):
    import ctypes as C
    arrays = _case(1, 16, 128, 512, 8)
    x, w1, b1, w2, b2 = arrays
    t = api.tensor(_bf(x).view(1, 16, 128).cuda())
    wts = api.TransWeights(128, 512, None, None, None, None)
    ins = api.TransInputs(1, 16, t.handle, None)
    api.lib().kutacc_af2_transition(C.byref(ins), C.byref(wts), t.handle)
    assert api.error_set() and "nullptr" in api.last_error()
    api.clear_error()
    ins = api.TransInputs(0, 16, t.handle, None)
    api.lib().kutacc_af2_transition(C.byref(ins), C.byref(wts), t.handle)
    assert api.error_set() and "<= 0" in api.last_error()
    api.clear_error()
