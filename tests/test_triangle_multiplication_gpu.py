"""Parity of the four triangle-multiplication steps (CUDA, through the C ABI) with the CPU oracle.

The reference's own tests for this operator only pass null handles (test/functest/cal/triangle_multiplication_test.cpp),
so the oracle restates src/attention/triangle_multiplication.cpp:25-158 line by line and the vectors under
tests/golden/ are the oracle's own.
"""
import numpy as np
import pytest
import torch

from kutacc_b200 import api
from kutacc_b200 import workloads as W
from oracle import cpu_oracle as O
from tests import helpers

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _bf(a, device=DEV):
    t = torch.from_numpy(W.bf16_bits(np.ascontiguousarray(a, dtype=np.float32)).view(np.int16)).view(torch.bfloat16)
    return t.to(device) if device != "cpu" else t


def _f32(t):
    return t.detach().to("cpu", torch.float32).numpy()


def _case(seed, n, c_o, c_i):
    rng = np.random.default_rng(seed)
    r = lambda a: W.as_f32(W.bf16_bits(a))
    A = {
        "x": r(rng.standard_normal((n, n, c_o), dtype=np.float32)),
        "mask": (rng.random((n, n)) >= 0.15).astype(np.float32),
        "pw": r(rng.standard_normal((c_i, c_o), dtype=np.float32) / np.sqrt(c_o)),
        "gw": r(rng.standard_normal((c_i, c_o), dtype=np.float32) / np.sqrt(c_o)),
        "pb": rng.standard_normal(c_i).astype(np.float32),
        "gb": rng.standard_normal(c_i).astype(np.float32),
        "gating_w": r(rng.standard_normal((c_o, c_o), dtype=np.float32) / np.sqrt(c_o)),
        "gating_b": rng.standard_normal(c_o).astype(np.float32),
        "out_w": r(rng.standard_normal((c_o, c_i), dtype=np.float32) / np.sqrt(c_i)),
        "out_b": rng.standard_normal(c_o).astype(np.float32),
    }
    return A


def _calc_proj(A, n, c_o, c_i, device=DEV):
    x, mask = _bf(A["x"], device), _bf(A["mask"], device)
    pw, gw = _bf(A["pw"], device), _bf(A["gw"], device)
    pb, gb = torch.from_numpy(A["pb"]).to(device), torch.from_numpy(A["gb"]).to(device)
    proj = torch.zeros((c_i, n, n), dtype=torch.bfloat16, device=device)
    gate = torch.zeros((c_i, n, n), dtype=torch.bfloat16, device=device)
    acts = api.make_tm_acts(n, n, proj, x, gate)
    weights = api.make_tm_proj_weights(c_o, c_i, pw, pb, gw, gb)
    api.tm_calc_proj(acts, api.tensor(mask), weights)
    if device != "cpu":
        torch.cuda.synchronize()
    return proj, gate


# (n, c_o, c_i): tensor-core shapes (c_o % 64 == 0, c_i % 128 == 0, n % 8 == 0), ragged n, and shapes only the
# CUDA-core kernels cover
SHAPES = [(64, 128, 128), (136, 64, 128), (40, 128, 256), (37, 48, 24), (50, 128, 128)]


@pytest.mark.parametrize("n,c_o,c_i", SHAPES)
def test_calc_proj_matches_oracle(kutacc_lib, n, c_o, c_i):
    A = _case(500 + n, n, c_o, c_i)
    proj, gate = _calc_proj(A, n, c_o, c_i)
    want_p, want_g = O.tm_calc_proj_bf16(W.bf16_bits(A["x"]), W.bf16_bits(A["mask"]), W.bf16_bits(A["pw"]), A["pb"],
                                         W.bf16_bits(A["gw"]), A["gb"])
    assert helpers.rel_err(_f32(gate), W.as_f32(want_g)) <= 2.0 ** -7        # one bf16 step where a sum lands on a tie
    assert helpers.rel_err(_f32(proj), W.as_f32(want_p)) <= helpers.BF16_TOL
    exact = O.tm_calc_proj_exact(A["x"], A["mask"], A["pw"], A["pb"], A["gw"], A["gb"])
    assert helpers.rel_err(_f32(proj), exact) <= helpers.BF16_TOL
    assert (_f32(proj)[:, A["mask"] == 0] == 0).all()                         # masked positions are exactly zero


@pytest.mark.parametrize("n,c_i", [(64, 8), (136, 4), (200, 3), (37, 5), (384, 2)])
@pytest.mark.parametrize("incoming", [False, True])
def test_equation_matches_oracle(kutacc_lib, n, c_i, incoming):
    rng = np.random.default_rng(600 + n)
    r = lambda a: W.as_f32(W.bf16_bits(a))
    L = r(rng.standard_normal((c_i, n, n), dtype=np.float32))
    R = r(rng.standard_normal((c_i, n, n), dtype=np.float32))
    left, right = _bf(L), _bf(R)
    center = torch.full((c_i, n, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    api.tm_equation(api.tensor(center), api.tensor(left), api.tensor(right), n, incoming)
    torch.cuda.synchronize()
    got = _f32(center)
    assert np.isfinite(got).all()
    want = W.as_f32(O.tm_equation_bf16(W.bf16_bits(L), W.bf16_bits(R), incoming))
    assert helpers.rel_err(got, want) <= 2.0 ** -7
    assert helpers.rel_err(got, O.tm_equation_exact(L, R, incoming)) <= helpers.BF16_TOL


@pytest.mark.parametrize("n,c_o,c_i", [(64, 128, 128), (50, 128, 128), (37, 48, 24)])
def test_gate_and_out_linear_then_last_match_oracle(kutacc_lib, n, c_o, c_i):
    A = _case(700 + n, n, c_o, c_i)
    rng = np.random.default_rng(701 + n)
    center = W.as_f32(W.bf16_bits(rng.standard_normal((n, n, c_i), dtype=np.float32)))
    x, cen = _bf(A["x"]), _bf(center)
    gate = torch.zeros((n, n, c_o), dtype=torch.bfloat16, device=DEV)
    out = torch.zeros((n, n, c_o), dtype=torch.bfloat16, device=DEV)
    acts = api.make_tm_acts(n, n, None, x, None)
    weights = api.make_tm_linear_weights(c_o, c_i, _bf(A["gating_w"]), torch.from_numpy(A["gating_b"]).to(DEV),
                                         _bf(A["out_w"]), torch.from_numpy(A["out_b"]).to(DEV))
    api.tm_gate_and_out_linear(api.tensor(gate), api.tensor(out), acts, api.tensor(cen), weights)
    torch.cuda.synchronize()
    want_gate = O.linear_bf16(W.bf16_bits(A["x"]).reshape(-1, c_o), W.bf16_bits(A["gating_w"]), A["gating_b"])
    want_out = O.linear_bf16(W.bf16_bits(center).reshape(-1, c_i), W.bf16_bits(A["out_w"]), A["out_b"])
    assert helpers.rel_err(_f32(gate).reshape(-1, c_o), W.as_f32(want_gate)) <= 2.0 ** -7
    assert helpers.rel_err(_f32(out).reshape(-1, c_o), W.as_f32(want_out)) <= 2.0 ** -7
    # last: out = out * sigmoid(gate), on the bits the GPU has just produced
    g_bits = gate.cpu().view(torch.int16).numpy().view(np.uint16)
    o_bits = out.cpu().view(torch.int16).numpy().view(np.uint16)
    api.tm_last(api.tensor(out), api.tensor(gate), n, n, c_o)
    torch.cuda.synchronize()
    want = W.as_f32(O.tm_last_bf16(o_bits, g_bits))
    assert helpers.rel_err(_f32(out), want) <= 2.0 ** -7


def test_whole_outgoing_update_against_exact_formula(kutacc_lib):
    """The four steps chained as a caller chains them (left and right projections, per-channel product, permute,
    output projection and gate) against the textbook formula in float64."""
    n, c = 64, 128
    L, R = _case(801, n, c, c), _case(802, n, c, c)
    lp, _ = _calc_proj(L, n, c, c)
    rp, _ = _calc_proj(R, n, c, c)
    center = torch.zeros((c, n, n), dtype=torch.bfloat16, device=DEV)
    api.tm_equation(api.tensor(center), api.tensor(lp), api.tensor(rp), n, False)
    cen = center.permute(1, 2, 0).contiguous()                       # the caller's LayerNorm is left out here
    gate = torch.zeros((n, n, c), dtype=torch.bfloat16, device=DEV)
    out = torch.zeros((n, n, c), dtype=torch.bfloat16, device=DEV)
    acts = api.make_tm_acts(n, n, None, _bf(L["x"]), None)
    weights = api.make_tm_linear_weights(c, c, _bf(L["gating_w"]), torch.from_numpy(L["gating_b"]).to(DEV), _bf(L["out_w"]),
                                         torch.from_numpy(L["out_b"]).to(DEV))
    api.tm_gate_and_out_linear(api.tensor(gate), api.tensor(out), acts, api.tensor(cen), weights)
    api.tm_last(api.tensor(out), api.tensor(gate), n, n, c)
    torch.cuda.synchronize()
    f = lambda a: np.asarray(a, dtype=np.float64)
    sig = lambda a: 1.0 / (1.0 + np.exp(-a))

    def proj(A):
        x = f(A["x"]).reshape(-1, c)
        return ((x @ f(A["pw"]).T + f(A["pb"])) * f(A["mask"]).reshape(-1, 1) * sig(x @ f(A["gw"]).T + f(A["gb"]))).reshape(n, n, c)

    lpe, rpe = proj(L), proj(R)
    ce = np.einsum("ikc,jkc->ijc", lpe, rpe)
    want = (ce.reshape(-1, c) @ f(L["out_w"]).T + f(L["out_b"])) * sig(f(L["x"]).reshape(-1, c) @ f(L["gating_w"]).T + f(L["gating_b"]))
    assert helpers.rel_err(_f32(out).reshape(-1, c), want) <= 2 * helpers.BF16_TOL


def test_host_tensors_and_strided_outputs(kutacc_lib):
    """Host-resident tensors give the same bits as device tensors, and a channel-major output whose rows are padded
    keeps its padding."""
    n, c_o, c_i = 40, 128, 128
    A = _case(900, n, c_o, c_i)
    dev_p, dev_g = _calc_proj(A, n, c_o, c_i)
    host_p, host_g = _calc_proj(A, n, c_o, c_i, device="cpu")
    assert torch.equal(dev_p.cpu(), host_p) and torch.equal(dev_g.cpu(), host_g)
    pad = 48
    x, mask = _bf(A["x"]), _bf(A["mask"])
    proj = torch.full((c_i, n, pad), 7.0, dtype=torch.bfloat16, device=DEV)
    gate = torch.full((c_i, n, pad), 7.0, dtype=torch.bfloat16, device=DEV)
    st = [n * pad, pad, 1]
    acts = api.make_tm_acts(n, n, api.tensor(proj, sizes=[c_i, n, n], strides=st), x, api.tensor(gate, sizes=[c_i, n, n], strides=st))
    weights = api.make_tm_proj_weights(c_o, c_i, _bf(A["pw"]), torch.from_numpy(A["pb"]).to(DEV), _bf(A["gw"]),
                                       torch.from_numpy(A["gb"]).to(DEV))
    api.tm_calc_proj(acts, api.tensor(mask), weights)
    torch.cuda.synchronize()
    assert torch.equal(proj[:, :, :n], dev_p) and torch.equal(gate[:, :, :n], dev_g)
    assert (proj[:, :, n:] == 7.0).all() and (gate[:, :, n:] == 7.0).all()


def test_null_arguments_are_reported(kutacc_lib):
    # the reference's own tests for this operator (triangle_multiplication_test.cpp): one null argument each
    L = api.lib()
    L.kutacc_af2_triangle_multiplication_calc_proj(None, None, None, True)
    assert api.error_set() and "input args nullptr error" in api.last_error()
    api.clear_error()
    L.kutacc_af2_triangle_multiplication_equation(None, None, None, 4, False)
    assert api.error_set() and "input args nullptr error" in api.last_error()
    api.clear_error()
    L.kutacc_af2_triangle_multiplication_last(None, None, 2, 2, 2)
    assert api.error_set() and "input args nullptr error" in api.last_error()
    api.clear_error()
