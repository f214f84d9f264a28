"""LayerNorm fused into the projections that follow it: kutacc_b200_gating_attention_ln and kutacc_b200_pair_bias_ln
against the unfused sequence of the CPU oracle (layernorm_bf16, then the operator), which is what a caller of the
reference computes (src/normalization/layernorm_kernel.h:22-53 followed by src/attention/gating_attention.cpp)."""
import numpy as np
import pytest
import torch

from kutacc_b200 import api, runner
from kutacc_b200 import workloads as W
from oracle import cpu_oracle as O
from tests import helpers

pytestmark = pytest.mark.gpu
EPS = 1e-5


def _ln_case(seed, B, S, H, D, mean_shift):
    """A gating case whose `x` is NOT normalised (per-row offset and scale), plus LayerNorm parameters."""
    w = W.random_gating_case(seed=seed, B=B, S=S, H=H, D=D, with_nb=True, full_mask_rows=1 if B > 1 else 0)
    rng = np.random.default_rng(seed + 1)
    C = H * D
    raw = w.arrays["x"] * rng.uniform(0.5, 3.0, size=(B, S, 1)).astype(np.float32) + mean_shift * rng.standard_normal((B, S, 1)).astype(np.float32)
    raw = W.as_f32(W.bf16_bits(raw))
    gamma = (1.0 + 0.3 * rng.standard_normal(C)).astype(np.float32)
    beta = (0.2 * rng.standard_normal(C)).astype(np.float32)
    return w, raw, gamma, beta


def _oracle(w, raw, gamma, beta):
    C = w.C
    normed = O.layernorm_bf16(W.bf16_bits(raw).reshape(-1, C), gamma, beta, EPS)
    w2 = W.Workload(name="ln", kind="gating", dtype="bf16", B=w.B, S=w.S, H=w.H, D=w.D, seed=0, has_nb=w.has_nb)
    w2.arrays = dict(w.arrays)
    w2.arrays["x"] = W.as_f32(normed).reshape(w.B, w.S, C)
    return helpers.oracle_faithful(w2)


# head size 32 (normalisation folded into the tcgen05 projection), other shapes (normalised copy in the workspace);
# the last case has row means many standard deviations away from zero
@pytest.mark.parametrize("B,S,H,D,shift", [(3, 96, 4, 32, 1.0), (2, 200, 8, 32, 2.0), (2, 70, 2, 16, 1.0), (2, 64, 4, 32, 40.0)])
def test_gating_attention_ln_matches_unfused_oracle(kutacc_lib, B, S, H, D, shift):
    w, raw, gamma, beta = _ln_case(900 + S, B, S, H, D, shift)
    case = runner.DeviceCase(w)
    x = runner._to_torch(raw, "bf16", "cuda:0")
    g, b = torch.from_numpy(gamma).cuda(), torch.from_numpy(beta).cuda()
    api.gating_attention_ln(api.tensor(x, sizes=[B * S, w.C], strides=[w.C, 1]), case.inputs, case.t_bias, case.t_nb, case.weights,
                            g.data_ptr(), b.data_ptr(), EPS, case.t_out)
    torch.cuda.synchronize()
    got = runner.out_to_f32(case.out)
    assert np.isfinite(got).all()
    assert helpers.rel_err(got, _oracle(w, raw, gamma, beta)) <= helpers.BF16_TOL


def test_gating_attention_ln_host_parameters_and_chunked_host_call(kutacc_lib):
    # gamma/beta in host memory, activations and result in pinned host memory (the chunked path normalises chunk by chunk)
    w, raw, gamma, beta = _ln_case(950, 35, 256, 4, 32, 1.5)
    host = runner.HostCase(w)
    x = runner._to_torch(raw, "bf16", "cpu", pin=True)
    api.gating_attention_ln(api.tensor(x, sizes=[w.B * w.S, w.C], strides=[w.C, 1]), host.inputs, host.t_bias, host.t_nb,
                            host.weights, gamma.ctypes.data, beta.ctypes.data, EPS, host.t_out)
    got = runner.out_to_f32(host.out)
    rows = [0, 17, 34]
    sub, sub_raw = W.Workload(name="s", kind="gating", dtype="bf16", B=len(rows), S=w.S, H=w.H, D=w.D, seed=0, has_nb=True), raw[rows]
    sub.arrays = dict(w.arrays)
    sub.arrays["bias"] = w.arrays["bias"][rows]
    assert helpers.rel_err(got[rows], _oracle(sub, sub_raw, gamma, beta)) <= helpers.BF16_TOL


@pytest.mark.parametrize("R,Nk,Cz,H,shift", [(40, 40, 128, 4, 1.0), (33, 50, 64, 8, 2.0), (20, 24, 32, 4, 1.0), (16, 64, 128, 4, 30.0)])
def test_pair_bias_ln_matches_unfused_oracle(kutacc_lib, R, Nk, Cz, H, shift):
    rng = np.random.default_rng(970 + Cz + R)
    z = W.as_f32(W.bf16_bits(rng.standard_normal((R, Nk, Cz), dtype=np.float32) * rng.uniform(0.5, 3.0, size=(R, Nk, 1)).astype(np.float32)
                             + shift * rng.standard_normal((R, Nk, 1)).astype(np.float32)))
    wb = W.as_f32(W.bf16_bits(rng.standard_normal((H, Cz), dtype=np.float32) / np.sqrt(Cz)))
    gamma = (1.0 + 0.3 * rng.standard_normal(Cz)).astype(np.float32)
    beta = (0.2 * rng.standard_normal(Cz)).astype(np.float32)
    zt, wt = runner._to_torch(z, "bf16", "cuda:0"), runner._to_torch(wb, "bf16", "cuda:0")
    nb = torch.zeros((H, R, Nk), dtype=torch.bfloat16, device="cuda:0")
    g, b = torch.from_numpy(gamma).cuda(), torch.from_numpy(beta).cuda()
    api.pair_bias_ln(api.tensor(zt), g.data_ptr(), b.data_ptr(), EPS, api.tensor(wt), api.tensor(nb))
    torch.cuda.synchronize()
    normed = W.as_f32(O.layernorm_bf16(W.bf16_bits(z).reshape(-1, Cz), gamma, beta, EPS))
    want = W.as_f32(O.linear_bf16(W.bf16_bits(normed), W.bf16_bits(wb), None)).T.reshape(H, R, Nk)
    got = nb.float().cpu().numpy()
    assert helpers.rel_err(got, want) <= helpers.BF16_TOL
