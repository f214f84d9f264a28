"""kutacc_af2_linear, the fused pair-bias projection and the single-rank all-gather on the GPU."""
import numpy as np
import pytest
import torch

from kutacc_b200 import api
from kutacc_b200 import workloads as W
from oracle import cpu_oracle as O
from tests import helpers

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _bf16_cuda(a):
    return torch.from_numpy(W.bf16_bits(a).view(np.int16)).view(torch.bfloat16).to(DEV)


@pytest.mark.parametrize("M,N,K,bias,beta", [(300, 128, 128, True, 0), (513, 256, 192, False, 0), (1000, 4, 128, False, 0), (77, 8, 64, False, 0),
                                             (50, 24, 40, True, 0), (64, 64, 64, True, 1), (33, 5, 17, False, 2)])
def test_linear_bf16(kutacc_lib, M, N, K, bias, beta):
    rng = np.random.default_rng(M + N)
    a = W.as_f32(W.bf16_bits(rng.standard_normal((M, K)).astype(np.float32)))
    w = W.as_f32(W.bf16_bits(rng.standard_normal((N, K)).astype(np.float32) / np.sqrt(K)))
    b = rng.standard_normal(N).astype(np.float32) if bias else None
    prev = W.as_f32(W.bf16_bits(rng.standard_normal((M, N)).astype(np.float32)))
    ref = W.as_f32(O.linear_bf16(W.bf16_bits(a), W.bf16_bits(w), b, beta=beta, result=W.bf16_bits(prev)))
    ta, tw, tr = _bf16_cuda(a), _bf16_cuda(w), _bf16_cuda(prev)
    tb = torch.from_numpy(b).to(DEV) if bias else None
    api.linear(api.tensor(ta), api.tensor(tw), tb.data_ptr() if bias else None, api.tensor(tr), beta)
    got = tr.float().cpu().numpy()
    assert helpers.rel_err(got, ref) <= 5e-3


def test_linear_fp32(kutacc_lib):
    rng = np.random.default_rng(5)
    a = rng.standard_normal((200, 96)).astype(np.float32)
    w = (rng.standard_normal((10, 96)) / 10).astype(np.float32)
    b = rng.standard_normal(10).astype(np.float32)
    ta, tw, tb = torch.from_numpy(a).to(DEV), torch.from_numpy(w).to(DEV), torch.from_numpy(b).to(DEV)
    tr = torch.zeros((200, 10), dtype=torch.float32, device=DEV)
    api.linear(api.tensor(ta), api.tensor(tw), tb.data_ptr(), api.tensor(tr), 0)
    assert helpers.rel_err(tr.cpu().numpy(), O.linear_exact(a, w, b)) <= helpers.FP32_TOL


@pytest.mark.parametrize("M,N,K,bias", [(300, 128, 96, True), (1000, 384, 256, False), (77, 256, 32, True)])
def test_linear_fp32_on_the_tensor_memory_gemm(kutacc_lib, M, N, K, bias):
    # fp32 with n % 128 == 0 and k % 32 == 0: tcgen05 kind::tf32 on operands split into head and tail; large values
    # next to small ones in one row show a dropped tail at once
    rng = np.random.default_rng(M + N)
    a = (rng.standard_normal((M, K)) * rng.choice([1e-3, 1.0, 300.0], (M, K))).astype(np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32) if bias else None
    ta, tw = torch.from_numpy(a).to(DEV), torch.from_numpy(w).to(DEV)
    tb = torch.from_numpy(b).to(DEV) if bias else None
    tr = torch.full((M, N), 7.0, dtype=torch.float32, device=DEV)
    api.set_profile(True)
    api.profile_read()
    api.linear(api.tensor(ta), api.tensor(tw), tb.data_ptr() if bias else None, api.tensor(tr), 0)
    names = [k for k, _ in api.profile_read()]
    api.set_profile(False)
    assert "gemm_tf32x3_tc" in names
    ref = O.linear_exact(a, w, b)
    got = tr.cpu().numpy()
    # against the magnitude of the terms of each dot product, not of the (possibly cancelling) result
    scale = (np.abs(a).astype(np.float64) @ np.abs(w).astype(np.float64).T).max()
    assert np.abs(got.astype(np.float64) - ref).max() <= 5e-6 * scale          # a dropped tail term would cost 2^-11


@pytest.mark.parametrize("R,Nk,Cz,H", [(8, 384, 128, 4), (5, 100, 128, 8), (3, 33, 64, 4), (2, 50, 40, 3)])
def test_pair_bias_matches_linear_then_permute(kutacc_lib, R, Nk, Cz, H):
    rng = np.random.default_rng(R * Nk)
    z = W.as_f32(W.bf16_bits(rng.standard_normal((R, Nk, Cz)).astype(np.float32)))
    wb = W.as_f32(W.bf16_bits(rng.standard_normal((H, Cz)).astype(np.float32) / np.sqrt(Cz)))
    lin = W.as_f32(O.linear_bf16(W.bf16_bits(z.reshape(-1, Cz)), W.bf16_bits(wb), None))      # [R*Nk, H]
    ref = lin.reshape(R, Nk, H).transpose(2, 0, 1)
    tz, tw = _bf16_cuda(z), _bf16_cuda(wb)
    nb = torch.zeros((H, R, Nk), dtype=torch.bfloat16, device=DEV)
    api.pair_bias(api.tensor(tz), api.tensor(tw), api.tensor(nb))
    got = nb.float().cpu().numpy()
    # same products, different summation order: at most one bf16 ulp apart
    assert helpers.rel_err(got, ref) <= 2.0 ** -7


def test_device_prepack_copies_rows(kutacc_lib):
    w = torch.arange(40 * 24, dtype=torch.int16, device=DEV).reshape(40, 24)
    packed = torch.zeros((40, 16), dtype=torch.int16, device=DEV)
    kutacc_lib.kutacc_af2_linear_weight_prepack(w.data_ptr(), packed.data_ptr(), 40, 16, 24, 0)
    api.raise_if_error()
    assert torch.equal(packed, w[:, :16])


def test_all_gather_single_rank_copies_with_byte_strides(kutacc_lib):
    # world_size == 1: the gather degenerates to a strided byte copy (all_gather.cpp:45-61)
    src = torch.arange(4 * 5 * 8, dtype=torch.uint8, device=DEV).reshape(4, 5, 8)
    dst = torch.zeros((4, 5, 16), dtype=torch.uint8, device=DEV)
    api.all_gather(api.tensor(src, sizes=[4, 5, 8], strides=[40, 8, 1]),
                   api.tensor(dst, sizes=[4, 5, 8], strides=[80, 16, 1]))
    assert torch.equal(dst[:, :, :8], src) and int(dst[:, :, 8:].sum()) == 0
    # host buffers, the reference's own grid for one rank
    grid = np.arange(20, dtype=np.uint8).reshape(4, 5, 1)
    out = np.zeros((4, 5, 1), dtype=np.uint8)
    api.all_gather(api.tensor(grid), api.tensor(out))
    assert np.array_equal(out, grid)


@pytest.mark.parametrize("R,Nk,Cz,H", [(8, 384, 128, 4), (5, 100, 64, 8)])
def test_pair_bias_written_with_the_heads_inside_the_rows(kutacc_lib, R, Nk, Cz, H):
    # nb [H, R, Nk] as a strided view of a [R, H, Nk] storage: the same values as the dense output, nothing else touched
    rng = np.random.default_rng(R + Nk)
    z = W.as_f32(W.bf16_bits(rng.standard_normal((R, Nk, Cz)).astype(np.float32)))
    wb = W.as_f32(W.bf16_bits((rng.standard_normal((H, Cz)) / np.sqrt(Cz)).astype(np.float32)))
    tz = torch.from_numpy(W.bf16_bits(z).view(np.int16)).view(torch.bfloat16).to(DEV)
    tw = torch.from_numpy(W.bf16_bits(wb).view(np.int16)).view(torch.bfloat16).to(DEV)
    dense = torch.zeros((H, R, Nk), dtype=torch.bfloat16, device=DEV)
    api.pair_bias(api.tensor(tz), api.tensor(tw), api.tensor(dense))
    store = torch.full((R, H + 1, Nk), 7.0, dtype=torch.bfloat16, device=DEV)       # one spare "head" of padding per row
    view = api.Tensor(store.data_ptr(), [H, R, Nk], [Nk, (H + 1) * Nk, 1], api.DTYPE_BF16, keep=store)
    api.pair_bias(api.tensor(tz), api.tensor(tw), view)
    torch.cuda.synchronize()
    assert torch.equal(store[:, :H, :].permute(1, 0, 2), dense)
    assert (store[:, H, :] == 7.0).all()
