"""The CPU oracle against golden vectors, textbook float64 formulas and known properties."""
import os

import numpy as np
import pytest

from kutacc_b200 import workloads as W
from oracle import cpu_oracle as O
from tests import helpers

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_bf16_conversion_matches_torch():
    import torch
    rng = np.random.default_rng(0)
    a = np.concatenate([rng.standard_normal(4096).astype(np.float32) * 10.0 ** rng.integers(-6, 6, 4096),
                        np.array([0.0, -0.0, 1.0, 1.00390625, 1.01171875, 3.3895314e38, np.inf, -np.inf], np.float32)])
    ours = O.f32_to_bf16(a)
    ref = torch.from_numpy(a).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(ours, ref)
    assert np.array_equal(W.bf16_bits(a), ref)                    # the numpy twin used by the workloads
    assert np.array_equal(O.bf16_to_f32(ours), W.as_f32(ours))


def test_fexpa_exp_properties():
    # exact at multiples of ln2/64 that land on table entry 0: powers of two
    assert O.fexpa_exp(0.0) == 1.0
    assert O.fexpa_exp(-1e9) == 0.0            # very negative saturates to +0 (softmax of masked keys)
    assert O.fexpa_exp(-1e4) == 0.0
    xs = np.linspace(-20.0, 5.0, 2001)
    ys = np.array([O.fexpa_exp(float(x)) for x in xs])
    rel = np.abs(ys - np.exp(xs)) / np.exp(xs)
    assert rel.max() <= 2 ** (1 / 128) - 1 + 1e-4      # quantised to 1/64 octave
    assert np.all(np.diff(ys) >= 0)                    # monotone
    # the table: result is 2^(n/64) for integer n
    n = np.round(np.log2(ys[ys > 0]) * 64)
    assert np.allclose(np.log2(ys[ys > 0]) * 64, n, atol=1e-3)


def _textbook_gating(w):
    A = w.arrays
    B, S, H, D, C = w.B, w.S, w.H, w.D, w.C
    x = A["x"].astype(np.float64)
    q = (x @ A["wq"].T.astype(np.float64)).reshape(B, S, H, D)
    k = (x @ A["wk"].T.astype(np.float64)).reshape(B, S, H, D)
    v = (x @ A["wv"].T.astype(np.float64)).reshape(B, S, H, D)
    g = (x @ A["wg"].T.astype(np.float64) + A["bg"]).reshape(B, S, H, D)
    lg = np.einsum("bqhd,bkhd->bhqk", q, k) / np.sqrt(D)
    lg = (lg.astype(np.float32) + A["bias"][:, None, None, :]).astype(np.float32)
    if w.has_nb:
        lg = lg + A["nb"][None]
    lg = lg.astype(np.float64)
    p = np.exp(lg - lg.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    o = np.einsum("bhqk,bkhd->bqhd", p, v) / (1 + np.exp(-g))
    return o.reshape(B, S, C) @ A["wo"].T.astype(np.float64) + A["bo"]


@pytest.mark.parametrize("with_nb", [True, False])
def test_gating_exact_matches_textbook(with_nb):
    w = W.random_gating_case(seed=3, B=3, S=70, H=2, D=32, with_nb=with_nb, full_mask_rows=1)
    ex = helpers.oracle_exact(w)
    ref = _textbook_gating(w)
    assert helpers.rel_err(ex, ref) < 1e-6


def test_gating_faithful_close_to_exact_and_masked_row_uniform():
    w = W.random_gating_case(seed=4, B=2, S=64, H=2, D=32, with_nb=True, full_mask_rows=1)
    fa = helpers.oracle_faithful(w, block_size=16)
    ex = helpers.oracle_exact(w)
    # FEXPA (0.54 % per exp) and the bf16 round trips bound the distance between the two modes
    assert helpers.rel_err(fa, ex) < 1e-2
    # block_size only tiles the query loop: results do not depend on it
    fb = helpers.oracle_faithful(w, block_size=64)
    assert np.array_equal(fa, fb)


def test_fully_masked_row_is_uniform_average():
    # all keys of batch row 0 carry -1e9: fp32 absorbs the logits, softmax is uniform (1/S each)
    w = W.random_gating_case(seed=5, B=1, S=32, H=1, D=16, with_nb=False, full_mask_rows=1)
    A = w.arrays
    A["bg"][:] = 50.0            # sigmoid -> 1
    A["wo"] = np.eye(w.C, dtype=np.float32)
    A["bo"][:] = 0.0
    ex = helpers.oracle_exact(w)
    v = A["x"].reshape(w.S, w.C).astype(np.float64) @ A["wv"].T.astype(np.float64)
    assert np.allclose(ex[0], np.broadcast_to(v.mean(0), (w.S, w.C)), atol=1e-5)


def _textbook_global(w):
    A = w.arrays
    B, S, H, D, C = w.B, w.S, w.H, w.D, w.C
    x = A["x"].astype(np.float64)
    m = A["mask"].astype(np.float64)
    qa = (m[..., None] * x).sum(1) / (m.sum(1, keepdims=True) + 1e-10)
    q = (qa @ A["wq"].T.astype(np.float64)).reshape(B, H, D)
    k = x @ A["wk"].T.astype(np.float64)
    v = x @ A["wv"].T.astype(np.float64)
    lg = np.einsum("bhd,bsd->bhs", q, k) / np.sqrt(D)
    lg = lg.astype(np.float32) + (A["mask"] * np.float32(1e9) - np.float32(1e9))[:, None, :]
    lg = lg.astype(np.float64)
    p = np.exp(lg - lg.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    wa = np.einsum("bhs,bsd->bhd", p, v).reshape(B, 1, C)
    g = 1 / (1 + np.exp(-(x @ A["wg"].T.astype(np.float64) + A["bg"])))
    return (g * wa) @ A["wo"].T.astype(np.float64) + A["bo"]


def test_global_exact_matches_textbook_and_faithful_is_close():
    w = W.random_global_case(seed=6, B=3, S=96, zero_mask_rows=1)
    ex = helpers.oracle_exact(w)
    assert helpers.rel_err(ex, _textbook_global(w)) < 1e-6
    assert helpers.rel_err(helpers.oracle_faithful(w), ex) < 1e-2


def test_linear_modes_agree():
    rng = np.random.default_rng(7)
    a = W.as_f32(W.bf16_bits(rng.standard_normal((37, 48)).astype(np.float32)))
    w = W.as_f32(W.bf16_bits(rng.standard_normal((5, 48)).astype(np.float32) / 7))
    bias = rng.standard_normal(5).astype(np.float32)
    fa = W.as_f32(O.linear_bf16(W.bf16_bits(a), W.bf16_bits(w), bias))
    ex = O.linear_exact(a, w, bias)
    assert np.allclose(ex, a.astype(np.float64) @ w.T.astype(np.float64) + bias, atol=1e-5)
    assert helpers.rel_err(fa, ex) < 5e-3
    prev = W.bf16_bits(rng.standard_normal((37, 5)).astype(np.float32))
    fb = W.as_f32(O.linear_bf16(W.bf16_bits(a), W.bf16_bits(w), None, beta=1, result=prev))
    assert helpers.rel_err(fb, a @ w.T + W.as_f32(prev)) < 5e-3


def test_all_gather_reference_grid():
    """Golden vector of the reference's own collective test (all_gather_test.cpp:29-67)."""
    g = np.load(os.path.join(GOLD, "all_gather_grid.npz"))
    out = O.all_gather_bytes([g["shard0"], g["shard1"]], (8, 5, 1), data_size0=4)
    assert np.array_equal(out, g["expect"])
    # the closed form the reference test spells out: 0..19 then 32..51
    assert out.reshape(-1).tolist() == list(range(20)) + list(range(32, 52))


def test_all_gather_ragged_and_dim1():
    rng = np.random.default_rng(8)
    full = rng.integers(0, 255, (7, 6, 3), dtype=np.uint8)
    world = 3                                    # block = 3: ranks own 3, 3, 1 rows
    shards = [full[r * 3:min(7, r * 3 + 3)] for r in range(world)]
    assert np.array_equal(O.all_gather_bytes(shards, (7, 6, 3), data_size0=shards[0].shape[0]), full)
    # sharded on dim 1: data.sizes[0] == out.sizes[0]
    shards1 = [np.ascontiguousarray(full[:, r * 2:r * 2 + 2]) for r in range(world)]
    assert np.array_equal(O.all_gather_bytes(shards1, (7, 6, 3), data_size0=7), full)


def test_oracle_regression_vectors():
    g = np.load(os.path.join(GOLD, "gating_small.npz"))
    w = W.random_gating_case(seed=11, B=2, S=40, H=2, D=16, full_mask_rows=1)
    assert np.array_equal(W.bf16_bits(helpers.oracle_faithful(w, block_size=16)), g["faithful"])
    assert np.allclose(helpers.oracle_exact(w), g["exact"], rtol=0, atol=1e-6)
    g = np.load(os.path.join(GOLD, "global_small.npz"))
    w = W.random_global_case(seed=12, B=2, S=48, zero_mask_rows=1)
    assert np.array_equal(W.bf16_bits(helpers.oracle_faithful(w)), g["faithful"])
    assert np.allclose(helpers.oracle_exact(w), g["exact"], rtol=0, atol=1e-6)


def test_workload_shapes_and_flops():
    # algorithmic work of the five benchmark shapes (2 FLOPs per multiply-add)
    expect = {"msa_row_fp32": 30.199, "triangle_start_384": 53.301, "msa_col_512": 231.928,
              "extra_msa_global": 36.997, "triangle_end_1024": 722.628}
    for name, gf in expect.items():
        kind, dtype, B, S, H, D, c_z, seed = W.spec(name)
        w = W.Workload(name=name, kind=kind, dtype=dtype, B=B, S=S, H=H, D=D, seed=seed, c_z=c_z, has_nb=c_z > 0)
        assert abs(w.flops() / 1e9 - gf) < 0.01, (name, w.flops() / 1e9)
    w = W.make("triangle_start_384", rows=4)
    assert w.arrays["x"].shape == (4, 384, 128) and w.arrays["nb"].shape == (4, 384, 384)
    assert w.arrays["bias"].shape == (4, 384)


def test_layernorm_oracle_against_textbook_formula():
    # the exact variant is the textbook formula; the faithful one (shifted-data sums in fp32, bf16 store,
    # layernorm_kernel.h:22-53) stays within bf16 rounding of it, also for rows with a large common offset
    from kutacc_b200.workloads import as_f32, bf16_bits
    rng = np.random.default_rng(11)
    for size, offset in [(64, 0.0), (128, 50.0), (256, -7.0), (100, 3.0)]:
        x = as_f32(bf16_bits(rng.standard_normal((9, size), dtype=np.float32) * 2 + offset))
        g = rng.standard_normal(size).astype(np.float32)
        b = rng.standard_normal(size).astype(np.float32)
        x64 = x.astype(np.float64)
        ref = (x64 - x64.mean(1, keepdims=True)) / np.sqrt(x64.var(1, keepdims=True) + 1e-5) * g + b
        exact = O.layernorm_exact(x, g, b, 1e-5)
        faithful = as_f32(O.layernorm_bf16(bf16_bits(x), g, b, 1e-5))
        assert np.abs(exact - ref).max() <= 1e-5 * max(np.abs(ref).max(), 1.0)
        assert np.abs(faithful - ref).max() <= 6e-3 * np.abs(ref).max()
    # a constant row: variance 0, output = beta exactly (rstd * 0 * gamma + beta)
    x = np.full((1, 64), 3.0, dtype=np.float32)
    out = as_f32(O.layernorm_bf16(bf16_bits(x), np.ones(64, np.float32), np.full(64, 0.5, np.float32), 1e-5))
    assert np.array_equal(out, np.full((1, 64), 0.5, dtype=np.float32))


def _transpose_golden(world, m, n):
    """The closed-form byte grids of the reference's own test (test/functest/comm/transpose_test.cpp:19-81):
    rank r holds an m x n byte grid counting up from 32*r; after the re-shard rank d holds column block d."""
    data = [((np.arange(m * n) + 32 * r) % 256).astype(np.uint8).reshape(m, n, 1) for r in range(world)]
    bn = (n + world - 1) // world
    full = np.concatenate(data, axis=0)                        # [world*m, n, 1]
    expect = [full[:, d * bn:min(n, (d + 1) * bn)] for d in range(world)]
    return data, expect


def test_transpose_oracle_reproduces_the_reference_golden_grid():
    # transpose_test.cpp: world 2, m = 5 rows per rank, n = 6, len = 1, out [10, 3]; expect_data_0 counts
    # 0,1,2 | 6,7,8 | ... with a jump to 32 at row 5, expect_data_1 the other three columns
    data, expect = _transpose_golden(2, 5, 6)
    got = O.transpose_bytes(data, 10, 6)
    exp0 = np.array([[0, 1, 2], [6, 7, 8], [12, 13, 14], [18, 19, 20], [24, 25, 26],
                     [32, 33, 34], [38, 39, 40], [44, 45, 46], [50, 51, 52], [56, 57, 58]], dtype=np.uint8)
    assert np.array_equal(got[0][:, :, 0], exp0)
    assert np.array_equal(got[1][:, :, 0], exp0 + 3)
    for d in range(2):
        assert np.array_equal(got[d], expect[d])
    # ragged: 7 rows and 5 columns over 3 ranks (the last rank is short in both directions), 4-byte elements
    rng = np.random.default_rng(3)
    full = rng.integers(0, 255, (7, 5, 4), dtype=np.uint8)
    shards = [full[r * 3:min(7, r * 3 + 3)] for r in range(3)]
    outs = O.transpose_bytes(shards, 7, 5)
    for d in range(3):
        assert np.array_equal(outs[d], full[:, d * 2:min(5, d * 2 + 2)])


def test_new_operator_oracles_against_committed_vectors():
    # regression vectors of the oracle itself (tests/golden/make_golden.py) plus the reference's re-shard grid
    from kutacc_b200.workloads import as_f32
    g = np.load(os.path.join(GOLD, "transpose_grid.npz"))
    outs = O.transpose_bytes([g["data0"], g["data1"]], 10, 6)
    assert np.array_equal(outs[0], g["expect0"]) and np.array_equal(outs[1], g["expect1"])
    ln = np.load(os.path.join(GOLD, "layernorm_small.npz"))
    assert np.array_equal(O.layernorm_bf16(ln["x"], ln["gamma"], ln["beta"], float(ln["eps"])), ln["faithful"])
    assert np.allclose(O.layernorm_exact(as_f32(ln["x"]), ln["gamma"], ln["beta"], float(ln["eps"])), ln["exact"], rtol=0, atol=1e-6)
    tr = np.load(os.path.join(GOLD, "transition_small.npz"))
    assert np.array_equal(O.transition_bf16(tr["x"], tr["w1"], tr["b1"], tr["w2"], tr["b2"]), tr["faithful"])
    assert np.allclose(O.transition_exact(as_f32(tr["x"]), as_f32(tr["w1"]), tr["b1"], as_f32(tr["w2"]), tr["b2"]), tr["exact"],
                       rtol=0, atol=1e-5)


def test_triangle_multiplication_oracle():
    """The restatement of src/attention/triangle_multiplication.cpp:25-158 against an independent float64 formula
    and against its committed vectors (tests/golden/make_golden.py)."""
    from kutacc_b200.workloads import as_f32, bf16_bits
    tm = np.load(os.path.join(GOLD, "triangle_multiplication_small.npz"))
    proj, gate = O.tm_calc_proj_bf16(tm["x"], tm["mask"], tm["pw"], tm["pb"], tm["gw"], tm["gb"])
    assert np.array_equal(proj, tm["proj"]) and np.array_equal(gate, tm["gate"])
    assert np.array_equal(O.tm_equation_bf16(proj, tm["right"], False), tm["outgoing"])
    assert np.array_equal(O.tm_equation_bf16(proj, tm["right"], True), tm["incoming"])
    assert np.array_equal(O.tm_last_bf16(proj, gate), tm["last"])
    # float64 textbook formula
    f = lambda a: as_f32(a).astype(np.float64)
    x, mask, pw, gw = f(tm["x"]), f(tm["mask"]), f(tm["pw"]), f(tm["gw"])
    n, c_o = x.shape[0], x.shape[2]
    c_i = pw.shape[0]
    lin = x.reshape(-1, c_o) @ pw.T + tm["pb"]
    g = x.reshape(-1, c_o) @ gw.T + tm["gb"]
    want = (lin * mask.reshape(-1, 1) / (1 + np.exp(-g))).T.reshape(c_i, n, n)
    exact = O.tm_calc_proj_exact(as_f32(tm["x"]), as_f32(tm["mask"]), as_f32(tm["pw"]), tm["pb"], as_f32(tm["gw"]), tm["gb"])
    assert np.abs(exact - want).max() <= 1e-5
    assert np.abs(as_f32(proj) - want).max() <= 1e-2 * np.abs(want).max()
    L, R = f(proj), f(tm["right"])
    for incoming, eq in ((False, "cak,cbk->cab"), (True, "cka,ckb->cab")):
        a, b = (L, R) if not incoming else (R, L)
        ref = np.einsum(eq, a, b)
        got = O.tm_equation_exact(as_f32(proj), as_f32(tm["right"]), incoming)
        assert np.abs(got - ref).max() <= 1e-4
        assert np.abs(as_f32(O.tm_equation_bf16(proj, tm["right"], incoming)) - ref).max() <= 2.0 ** -8 * np.abs(ref).max()
    sig = 1 / (1 + np.exp(-f(gate)))
    assert np.abs(as_f32(O.tm_last_bf16(proj, gate)) - f(proj) * sig).max() <= 1e-2 * np.abs(f(proj)).max()
