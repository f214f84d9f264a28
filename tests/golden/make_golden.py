"""Regenerate tests/golden/*.npz.

Two kinds of vectors live here:
  * all_gather_grid.npz  - the byte grid of the reference's own collective test
    (test/functest/comm/all_gather_test.cpp:29-67), restated from its closed form: rank r holds a
    4 x 5 grid of bytes 32*r + running index; the gathered 8 x 5 grid is the two stacked.
  * transpose_grid.npz   - the byte grids of the reference's re-shard test
    (test/functest/comm/transpose_test.cpp:19-81), restated from their closed form: rank r holds a 5 x 6
    grid counting up from 32*r; afterwards rank d holds the three columns of block d of the stacked grid.
  * gating_small.npz / global_small.npz / layernorm_small.npz / transition_small.npz / triangle_multiplication_small.npz -
    outputs of the CPU oracle (oracle/kutacc_oracle.cpp) on
    small seeded cases. The reference cannot be executed here (ARM SVE sources, closed GEMM), so
    these pin the oracle against accidental change; they are not outputs of the reference.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from kutacc_b200 import workloads as W  # noqa: E402
from tests import helpers  # noqa: E402


def all_gather_grid():
    m, n, world = 4, 5, 2
    shards = [np.array([32 * r + i for i in range(m * n)], dtype=np.uint8).reshape(m, n, 1) for r in range(world)]
    expect = np.concatenate(shards, axis=0)
    np.savez(os.path.join(HERE, "all_gather_grid.npz"), shard0=shards[0], shard1=shards[1], expect=expect)


def gating_small():
    w = W.random_gating_case(seed=11, B=2, S=40, H=2, D=16, full_mask_rows=1)
    np.savez(os.path.join(HERE, "gating_small.npz"), faithful=W.bf16_bits(helpers.oracle_faithful(w, block_size=16)),
             exact=helpers.oracle_exact(w))


def global_small():
    w = W.random_global_case(seed=12, B=2, S=48, zero_mask_rows=1)
    np.savez(os.path.join(HERE, "global_small.npz"), faithful=W.bf16_bits(helpers.oracle_faithful(w)),
             exact=helpers.oracle_exact(w))


def transpose_grid():
    m, n, world = 5, 6, 2
    bn = (n + world - 1) // world
    data = [np.array([(32 * r + i) % 256 for i in range(m * n)], dtype=np.uint8).reshape(m, n, 1) for r in range(world)]
    # expect_data_0 / expect_data_1 of the reference test: rows of both ranks stacked, columns of block d
    expect = []
    for d in range(world):
        e = np.zeros((world * m, bn, 1), dtype=np.uint8)
        for i in range(world * m):
            src_rank, row = divmod(i, m)
            for j in range(bn):
                e[i, j, 0] = (32 * src_rank + row * n + d * bn + j) % 256
        expect.append(e)
    np.savez(os.path.join(HERE, "transpose_grid.npz"), data0=data[0], data1=data[1], expect0=expect[0], expect1=expect[1])


def layernorm_small():
    from oracle import cpu_oracle as O
    rng = np.random.default_rng(13)
    x = W.bf16_bits(rng.standard_normal((6, 96), dtype=np.float32) * 1.5 + 2.0)
    g = rng.standard_normal(96).astype(np.float32)
    b = rng.standard_normal(96).astype(np.float32)
    np.savez(os.path.join(HERE, "layernorm_small.npz"), x=x, gamma=g, beta=b, eps=np.float32(1e-5),
             faithful=O.layernorm_bf16(x, g, b, 1e-5), exact=O.layernorm_exact(W.as_f32(x), g, b, 1e-5))


def transition_small():
    from oracle import cpu_oracle as O
    rng = np.random.default_rng(14)
    x = W.bf16_bits(rng.standard_normal((10, 32), dtype=np.float32))
    w1 = W.bf16_bits(rng.standard_normal((128, 32), dtype=np.float32) / np.sqrt(32))
    w2 = W.bf16_bits(rng.standard_normal((32, 128), dtype=np.float32) / np.sqrt(128))
    b1 = rng.standard_normal(128).astype(np.float32)
    b2 = rng.standard_normal(32).astype(np.float32)
    np.savez(os.path.join(HERE, "transition_small.npz"), x=x, w1=w1, b1=b1, w2=w2, b2=b2,
             faithful=O.transition_bf16(x, w1, b1, w2, b2),
             exact=O.transition_exact(W.as_f32(x), W.as_f32(w1), b1, W.as_f32(w2), b2))


def triangle_multiplication_small():
    from oracle import cpu_oracle as O
    rng = np.random.default_rng(15)
    n, c_o, c_i = 10, 16, 8
    x = W.bf16_bits(rng.standard_normal((n, n, c_o), dtype=np.float32))
    mask = W.bf16_bits((rng.random((n, n)) >= 0.2).astype(np.float32))
    pw = W.bf16_bits(rng.standard_normal((c_i, c_o), dtype=np.float32) / 4)
    gw = W.bf16_bits(rng.standard_normal((c_i, c_o), dtype=np.float32) / 4)
    pb = rng.standard_normal(c_i).astype(np.float32)
    gb = rng.standard_normal(c_i).astype(np.float32)
    right = W.bf16_bits(rng.standard_normal((c_i, n, n), dtype=np.float32))
    proj, gate = O.tm_calc_proj_bf16(x, mask, pw, pb, gw, gb)
    np.savez(os.path.join(HERE, "triangle_multiplication_small.npz"), x=x, mask=mask, pw=pw, pb=pb, gw=gw, gb=gb, right=right,
             proj=proj, gate=gate, outgoing=O.tm_equation_bf16(proj, right, False),
             incoming=O.tm_equation_bf16(proj, right, True), last=O.tm_last_bf16(proj, gate))


if __name__ == "__main__":
    all_gather_grid()
    transpose_grid()
    gating_small()
    global_small()
    layernorm_small()
    transition_small()
    triangle_multiplication_small()
    print("golden vectors written to", HERE)
