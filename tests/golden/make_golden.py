"""Regenerate tests/golden/*.npz.

Two kinds of vectors live here:
  * all_gather_grid.npz  - the byte grid of the reference's own collective test
    (test/functest/comm/all_gather_test.cpp:29-67), restated from its closed form: rank r holds a
    4 x 5 grid of bytes 32*r + running index; the gathered 8 x 5 grid is the two stacked.
  * gating_small.npz / global_small.npz - outputs of the CPU oracle (oracle/kutacc_oracle.cpp) on
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


if __name__ == "__main__":
    all_gather_grid()
    gating_small()
    global_small()
    print("golden vectors written to", HERE)
