"""kutacc_comm_init / kutacc_af2_all_gather over NCCL, one process per GPU (needs >= 2 GPUs).

Follows the reference's collective test (test/functest/comm/all_gather_test.cpp:19-70): rank r holds a
4 x 5 byte grid starting at 32*r and the gathered grid must equal the closed form byte for byte; plus a
ragged, strided, device-resident case checked against the oracle's restatement of the collective.
NVLS is switched off for these short-lived ranks.
"""
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys
    import numpy as np, torch
    sys.path.insert(0, {root!r})
    from kutacc_b200 import api
    from oracle import cpu_oracle as O
    rank, world = int(sys.argv[1]), int(sys.argv[2])
    torch.cuda.set_device(rank)
    api.comm_init(world, rank, 4 * 5)
    # (1) the reference's golden grid, host buffers, sharded on dim 0
    m, n = 4, 5
    mine = (np.arange(m * n, dtype=np.uint8) + 32 * rank).reshape(m, n, 1)
    out = np.zeros((world * m, n, 1), dtype=np.uint8)
    api.all_gather(api.tensor(mine), api.tensor(out))
    expect = np.concatenate([(np.arange(m * n, dtype=np.uint8) + 32 * r).reshape(m, n, 1) for r in range(world)])
    assert np.array_equal(out, expect), (rank, out.reshape(-1).tolist())
    # (2) ragged rows (7 rows over `world` ranks), device tensors, padded output rows
    rng = np.random.default_rng(5)
    full = rng.integers(0, 255, (7, 6, 16), dtype=np.uint8)
    blk = (7 + world - 1) // world
    lo, hi = min(7, rank * blk), min(7, rank * blk + blk)
    src = torch.from_numpy(np.ascontiguousarray(full[lo:hi])).cuda() if hi > lo else torch.zeros((1, 6, 16), dtype=torch.uint8, device="cuda")
    dst = torch.zeros((7, 6, 32), dtype=torch.uint8, device="cuda")
    api.all_gather(api.tensor(src, sizes=[max(hi - lo, 0), 6, 16], strides=[96, 16, 1]),
                   api.tensor(dst, sizes=[7, 6, 16], strides=[192, 32, 1]))
    torch.cuda.synchronize()
    got = dst.cpu().numpy()
    assert np.array_equal(got[:, :, :16], full) and got[:, :, 16:].sum() == 0, rank
    # (3) sharded on dim 1 (data.sizes[0] == out.sizes[0]), in place of the caller's permute
    full1 = rng.integers(0, 255, (4, 2 * world, 8), dtype=np.uint8)
    src1 = torch.from_numpy(np.ascontiguousarray(full1[:, 2 * rank:2 * rank + 2])).cuda()
    dst1 = torch.zeros((4, 2 * world, 8), dtype=torch.uint8, device="cuda")
    api.all_gather(api.tensor(src1), api.tensor(dst1))
    torch.cuda.synchronize()
    assert np.array_equal(dst1.cpu().numpy(), full1), rank
    api.comm_fini()
    print("rank", rank, "ok")
""")


SHARDED_WORKER = textwrap.dedent("""
    import os, sys
    import numpy as np, torch
    sys.path.insert(0, {root!r})
    from kutacc_b200 import api, sharding
    from kutacc_b200 import workloads as W
    rank, world = int(sys.argv[1]), int(sys.argv[2])
    torch.cuda.set_device(rank)
    dev = "cuda:%d" % rank
    w = W.make("triangle_start_384", rows=128, seq=128)
    alone = sharding.ShardedTriangleAttention(w, 0, 1, 1, dev).step().float().cpu().numpy()
    torch.cuda.synchronize()
    api.comm_init(world, rank, 0)
    op = sharding.ShardedTriangleAttention(w, rank, world, 2, dev)
    for _ in range(2):                      # the second step reuses every buffer
        got = op.step().float().cpu().numpy()
    torch.cuda.synchronize()
    api.raise_if_error()
    api.comm_fini()
    # rows are independent and the kernels are the same: every rank holds the whole result, bit for bit
    assert np.array_equal(got, alone), (rank, float(np.abs(got - alone).max()))
    print("rank", rank, "ok")
""")


TRANSPOSE_WORKER = textwrap.dedent("""
    import os, sys
    import numpy as np, torch
    sys.path.insert(0, {root!r})
    from kutacc_b200 import api
    from oracle import cpu_oracle as O
    rank, world = int(sys.argv[1]), int(sys.argv[2])
    torch.cuda.set_device(rank)
    api.comm_init(world, rank, 5 * 6)
    # (1) the reference's golden grid (test/functest/comm/transpose_test.cpp:19-81), host buffers
    m, n = 5, 6
    bn = (n + world - 1) // world
    grids = [((np.arange(m * n) + 32 * r) % 256).astype(np.uint8).reshape(m, n, 1) for r in range(world)]
    out = np.zeros((world * m, bn, 1), dtype=np.uint8)
    api.transpose(api.tensor(grids[rank]), api.tensor(out))
    want = O.transpose_bytes(grids, world * m, n)[rank]
    assert np.array_equal(out[:, :want.shape[1]], want), (rank, out.reshape(-1).tolist())
    if world == 2:
        first = [0, 1, 2] if rank == 0 else [3, 4, 5]
        assert out[0, :, 0].tolist() == first and out[5, :, 0].tolist() == [v + 32 for v in first]
    # (2) ragged rows and columns, device tensors, 8-byte elements, there and back again
    M, N, L = 7, 5, 8
    rng = np.random.default_rng(9)
    full = rng.integers(0, 255, (M, N, L), dtype=np.uint8)
    bm, bnn = (M + world - 1) // world, (N + world - 1) // world
    r0, r1 = min(M, rank * bm), min(M, rank * bm + bm)
    c0, c1 = min(N, rank * bnn), min(N, rank * bnn + bnn)
    rows = torch.from_numpy(np.ascontiguousarray(full[r0:r1])).cuda() if r1 > r0 else torch.zeros((1, N, L), dtype=torch.uint8, device="cuda")
    cols = torch.zeros((M, max(c1 - c0, 1), L), dtype=torch.uint8, device="cuda")
    api.transpose(api.tensor(rows, sizes=[r1 - r0, N, L], strides=[N * L, L, 1]),
                  api.tensor(cols, sizes=[M, c1 - c0, L], strides=[max(c1 - c0, 1) * L, L, 1]))
    torch.cuda.synchronize()
    assert np.array_equal(cols.cpu().numpy()[:, :c1 - c0], full[:, c0:c1]), rank
    back = torch.zeros((max(r1 - r0, 1), N, L), dtype=torch.uint8, device="cuda")
    api.transpose(api.tensor(cols, sizes=[M, c1 - c0, L], strides=[max(c1 - c0, 1) * L, L, 1]),
                  api.tensor(back, sizes=[r1 - r0, N, L], strides=[N * L, L, 1]))
    torch.cuda.synchronize()
    assert np.array_equal(back.cpu().numpy()[:r1 - r0], full[r0:r1]), rank
    api.comm_fini()
    print("rank", rank, "ok")
""")


def _run_ranks(script, world, tag):
    env = dict(os.environ, SHMID=f"kutacc_{tag}_{os.getpid()}", NCCL_NVLS_ENABLE="0", KUTACC_RENDEZVOUS_TIMEOUT_S="60")
    procs = [subprocess.Popen([sys.executable, str(script), str(r), str(world)], env=env, stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r} failed:\n{out[-2000:]}"


@pytest.mark.parametrize("world", [2])
def test_sharded_triangle_attention_over_nccl(kutacc_lib, tmp_path, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    script = tmp_path / "sharded_worker.py"
    script.write_text(SHARDED_WORKER.format(root=ROOT))
    _run_ranks(script, world, "sharded_test")


@pytest.mark.parametrize("world", [2])
def test_transpose_over_nccl(kutacc_lib, tmp_path, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    script = tmp_path / "transpose_worker.py"
    script.write_text(TRANSPOSE_WORKER.format(root=ROOT))
    _run_ranks(script, world, "transpose_test")


def test_transpose_on_one_rank_is_a_strided_copy(kutacc_lib):
    # world_size 1: chunk(x) = x, every element stays; strides in bytes, padded output rows are left alone
    rng = np.random.default_rng(4)
    full = rng.integers(0, 255, (6, 5, 16), dtype=np.uint8)
    src = torch.from_numpy(full).cuda()
    dst = torch.full((6, 5, 32), 9, dtype=torch.uint8, device="cuda")
    from kutacc_b200 import api
    api.transpose(api.tensor(src), api.tensor(dst, sizes=[6, 5, 16], strides=[160, 32, 1]))
    torch.cuda.synchronize()
    got = dst.cpu().numpy()
    assert np.array_equal(got[:, :, :16], full) and (got[:, :, 16:] == 9).all()


@pytest.mark.parametrize("world", [2])
def test_all_gather_over_nccl(kutacc_lib, tmp_path, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT))
    env = dict(os.environ, SHMID=f"kutacc_comm_test_{os.getpid()}", NCCL_NVLS_ENABLE="0", KUTACC_RENDEZVOUS_TIMEOUT_S="60")
    procs = [subprocess.Popen([sys.executable, str(script), str(r), str(world)], env=env, stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=180)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r} failed:\\n{out[-2000:]}"
