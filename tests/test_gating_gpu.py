"""Parity of kutacc_af2_gating_attention (CUDA, through the C ABI) with the CPU oracle."""
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


# (B, S, H, D, with_nb): tensor-core path shapes, including ragged sequence lengths
FAST_SHAPES = [
    (2, 64, 2, 32, True), (3, 70, 2, 32, True), (2, 129, 4, 32, False), (1, 200, 4, 16, True),
    (2, 96, 1, 64, True), (5, 33, 2, 32, False), (2, 384, 4, 32, True), (1, 8, 2, 32, True),
]


@pytest.mark.parametrize("B,S,H,D,with_nb", FAST_SHAPES)
def test_bf16_tensor_core_path_matches_faithful_oracle(kutacc_lib, B, S, H, D, with_nb):
    w = W.random_gating_case(seed=100 + S, B=B, S=S, H=H, D=D, with_nb=with_nb, full_mask_rows=1 if B > 1 else 0)
    before = api.launch_count()
    got = _run(w)
    # projection, attention core, output projection (a pair bias with unaligned rows is re-pitched by a
    # 2-D device copy first, which is not a kernel of this library)
    assert api.launch_count() - before == 3
    ref = helpers.oracle_faithful(w)
    assert helpers.rel_err(got, ref) <= helpers.BF16_TOL
    assert helpers.rel_err(got, helpers.oracle_exact(w)) <= 3 * helpers.BF16_TOL   # the reference's own distance
    assert np.isfinite(got).all()


# shapes outside the tensor-core kernels: odd head size / channel count, unaligned pair-bias rows
GENERIC_SHAPES = [(2, 37, 3, 8, True), (1, 50, 2, 12, False), (2, 45, 2, 32, True), (1, 40, 1, 80, True)]


@pytest.mark.parametrize("B,S,H,D,with_nb", GENERIC_SHAPES)
def test_bf16_generic_path_matches_faithful_oracle(kutacc_lib, B, S, H, D, with_nb):
    w = W.random_gating_case(seed=200 + S, B=B, S=S, H=H, D=D, with_nb=with_nb, full_mask_rows=0)
    got = _run(w)
    assert helpers.rel_err(got, helpers.oracle_faithful(w)) <= helpers.BF16_TOL


@pytest.mark.parametrize("B,S,H,D,with_nb", [(2, 64, 2, 32, True), (3, 50, 4, 16, False), (1, 100, 8, 32, True)])
def test_fp32_matches_exact_oracle(kutacc_lib, B, S, H, D, with_nb):
    w = W.random_gating_case(seed=300 + S, B=B, S=S, H=H, D=D, dtype="fp32", with_nb=with_nb, full_mask_rows=1)
    got = _run(w)
    assert helpers.rel_err(got, helpers.oracle_exact(w)) <= helpers.FP32_TOL


@pytest.mark.parametrize("B,S,H,D", [(3, 70, 4, 32), (2, 129, 8, 32), (1, 300, 8, 16)])
def test_fp32_projections_run_on_the_tensor_memory_gemm(kutacc_lib, B, S, H, D):
    """fp32 with nchannels a multiple of 128: the projections and the output projection go through the tcgen05 tf32
    GEMM on operands split into head and tail (three products per multiply), which must stay at fp32 accuracy; the
    row count B * S is not a multiple of the 128-row tile."""
    w = W.random_gating_case(seed=400 + S, B=B, S=S, H=H, D=D, dtype="fp32", with_nb=True, full_mask_rows=0)
    case = runner.DeviceCase(w)
    api.set_profile(True)
    api.profile_read()
    got = runner.out_to_f32(case.run())
    names = [k for k, _ in api.profile_read()]
    api.set_profile(False)
    assert names.count("gemm_tf32x3_tc") == 2 and "gemm_tf32x3" not in names
    assert helpers.rel_err(got, helpers.oracle_exact(w)) <= helpers.FP32_TOL
    # the host-buffer call takes the same kernels chunk by chunk
    assert np.array_equal(_run(w, device=False), got)


def test_fully_masked_row_is_uniform(kutacc_lib):
    # every key of batch row 0 carries -1e9: the softmax must be uniform, not NaN or zero
    w = W.random_gating_case(seed=5, B=2, S=128, H=2, D=32, with_nb=True, full_mask_rows=1)
    got = _run(w)
    ref = helpers.oracle_faithful(w)
    assert np.isfinite(got).all()
    assert helpers.rel_err(got[0], ref[0]) <= helpers.BF16_TOL


def test_running_max_that_grows_late_in_the_key_sequence(kutacc_lib):
    """The kernel forms probabilities against a running max that it raises lazily. Rows whose first keys are masked
    (-1e9) and whose later keys are not make the max grow by far more than the 2^8 slack at a later tile: in the
    first or in the second group of 16 keys of a thread's half of the tile (the second group also rescales the
    probabilities the first one has already stored), and large pair-bias steps do the same without any mask."""
    w = W.random_gating_case(seed=21, B=6, S=320, H=4, D=32, with_nb=True, mask_frac=0.0)
    A = w.arrays
    mask = np.ones((w.B, w.S), np.float32)
    mask[0, :80] = 0.0           # tile 1: keys 64..79 masked, 80.. open -> growth in the second group of half 0
    mask[1, :96] = 0.0           # tile 1: half 0 masked whole, growth in the first group of half 1
    mask[2, :200] = 0.0          # growth in tile 3
    mask[3, 10:300] = 0.0        # open keys first, a long masked stretch, open again
    mask[4, :] = 0.0             # fully masked
    A["mask"] = mask
    A["bias"] = np.ascontiguousarray(1e9 * (mask - 1.0), np.float32)
    nb = A["nb"].copy()
    nb[:, :, 150:170] += 40.0    # a step of 40 in the logits late in the sequence (row 5 has no mask at all)
    A["nb"] = W.as_f32(W.bf16_bits(nb))
    got = _run(w)
    assert np.isfinite(got).all()
    assert helpers.rel_err(got, helpers.oracle_faithful(w)) <= helpers.BF16_TOL


def test_host_pointers_give_the_same_bits_as_device_pointers(kutacc_lib):
    w = W.random_gating_case(seed=7, B=3, S=96, H=4, D=32, with_nb=True)
    dev = _run(w, device=True)
    host = _run(w, device=False)
    assert np.array_equal(dev, host)


def test_pipelined_host_path_matches_device_path(kutacc_lib):
    # large enough (>= 8 batch rows, >= 4 MiB of activations) for the chunked upload/compute/download pipeline
    w = W.random_gating_case(seed=8, B=35, S=256, H=8, D=32, with_nb=True, full_mask_rows=2)
    dev = _run(w, device=True)
    host = _run(w, device=False)
    assert np.array_equal(dev, host)
    assert np.array_equal(_run(w, device=False), host)       # staging buffers are reused across calls


def test_strided_host_out_keeps_the_bytes_between_rows(kutacc_lib):
    """A HOST `out` whose row stride is wider than nchannels: the reference writes through strides()[1] and
    touches only the C elements of each row, so the padding must come back unchanged (plain and chunked path)."""
    for B, S in ((2, 64), (35, 256)):
        w = W.random_gating_case(seed=19, B=B, S=S, H=4, D=32, with_nb=False)
        dense = _run(w, device=False).copy()
        host = runner.HostCase(w)
        pad = torch.full((w.B, w.S, w.C + 16), 7.0, dtype=torch.bfloat16).pin_memory()
        api.gating_attention(host.t_x, host.inputs, host.t_bias, host.t_nb, host.weights,
                             api.tensor(pad, sizes=[w.B, w.S, w.C], strides=[w.S * (w.C + 16), w.C + 16, 1]))
        got = pad.float().numpy()
        assert np.array_equal(got[:, :, :w.C], dense)
        assert (got[:, :, w.C:] == 7.0).all()


def test_strided_out_and_bias(kutacc_lib):
    # out row stride (strides[1]) and bias row stride (strides[0]) are honoured
    w = W.random_gating_case(seed=9, B=2, S=64, H=2, D=32, with_nb=False)
    case = runner.DeviceCase(w)
    dense = runner.out_to_f32(case.run()).copy()
    pad = torch.full((w.B, w.S, w.C + 16), 7.0, dtype=torch.bfloat16, device="cuda:0")
    bias_pad = torch.zeros((w.B, w.S + 8), dtype=torch.bfloat16, device="cuda:0")
    bias_pad[:, :w.S] = case.bias
    api.gating_attention(case.t_x, case.inputs, api.tensor(bias_pad, sizes=[w.B, w.S], strides=[w.S + 8, 1]), case.t_nb,
                         case.weights, api.tensor(pad, sizes=[w.B, w.S, w.C], strides=[w.S * (w.C + 16), w.C + 16, 1]))
    torch.cuda.synchronize()
    got = pad.float().cpu().numpy()
    assert np.array_equal(got[:, :, :w.C], dense)
    assert (got[:, :, w.C:] == 7.0).all()              # padding untouched


@pytest.mark.parametrize("name,rows", [("triangle_start_384", 24), ("msa_col_512", 12), ("triangle_end_1024", 4)])
def test_benchmark_shapes_subsampled_rows(kutacc_lib, name, rows):
    # the benchmark shapes at full sequence length on the first `rows` batch rows
    w = W.make(name, rows=rows)
    got = _run(w)
    assert helpers.rel_err(got, helpers.oracle_faithful(w)) <= helpers.BF16_TOL


def _pick_rows(w, rows):
    """The batch rows `rows` of a gating workload as a workload of their own (weights and pair bias shared)."""
    pick = W.Workload(name="pick", kind="gating", dtype=w.dtype, B=len(rows), S=w.S, H=w.H, D=w.D, seed=0, has_nb=w.has_nb)
    pick.arrays = dict(w.arrays)
    pick.arrays["x"] = w.arrays["x"][rows]
    pick.arrays["bias"] = w.arrays["bias"][rows]
    return pick


@pytest.mark.parametrize("name,rows", [("triangle_end_1024", [0, 1, 510, 511, 1022, 1023]),
                                       ("msa_col_512", [0, 1, 190, 191, 382, 383])])
def test_full_size_rows_spread_over_the_batch(kutacc_lib, name, rows):
    """The two largest gating shapes at FULL size on the GPU; the oracle checks rows at the start, in the middle
    and at the end of the batch (both rows of a pair the kernel processes together), and a sub-batch must give
    the same bits as the full call (rows are independent problems)."""
    w = W.make(name)
    full = _run(w)
    assert np.isfinite(full).all()
    assert helpers.rel_err(full[rows], helpers.oracle_faithful(_pick_rows(w, rows))) <= helpers.BF16_TOL
    sub = W.make(name, rows=5)                           # odd: the last row has no partner in its pair
    assert np.array_equal(_run(sub), full[:5])


def test_msa_row_fp32_shape_subsampled(kutacc_lib):
    w = W.make("msa_row_fp32", rows=6)
    got = _run(w)
    assert helpers.rel_err(got, helpers.oracle_exact(w)) <= helpers.FP32_TOL


def test_full_size_properties_triangle_start(kutacc_lib):
    """Size-independent checks at the full benchmark size (the oracle is too slow for all of it):
    rows are independent problems, and the output bias enters linearly."""
    w = W.make("triangle_start_384")
    case = runner.DeviceCase(w)
    full = runner.out_to_f32(case.run()).copy()
    assert np.isfinite(full).all()
    # (1) a sub-batch gives bit-identical rows
    sub = W.make("triangle_start_384", rows=16)
    assert np.array_equal(runner.out_to_f32(runner.DeviceCase(sub).run()), full[:16])
    # (2) oracle on a few rows spread over the batch, including a fully masked one
    masked = np.where(w.arrays["mask"].sum(1) == 0)[0]
    rows = sorted(set([0, 191, 383] + masked[:1].tolist()))
    assert helpers.rel_err(full[rows], helpers.oracle_faithful(_pick_rows(w, rows))) <= helpers.BF16_TOL
    # (3) shifting the output bias shifts the output by the same amount (up to bf16 rounding)
    case.bo += 0.5
    shifted = runner.out_to_f32(case.run())
    assert np.abs((shifted - full) - 0.5).max() <= 2.0 ** -6 * max(1.0, np.abs(full).max())


def test_repeat_calls_are_deterministic(kutacc_lib):
    w = W.random_gating_case(seed=13, B=4, S=160, H=4, D=32, with_nb=True)
    case = runner.DeviceCase(w)
    a = runner.out_to_f32(case.run()).copy()
    b = runner.out_to_f32(case.run()).copy()
    assert np.array_equal(a, b)


def test_sharded_triangle_flow_on_one_rank_matches_the_plain_call(kutacc_lib):
    # pair-bias projection + attention slab by slab (kutacc_b200/sharding.py) against one call with the
    # workload's own pair bias; the two biases may differ in the last bf16 bit (fp32 summation order of the host's
    # BLAS against the kernel's), which can move an output by one bf16 step (2^-8 relative)
    from kutacc_b200 import sharding
    w = W.make("triangle_start_384", rows=128, seq=128)
    want = runner.out_to_f32(runner.DeviceCase(w).run())
    op = sharding.ShardedTriangleAttention(w, 0, 1, 2, "cuda:0")
    got = runner.out_to_f32(op.step())
    torch.cuda.synchronize()
    api.raise_if_error()
    assert helpers.rel_err(got, want) <= 5e-3
    assert helpers.rel_err(got, helpers.oracle_faithful(w)) <= helpers.BF16_TOL


def test_host_rows_flow_with_and_without_prefetch_matches_the_device_flow(kutacc_lib):
    # rows of z in pinned host memory, output rows to pinned host memory (sharding.HostShardedTriangleAttention):
    # every step, stand-alone or with the next step's upload already in flight, gives the device flow's bits
    from kutacc_b200 import sharding
    w = W.make("triangle_start_384", rows=128, seq=128)
    want = runner.out_to_f32(sharding.ShardedTriangleAttention(w, 0, 1, 1, "cuda:0").step()).copy()
    host = sharding.HostShardedTriangleAttention(w, 0, 1, "cuda:0")
    for prefetch in (False, True, True, False, True):
        out = host.step(prefetch=prefetch)
        if prefetch:
            host.drain()                      # a prefetching step only queues its work
        assert np.array_equal(out.float().numpy(), want)
        host.hout.zero_()
    # three steps queued back to back before anything is waited for
    for _ in range(3):
        host.step()
    host.drain()
    assert np.array_equal(host.hout.float().numpy(), want)
    torch.cuda.synchronize()
    api.raise_if_error()


def test_enqueue_only_call_with_host_out_is_complete_after_synchronize(kutacc_lib):
    """An enqueue-only call whose `out` is in HOST memory returns with its chunked downloads in flight;
    kutacc_b200_synchronize waits for them, and a following call of another shape orders itself after them."""
    w = W.random_gating_case(seed=8, B=35, S=256, H=8, D=32, with_nb=True, full_mask_rows=2)
    want = _run(w, device=True)
    host = runner.HostCase(w)
    other = W.random_gating_case(seed=9, B=18, S=512, H=8, D=32, with_nb=False)       # chunked too, other chunks
    tiny = W.random_gating_case(seed=10, B=2, S=64, H=2, D=32, with_nb=True)           # one chunk, staged whole
    want_other, want_tiny = _run(other, device=True), _run(tiny, device=True)
    host_other, host_tiny = runner.HostCase(other), runner.HostCase(tiny)
    api.set_async(True)
    try:
        for _ in range(2):                    # the second call finds the downloads of the first in flight
            api.gating_attention(host.t_x, host.inputs, host.t_bias, host.t_nb, host.weights, host.t_out)
        for c in (host_other, host, host_tiny):
            api.gating_attention(c.t_x, c.inputs, c.t_bias, c.t_nb, c.weights, c.t_out)
        api.synchronize()
    finally:
        api.set_async(False)
    assert np.array_equal(runner.out_to_f32(host.out), want)
    assert np.array_equal(runner.out_to_f32(host_other.out), want_other)
    assert np.array_equal(runner.out_to_f32(host_tiny.out), want_tiny)


@pytest.mark.parametrize("B,S,H,D", [(3, 200, 4, 32), (2, 129, 4, 32), (2, 70, 2, 16)])
def test_pair_bias_stored_with_the_heads_inside_the_rows(kutacc_lib, B, S, H, D):
    """The pair bias handed over as [H, S, S] through strides over a [S, H, S] storage (what the sharded flow
    gathers in place): the same bits as with the dense [H, S, S] tensor (head size 32: the tcgen05 core with the
    tensor-map dimensions in stride order; head size 16: the generic kernel)."""
    w = W.random_gating_case(seed=60 + S, B=B, S=S, H=H, D=D, with_nb=True, full_mask_rows=1 if B > 2 else 0)
    case = runner.DeviceCase(w)
    want = runner.out_to_f32(case.run()).copy()
    sp = (S + 7) // 8 * 8                                   # rows of 16-byte multiples for the TMA path
    store = torch.zeros((S, H, sp), dtype=case.nb.dtype, device="cuda:0")
    store[:, :, :S] = case.nb.permute(1, 0, 2)
    t_nb = api.Tensor(store.data_ptr(), [H, S, S], [sp, H * sp, 1], api.DTYPE_BF16, keep=store)
    api.gating_attention(case.t_x, case.inputs, case.t_bias, t_nb, case.weights, case.t_out)
    torch.cuda.synchronize()
    assert np.array_equal(runner.out_to_f32(case.out), want)


def test_pair_bias_still_on_its_way_is_waited_for(kutacc_lib):
    """kutacc_b200_set_pair_bias_event: the pair bias is written by another stream long after the call has been
    queued; the call's attention kernel (not its projections) waits for the event, once."""
    w = W.random_gating_case(seed=31, B=4, S=200, H=4, D=32, with_nb=True)
    case = runner.DeviceCase(w)
    want = runner.out_to_f32(case.run()).copy()
    nb_src = case.nb.clone()
    # two streams of their own: the legacy default stream would wait for the side stream by itself
    main, side = torch.cuda.Stream(), torch.cuda.Stream()
    ev = torch.cuda.Event()
    api.set_async(True)
    api.set_stream(main.cuda_stream)
    try:
        for _ in range(2):                                   # the second call must not wait for anything
            case.nb.zero_()
            torch.cuda.synchronize()
            with torch.cuda.stream(side):
                torch.cuda._sleep(20_000_000)                # about 10 ms: the call below is queued long before the bias exists
                case.nb.copy_(nb_src, non_blocking=True)
                ev.record(side)
            api.set_pair_bias_event(ev)
            out = case.run()
            main.synchronize()
            assert np.array_equal(runner.out_to_f32(out), want)
            torch.cuda.synchronize()
            out = case.run()                                 # no event set: uses the bias as it lies
            main.synchronize()
            assert np.array_equal(runner.out_to_f32(out), want)
    finally:
        api.set_stream(0)
        api.set_async(False)
        api.set_pair_bias_event(None)


def test_sm_margin_changes_the_grid_not_the_result(kutacc_lib):
    # the persistent kernels walk their work items with a stride of the grid size: leaving SMs free for a
    # collective must not change a single bit
    w = W.random_gating_case(seed=77, B=6, S=200, H=4, D=32)
    case = runner.DeviceCase(w)
    want = runner.out_to_f32(case.run()).copy()
    api.set_sm_margin(40)
    try:
        got = runner.out_to_f32(case.run()).copy()
    finally:
        api.set_sm_margin(0)
    torch.cuda.synchronize()
    assert np.array_equal(got, want)
