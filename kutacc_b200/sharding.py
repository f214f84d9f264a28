"""Row partition used when the batch rows of an attention call are spread over several GPUs.

Same formula as the reference's collectives (include/kutacc.h:58-74, src/comm/all_gather.cpp:35,48):
block(x) = ceil(x / world), rank r owns rows [r*block, min((r+1)*block, x)).
"""
from __future__ import annotations

from typing import Tuple


def block(x: int, world: int) -> int:
    return (x + world - 1) // world


def chunk(x: int, world: int, rank: int) -> int:
    return max(0, min(block(x, world), x - rank * block(x, world)))


def row_range(x: int, world: int, rank: int) -> Tuple[int, int]:
    b = block(x, world)
    lo = min(x, rank * b)
    return lo, lo + chunk(x, world, rank)


# ---------------------------------------------------------------------------------------------------
# Triangle attention with its rows spread over several GPUs
#
# The operator itself never communicates (as in the reference, where the caller shards and gathers):
# every rank projects the pair bias of the rows of z it holds, the ranks all-gather the bias
# [H, N, N], every rank runs the gated attention on its rows against the whole bias, and the ranks
# all-gather the output rows. To let the output gather of one part run while the next part is being
# computed, the N rows are cut into `nslab` contiguous slabs and inside each slab rank r owns block r:
# the gather of a slab is then a dense in-place all-gather, issued on its own stream.
# ---------------------------------------------------------------------------------------------------
def slab_plan(n_rows: int, world: int, nslab: int):
    """[(slab_start, slab_rows, block_rows)] for each slab; every slab splits evenly over the ranks."""
    if nslab < 1 or n_rows % (world * nslab) != 0:
        raise ValueError(f"{n_rows} rows do not split into {nslab} slabs of {world} equal blocks")
    slab_rows = n_rows // nslab
    return [(c * slab_rows, slab_rows, slab_rows // world) for c in range(nslab)]


def owned_rows(n_rows: int, world: int, rank: int, nslab: int):
    """[(first_row, n)] of the rows rank `rank` owns, one entry per slab."""
    return [(start + rank * blk, blk) for start, _, blk in slab_plan(n_rows, world, nslab)]


class ShardedTriangleAttention:
    """One rank's share of a triangle-attention workload (x = z, pair bias projected from z).

    ``step()`` runs pair-bias projection -> bias all-gather -> per slab: attention, output all-gather
    (the gather of slab c overlaps the attention of slab c + 1). After ``step()`` every rank holds the
    whole output in ``out_full`` (with ``gather_output=False`` only its own rows, as the reference operator
    leaves them). With world == 1 the gathers are skipped.
    """

    def __init__(self, w, rank: int, world: int, nslab: int, device, sm_margin: int = 8, bias_gather_beside: bool = True):
        import numpy as np
        import torch
        from . import api
        from .runner import _to_torch
        assert w.kind == "gating" and "wb" in w.arrays and w.B == w.S, "needs a full triangle workload"
        self.w, self.rank, self.world, self.device = w, rank, world, device
        self.sm_margin = sm_margin if world > 1 else 0      # SMs left to the collective that runs beside the kernels
        self.bias_gather_beside = bias_gather_beside        # bias gather on the collective's stream, beside the projections
        self.api = api
        N, S, C, H = w.B, w.S, w.C, w.H
        self.slabs = slab_plan(N, world, nslab)
        self.mine = owned_rows(N, world, rank, nslab)
        A = w.arrays
        dt = api.DTYPE_BF16 if w.dtype == "bf16" else api.DTYPE_FP32
        esz = 2 if w.dtype == "bf16" else 4
        f = lambda a: _to_torch(a, w.dtype, device)
        f32 = lambda a: _to_torch(a, "fp32", device)
        # this rank's rows only (activations, mask bias); weights everywhere
        self.x = [f(A["x"][r0:r0 + n]) for r0, n in self.mine]
        self.bias = [f(A["bias"][r0:r0 + n]) for r0, n in self.mine]
        self.wq, self.wk, self.wv, self.wg, self.wo = (f(A[k]) for k in ("wq", "wk", "wv", "wg", "wo"))
        self.bg, self.bo = f32(A["bg"]), f32(A["bo"])
        self.wb = f(np.ascontiguousarray(A["wb"].T))                                   # [H, c_z]
        tdt = torch.bfloat16 if w.dtype == "bf16" else torch.float32
        # The pair bias is stored with the heads of a query row next to each other, [S, H, S]: the rows a rank
        # projects are then one dense block per slab, so a slab's share of the bias is gathered in place by ONE
        # collective (with [H, S, S] storage every (head, slab) strip needed a call of its own, and queueing those
        # calls cost more host time than the gather takes). The operators see it as [H, S, S] through strides.
        self.nb_full = torch.zeros((S, H, S), dtype=tdt, device=device)
        self.out_full = torch.zeros((N, S, C), dtype=tdt, device=device)
        self.weights = api.make_weights(C, H, w.D, self.wq, self.wk, self.wv, self.wg, self.bg, self.wo, self.bo)
        self.t_wb = api.tensor(self.wb)
        self.t_nb = api.Tensor(self.nb_full.data_ptr(), [H, S, S], [S, H * S, 1], dt, keep=self.nb_full)
        self.parts = []
        for (r0, n), (s0, srows, blk), x, bias in zip(self.mine, self.slabs, self.x, self.bias):
            nb_rows = self.nb_full[r0:r0 + n]
            out_rows = self.out_full[r0:r0 + n]
            part = {
                "inputs": api.make_inputs(n, S),
                "t_x": api.tensor(x, sizes=[n * S, C], strides=[C, 1]),
                "t_z": api.tensor(x),                                                   # z[q, k, :] = x[q, k, :]
                "t_bias": api.tensor(bias),
                "t_nb_rows": api.Tensor(nb_rows.data_ptr(), [H, n, S], [S, H * S, 1], dt, keep=self.nb_full),
                "t_out_rows": api.Tensor(out_rows.data_ptr(), [n, S, C], [S * C, C, 1], dt, keep=self.out_full),
                # byte views for the collectives: [m, n, len]
                "g_nb_src": api.Tensor(nb_rows.data_ptr(), [n, 1, H * S * esz], [H * S * esz, H * S * esz, 1],
                                       api.DTYPE_BF16, keep=self.nb_full),
                "g_nb_dst": api.Tensor(self.nb_full[s0:s0 + srows].data_ptr(), [srows, 1, H * S * esz],
                                       [H * S * esz, H * S * esz, 1], api.DTYPE_BF16, keep=self.nb_full),
                "g_out_src": api.Tensor(out_rows.data_ptr(), [n, S, C * esz], [S * C * esz, C * esz, 1], api.DTYPE_BF16,
                                        keep=self.out_full),
                "g_out_dst": api.Tensor(self.out_full[s0:s0 + srows].data_ptr(), [srows, S, C * esz],
                                        [S * C * esz, C * esz, 1], api.DTYPE_BF16, keep=self.out_full),
            }
            self.parts.append(part)
        # Every slab's share in ONE call: [S, H, S] with S = nslab * srows rows is also [nslab, srows, H * S], and inside
        # every slab rank r owns block r (the library gathers such strips in place, as one group of collectives).
        srows, blk = self.slabs[0][1], self.slabs[0][2]
        row = H * S * esz
        self.g_nb_src_all = api.Tensor(self.nb_full.data_ptr() + rank * blk * row, [nslab, blk, row], [srows * row, row, 1],
                                       api.DTYPE_BF16, keep=self.nb_full)
        self.g_nb_dst_all = api.Tensor(self.nb_full.data_ptr(), [nslab, srows, row], [srows * row, row, 1],
                                       api.DTYPE_BF16, keep=self.nb_full)
        self.compute = torch.cuda.current_stream(device)
        self.comm = torch.cuda.Stream(device=device)
        self.events = [torch.cuda.Event() for _ in self.parts]
        self.bias_projected, self.bias_gathered = torch.cuda.Event(), torch.cuda.Event()
        # phase marks of the last step, all on the compute stream
        self.marks = [torch.cuda.Event(enable_timing=True) for _ in range(5)]

    def phase_ms(self):
        """Device time of the phases of the last ``step()`` (synchronise first): pair-bias projection, bias
        all-gather, attention (all slabs, with the overlapped output gathers beside it), and the part of the
        output gather that was still running when the last attention kernel had finished."""
        m = self.marks
        return {"bias_projection": m[0].elapsed_time(m[1]), "bias_all_gather": m[1].elapsed_time(m[2]),
                "attention": m[2].elapsed_time(m[3]), "exposed_output_gather": m[3].elapsed_time(m[4])}

    def step(self, block_size: int = 128, gather_output: bool = True):
        api = self.api
        api.set_async(True)
        api.set_sm_margin(self.sm_margin)
        try:
            api.set_stream(self.compute.cuda_stream)
            self.marks[0].record(self.compute)
            for p in self.parts:
                api.pair_bias(p["t_z"], self.t_wb, p["t_nb_rows"])
            self.marks[1].record(self.compute)
            if self.world > 1 and not self.bias_gather_beside:
                api.all_gather(self.g_nb_src_all, self.g_nb_dst_all)        # one in-place gather per slab, one group
            elif self.world > 1:
                # the bias strips travel on the collective's stream while the first slab's projections run: the
                # attention call waits for the gather between its projections and its attention kernel
                self.bias_projected.record(self.compute)
                self.comm.wait_event(self.bias_projected)
                api.set_stream(self.comm.cuda_stream)
                api.all_gather(self.g_nb_src_all, self.g_nb_dst_all)        # one in-place gather per slab, one group
                self.bias_gathered.record(self.comm)
                api.set_stream(self.compute.cuda_stream)
                api.set_pair_bias_event(self.bias_gathered)
            self.marks[2].record(self.compute)
            for p, ev in zip(self.parts, self.events):
                api.set_stream(self.compute.cuda_stream)
                api.gating_attention(p["t_x"], p["inputs"], p["t_bias"], self.t_nb, self.weights, p["t_out_rows"],
                                     block_size)
                if self.world > 1 and gather_output:
                    ev.record(self.compute)
                    self.comm.wait_event(ev)
                    api.set_stream(self.comm.cuda_stream)
                    api.all_gather(p["g_out_src"], p["g_out_dst"])
            self.marks[3].record(self.compute)
            self.compute.wait_stream(self.comm)
            self.marks[4].record(self.compute)
        finally:
            api.set_stream(self.compute.cuda_stream)
            api.set_async(False)
            api.set_sm_margin(0)
        return self.out_full


class HostShardedTriangleAttention:
    """The same flow for a caller whose activations and result live in host memory: one rank's rows of z and of
    the mask bias are in pinned host buffers, its rows of the output land in a pinned host buffer.

    ``step()`` copies the rows to the device, projects their pair bias, all-gathers the bias (world > 1) and calls
    the gated attention with a HOST ``out``: the library then runs the batch rows in chunks and overlaps the
    download of chunk i with the kernels of chunk i + 1. Every rank ends with its own rows in host memory (the
    ranks of one node share that memory, so nothing is gathered). Rank r owns the contiguous block r.

    The attention of a step needs the pair bias of EVERY row, so inside one step the upload cannot overlap the
    kernels or the download. With ``prefetch=True`` (the default) the device side of the input is double-buffered
    and a step starts the upload of the NEXT step's rows on a stream of its own just before it queues the
    attention call: the upload of step i + 1 then travels beside the kernels and the download of step i (the link
    is full duplex), and the calls only queue work, so the first chunks of step i + 1 are computed beside the last
    downloads of step i. ``step(prefetch=False)`` runs one step on its own (its latency). ``drain()`` waits for
    everything queued.
    """

    def __init__(self, w, rank: int, world: int, device):
        import numpy as np
        import torch
        from . import api
        from .runner import _to_torch
        assert w.kind == "gating" and "wb" in w.arrays and w.B == w.S, "needs a full triangle workload"
        self.w, self.rank, self.world, self.device, self.api = w, rank, world, device, api
        N, S, C, H = w.B, w.S, w.C, w.H
        r0, r1 = row_range(N, world, rank)
        n = r1 - r0
        assert n > 0 and N % world == 0, "rows must split evenly over the ranks"
        self.rows = (r0, n)
        A = w.arrays
        dt = api.DTYPE_BF16 if w.dtype == "bf16" else api.DTYPE_FP32
        esz = 2 if w.dtype == "bf16" else 4
        tdt = torch.bfloat16 if w.dtype == "bf16" else torch.float32
        self.hx = _to_torch(A["x"][r0:r0 + n], w.dtype, "cpu", pin=True)
        self.hbias = _to_torch(A["bias"][r0:r0 + n], w.dtype, "cpu", pin=True)
        self.hout = torch.zeros((n, S, C), dtype=tdt).pin_memory()
        self.xs = [torch.empty((n, S, C), dtype=tdt, device=device) for _ in range(2)]
        self.biases = [torch.empty((n, S), dtype=tdt, device=device) for _ in range(2)]
        self.x = self.xs[0]
        f = lambda a: _to_torch(a, w.dtype, device)
        f32 = lambda a: _to_torch(a, "fp32", device)
        self.wq, self.wk, self.wv, self.wg, self.wo = (f(A[k]) for k in ("wq", "wk", "wv", "wg", "wo"))
        self.bg, self.bo = f32(A["bg"]), f32(A["bo"])
        self.wb = f(np.ascontiguousarray(A["wb"].T))
        # [S, H, S] storage (see ShardedTriangleAttention): this rank's rows are one dense block, gathered in place
        self.nb_full = torch.zeros((S, H, S), dtype=tdt, device=device)
        self.weights = api.make_weights(C, H, w.D, self.wq, self.wk, self.wv, self.wg, self.bg, self.wo, self.bo)
        self.inputs = api.make_inputs(n, S)
        self.t_wb = api.tensor(self.wb)
        self.t_nb = api.Tensor(self.nb_full.data_ptr(), [H, S, S], [S, H * S, 1], dt, keep=self.nb_full)
        self.t_x = [api.tensor(x, sizes=[n * S, C], strides=[C, 1]) for x in self.xs]
        self.t_z = [api.tensor(x) for x in self.xs]
        self.t_bias = [api.tensor(b) for b in self.biases]
        self.t_out = api.tensor(self.hout)
        nb_rows = self.nb_full[r0:r0 + n]
        self.t_nb_rows = api.Tensor(nb_rows.data_ptr(), [H, n, S], [S, H * S, 1], dt, keep=self.nb_full)
        self.g_nb_src = api.Tensor(nb_rows.data_ptr(), [n, 1, H * S * esz], [H * S * esz, H * S * esz, 1], api.DTYPE_BF16,
                                   keep=self.nb_full)
        self.g_nb_dst = api.Tensor(self.nb_full.data_ptr(), [N, 1, H * S * esz], [H * S * esz, H * S * esz, 1],
                                   api.DTYPE_BF16, keep=self.nb_full)
        self.compute = torch.cuda.current_stream(device)
        self.comm = torch.cuda.Stream(device)
        self.bias_projected, self.bias_gathered = torch.cuda.Event(), torch.cuda.Event()
        self.upload = torch.cuda.Stream(device)
        self.uploaded = [torch.cuda.Event() for _ in range(2)]
        self.computed = [None, None]   # recorded after the kernels of the last step that read device buffer 0 / 1
        self.index = 0                 # number of the next step
        self.in_flight = -1            # step whose rows have been sent to the device (or are on their way)
        self.torch = torch

    def h2d_bytes(self) -> int:
        return int(self.hx.numel() * self.hx.element_size() + self.hbias.numel() * self.hbias.element_size())

    def d2h_bytes(self) -> int:
        return int(self.hout.numel() * self.hout.element_size())

    def _send(self, i: int):
        """Queue the upload of step i's rows on the upload stream, after the kernels of step i - 2 (the last reader
        of device buffer i % 2)."""
        j = i & 1
        if self.computed[j] is not None:
            self.upload.wait_event(self.computed[j])
        with self.torch.cuda.stream(self.upload):
            self.xs[j].copy_(self.hx, non_blocking=True)
            self.biases[j].copy_(self.hbias, non_blocking=True)
            self.uploaded[j].record(self.upload)
        self.in_flight = i

    def drain(self):
        """Wait (on the host) until every queued step has delivered its rows and no upload is in flight."""
        if self.in_flight >= 0:
            self.compute.wait_event(self.uploaded[self.in_flight & 1])
        self.api.set_stream(self.compute.cuda_stream)
        self.api.synchronize()

    def step(self, block_size: int = 128, prefetch: bool = True):
        """One step. With ``prefetch`` the call only queues work: the next step's rows start their way to the device
        and the output rows of this step are complete in ``hout`` after a later ``drain()`` (or after the next
        stand-alone step). Without it the step runs on its own and ``hout`` is complete on return."""
        api = self.api
        i, j = self.index, self.index & 1
        api.set_async(True)
        try:
            api.set_stream(self.compute.cuda_stream)
            if self.in_flight != i:
                self.upload.wait_stream(self.compute)
                self._send(i)
            self.compute.wait_event(self.uploaded[j])
            api.pair_bias(self.t_z[j], self.t_wb, self.t_nb_rows)
            if self.world > 1:
                # the gather runs on its own stream beside the projections of the attention call (see
                # ShardedTriangleAttention.step)
                self.bias_projected.record(self.compute)
                self.comm.wait_event(self.bias_projected)
                api.set_stream(self.comm.cuda_stream)
                api.all_gather(self.g_nb_src, self.g_nb_dst)
                self.bias_gathered.record(self.comm)
                api.set_stream(self.compute.cuda_stream)
                api.set_pair_bias_event(self.bias_gathered)
            if prefetch:
                self._send(i + 1)
            # enqueue-only: the library downloads the output rows chunk by chunk on its copy stream while the later
            # chunks (and, with prefetch, the first chunks of the next step) are computed
            api.gating_attention(self.t_x[j], self.inputs, self.t_bias[j], self.t_nb, self.weights, self.t_out, block_size)
            if self.computed[j] is None:
                self.computed[j] = self.torch.cuda.Event()
            self.computed[j].record(self.compute)
            if not prefetch:
                api.synchronize()
        finally:
            api.set_async(False)
        self.index = i + 1
        return self.hout
