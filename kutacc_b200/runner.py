"""Run a :class:`~kutacc_b200.workloads.Workload` through libkutacc.so.

``DeviceCase`` keeps every tensor resident on the GPU (kernel-only timing, parity tests);
``HostCase`` keeps them in pinned host memory so that each call pays the host<->device copies
inside the library, which is what a caller of the CPU reference would see.
"""
from __future__ import annotations

import numpy as np
import torch

from . import api
from .workloads import Workload, bf16_bits


def _to_torch(arr: np.ndarray, dtype: str, device, pin: bool = False) -> torch.Tensor:
    if dtype == "bf16":
        t = torch.from_numpy(bf16_bits(arr).view(np.int16)).view(torch.bfloat16)
    else:
        t = torch.from_numpy(np.ascontiguousarray(arr, dtype=np.float32))
    if device == "cpu":
        return t.pin_memory() if pin else t
    return t.to(device)


def out_to_f32(t: torch.Tensor) -> np.ndarray:
    return t.detach().to("cpu", torch.float32).numpy()


class _Case:
    def __init__(self, w: Workload, device, pin: bool):
        self.w = w
        self.device = device
        A = w.arrays
        f = lambda key: _to_torch(A[key], w.dtype, device, pin)
        f32 = lambda key: _to_torch(A[key], "fp32", device, pin)
        self.x = f("x")
        self.wq, self.wk, self.wv, self.wg, self.wo = f("wq"), f("wk"), f("wv"), f("wg"), f("wo")
        self.bg, self.bo = f32("bg"), f32("bo")
        self.out = torch.empty((w.B, w.S, w.C), dtype=self.x.dtype, device=device)
        if pin and device == "cpu":
            self.out = self.out.pin_memory()
        dt = api.DTYPE_BF16 if w.dtype == "bf16" else api.DTYPE_FP32
        self.weights = api.make_weights(w.C, w.H, w.D, self.wq, self.wk, self.wv, self.wg, self.bg, self.wo, self.bo)
        self.inputs = api.make_inputs(w.B, w.S)
        self.t_out = api.tensor(self.out)
        if w.kind == "gating":
            self.bias = f("bias")
            self.nb = f("nb") if w.has_nb else None
            self.t_x = api.tensor(self.x, sizes=[w.B * w.S, w.C], strides=[w.C, 1])
            self.t_bias = api.tensor(self.bias)
            self.t_nb = api.tensor(self.nb) if self.nb is not None else api.empty_tensor(dt)
        else:
            self.mask = f("mask")
            self.t_x = api.tensor(self.x)
            self.t_mask = api.tensor(self.mask, sizes=[w.B, w.S, 1], strides=[w.S, 1, 1])

    def h2d_bytes(self) -> int:
        ts = [self.x, self.wq, self.wk, self.wv, self.wg, self.wo, self.bg, self.bo]
        ts += [self.bias] if self.w.kind == "gating" else [self.mask]
        if getattr(self, "nb", None) is not None:
            ts.append(self.nb)
        return int(sum(t.numel() * t.element_size() for t in ts))

    def d2h_bytes(self) -> int:
        return int(self.out.numel() * self.out.element_size())

    def run(self, block_size: int = 128) -> torch.Tensor:
        if self.w.kind == "gating":
            api.gating_attention(self.t_x, self.inputs, self.t_bias, self.t_nb, self.weights, self.t_out, block_size)
        else:
            api.global_attention(self.inputs, self.t_x, self.t_mask, self.weights, self.t_out)
        return self.out


class DeviceCase(_Case):
    def __init__(self, w: Workload, device="cuda:0"):
        super().__init__(w, device, pin=False)


class HostCase(_Case):
    def __init__(self, w: Workload):
        super().__init__(w, "cpu", pin=True)
