"""Seeded synthetic inputs for the five benchmark shapes of the gated-attention path.

The shapes are AlphaFold2 model dimensions; no dataset is involved. Every array is drawn with
``numpy.random.default_rng(seed)`` in a fixed order (activations, pair activations, Wq, Wk, Wv, Wg,
Wo, Wb, mask) in fp32, weights scaled by 1/sqrt(fan_in); for the bf16 shapes each array is rounded
to bf16 once, so the CPU oracle and the GPU library consume the same bits.

bf16 arrays are carried as ``uint16`` bit patterns (``*_bits``); ``as_f32`` widens them.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional

import numpy as np


def bf16_bits(a: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit pattern, round to nearest even (NaN kept quiet)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32)
    r = u >> 16                       # in-place uint32 arithmetic: the only bit patterns whose rounding sum would
    r &= 1                            # wrap are negative NaNs, and NaNs are patched below
    r += 0x7FFF
    r += u
    r >>= 16
    r = r.astype(np.uint16)
    nan = np.isnan(a)
    if nan.any():
        r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r


def as_f32(bits: np.ndarray) -> np.ndarray:
    """bf16 bit pattern -> fp32 (exact)."""
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


@dataclass
class Workload:
    name: str
    kind: str            # "gating" | "global"
    dtype: str           # "bf16" | "fp32"
    B: int
    S: int
    H: int
    D: int
    seed: int
    arrays: Dict[str, np.ndarray] = field(default_factory=dict)   # fp32 values (already bf16-representable for bf16)
    has_nb: bool = False
    c_z: int = 0          # channels of the pair activations the pair bias was projected from (0 = none)

    @property
    def C(self) -> int:
        return self.H * self.D

    def bits(self, key: str) -> np.ndarray:
        return bf16_bits(self.arrays[key])

    # ---- algorithmic work (2 FLOPs per multiply-add; exp/softmax/sigmoid not counted) ----
    def flops(self, rows: Optional[int] = None, pair_bias: bool = True) -> float:
        """``pair_bias=False`` leaves out the projection of the pair bias from z (callers that are handed the
        projected bias as an input do not run it)."""
        B = self.B if rows is None else rows
        S, C, H, D = self.S, self.C, self.H, self.D
        if self.kind == "gating":
            f = 10.0 * B * S * C * C + 4.0 * B * S * S * C
            if pair_bias and self.c_z and (self.has_nb or "wb" in self.arrays):
                f += 2.0 * S * S * self.c_z * H
            return f
        # global: pool, q, k, v, gate, logits, PV, out
        return (2.0 * B * S * C + 2.0 * B * C * C + 4.0 * B * S * C * D + 2.0 * B * S * C * C
                + 4.0 * B * S * H * D + 2.0 * B * S * C * C)

    # ---- compulsory HBM bytes: input once, output once, weights, mask, pair bias once ----
    def bytes(self, rows: Optional[int] = None) -> float:
        B = self.B if rows is None else rows
        e = 2 if self.dtype == "bf16" else 4
        S, C, H = self.S, self.C, self.H
        n = 2.0 * B * S * C * e                      # x in, out
        n += 5.0 * C * C * e + 2.0 * C * 4            # weights, biases
        n += B * S * e                                # mask bias
        if self.has_nb:
            n += H * S * S * e
        return n


_SPECS = {
    # name: (kind, dtype, B, S, H, D, c_z, seed)
    "msa_row_fp32": ("gating", "fp32", 128, 256, 8, 32, 128, 0),
    "triangle_start_384": ("gating", "bf16", 384, 384, 4, 32, 128, 1),
    "msa_col_512": ("gating", "bf16", 384, 512, 8, 32, 0, 2),
    "extra_msa_global": ("global", "bf16", 384, 5120, 8, 8, 0, 3),
    "triangle_end_1024": ("gating", "bf16", 1024, 1024, 4, 32, 128, 4),
}
NAMES = list(_SPECS)


def spec(name: str):
    return _SPECS[name]


def make(name: str, rows: Optional[int] = None, seq: Optional[int] = None, with_nb: bool = True) -> Workload:
    """Build a workload. ``rows`` keeps only the first ``rows`` batch rows (cheap sub-sample with the
    same per-row distribution); ``seq`` overrides the sequence length (tests on reduced shapes);
    ``with_nb=False`` leaves out the projected pair bias ``nb`` (callers that project it themselves from
    ``z`` and ``wb``, as the sharded flow does, save the host-side product)."""
    kind, dtype, B, S, H, D, c_z, seed = _SPECS[name]
    if seq is not None:
        S = int(seq)
    Bgen = B if rows is None else min(B, int(rows))
    C = H * D
    rng = np.random.default_rng(seed)
    rnd = (lambda a: as_f32(bf16_bits(a))) if dtype == "bf16" else (lambda a: np.ascontiguousarray(a, np.float32))
    w = Workload(name=name, kind=kind, dtype=dtype, B=Bgen, S=S, H=H, D=D, seed=seed, c_z=c_z)
    A = w.arrays

    x = rng.standard_normal((Bgen, S, C), dtype=np.float32)
    pair_input = name in ("triangle_start_384", "triangle_end_1024")
    if not pair_input:
        # consume the draws of the rows that were left out, so that every later array (weights, mask)
        # is the same whatever `rows` is
        left = (B - Bgen) * S * C
        while left > 0:
            n = min(left, 1 << 24)
            rng.standard_normal(n, dtype=np.float32)
            left -= n
    if pair_input:
        # the activations are the pair representation itself: x[i, j, :] = z[i, j, :]; the pair bias
        # of query row q and key k is z[q, k, :] . Wb, so z needs all S rows even when rows < S
        zfull = x if Bgen == S else np.concatenate(
            [x, rng.standard_normal((S - Bgen, S, C), dtype=np.float32)], axis=0)
        z = zfull
    elif c_z:
        z = rng.standard_normal((S, S, c_z), dtype=np.float32)
    else:
        z = None
    A["x"] = rnd(x)
    if kind == "gating":
        for key in ("wq", "wk", "wv", "wg", "wo"):
            A[key] = rnd(rng.standard_normal((C, C), dtype=np.float32) / np.sqrt(C))
    else:
        A["wq"] = rnd(rng.standard_normal((C, C), dtype=np.float32) / np.sqrt(C))
        A["wk"] = rnd(rng.standard_normal((D, C), dtype=np.float32) / np.sqrt(C))
        A["wv"] = rnd(rng.standard_normal((D, C), dtype=np.float32) / np.sqrt(C))
        A["wg"] = rnd(rng.standard_normal((C, C), dtype=np.float32) / np.sqrt(C))
        A["wo"] = rnd(rng.standard_normal((C, C), dtype=np.float32) / np.sqrt(C))
    A["bg"] = np.ones((C,), dtype=np.float32)
    A["bo"] = np.zeros((C,), dtype=np.float32)
    if z is not None:
        zc = z.shape[-1]
        wb = rnd(rng.standard_normal((zc, H), dtype=np.float32) / np.sqrt(zc))
        A["wb"] = wb
        zr = A["x"] if (pair_input and Bgen == S) else rnd(z)
        A["z"] = zr
        if with_nb:
            nb = (zr.reshape(S * S, zc).astype(np.float32) @ wb).reshape(S, S, H)
            A["nb"] = rnd(np.ascontiguousarray(nb.transpose(2, 0, 1)))      # [H, S_q, S_k]
            w.has_nb = True

    # masks
    if name == "msa_row_fp32" or name == "triangle_end_1024":
        mask = np.ones((Bgen, S), dtype=np.float32)
    elif name == "triangle_start_384":
        keep = (rng.random(S) >= 0.05).astype(np.float32)
        mask = (keep[:, None] * keep[None, :])[:Bgen]                    # 5 % of rows fully masked
    elif name == "msa_col_512":
        keep = (rng.random(S) >= 0.10).astype(np.float32)
        mask = np.broadcast_to(keep[None, :], (Bgen, S)).copy()
    else:  # extra_msa_global: trailing 20 % of the rows are padding
        mask = np.ones((Bgen, S), dtype=np.float32)
        mask[:, int(S * 0.8):] = 0.0
    A["mask"] = mask
    if kind == "gating":
        A["bias"] = rnd(1e9 * (mask - 1.0))
    return w


def random_gating_case(seed: int, B: int, S: int, H: int, D: int, dtype: str = "bf16", with_nb: bool = True,
                       mask_frac: float = 0.2, full_mask_rows: int = 0) -> Workload:
    """Small randomised case for unit tests: non-zero biases, random mask, optional pair bias."""
    rng = np.random.default_rng(seed)
    C = H * D
    rnd = (lambda a: as_f32(bf16_bits(a))) if dtype == "bf16" else (lambda a: np.ascontiguousarray(a, np.float32))
    w = Workload(name=f"rand{seed}", kind="gating", dtype=dtype, B=B, S=S, H=H, D=D, seed=seed)
    A = w.arrays
    A["x"] = rnd(rng.standard_normal((B, S, C), dtype=np.float32))
    for key in ("wq", "wk", "wv", "wg", "wo"):
        A[key] = rnd(rng.standard_normal((C, C), dtype=np.float32) / np.sqrt(C))
    A["bg"] = rng.standard_normal(C).astype(np.float32)
    A["bo"] = rng.standard_normal(C).astype(np.float32)
    mask = (rng.random((B, S)) >= mask_frac).astype(np.float32)
    mask[:, 0] = 1.0
    for r in range(min(full_mask_rows, B)):
        mask[r, :] = 0.0
    A["mask"] = mask
    A["bias"] = rnd(1e9 * (mask - 1.0))
    if with_nb:
        A["nb"] = rnd(rng.standard_normal((H, S, S), dtype=np.float32))
        w.has_nb = True
    return w


def random_global_case(seed: int, B: int, S: int, H: int = 8, D: int = 8, zero_mask_rows: int = 0) -> Workload:
    rng = np.random.default_rng(seed)
    C = H * D
    rnd = lambda a: as_f32(bf16_bits(a))
    w = Workload(name=f"grand{seed}", kind="global", dtype="bf16", B=B, S=S, H=H, D=D, seed=seed)
    A = w.arrays
    A["x"] = rnd(rng.standard_normal((B, S, C), dtype=np.float32))
    A["wq"] = rnd(rng.standard_normal((C, C), dtype=np.float32) / np.sqrt(C))
    A["wk"] = rnd(rng.standard_normal((D, C), dtype=np.float32) / np.sqrt(C))
    A["wv"] = rnd(rng.standard_normal((D, C), dtype=np.float32) / np.sqrt(C))
    A["wg"] = rnd(rng.standard_normal((C, C), dtype=np.float32) / np.sqrt(C))
    A["wo"] = rnd(rng.standard_normal((C, C), dtype=np.float32) / np.sqrt(C))
    A["bg"] = rng.standard_normal(C).astype(np.float32)
    A["bo"] = rng.standard_normal(C).astype(np.float32)
    mask = (rng.random((B, S)) >= 0.25).astype(np.float32)
    for r in range(min(zero_mask_rows, B)):
        mask[r, :] = 0.0
    A["mask"] = mask
    return w
