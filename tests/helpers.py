"""Shared helpers for the parity tests: oracle calls on a Workload and the error metric."""
import numpy as np

from kutacc_b200 import workloads as W
from oracle import cpu_oracle as O

BF16_TOL = 1e-2   # relative max-abs error allowed against the faithful oracle (bf16 shapes)
FP32_TOL = 1e-4   # relative max-abs error allowed against the exact oracle (fp32 shapes)


def rel_err(y: np.ndarray, ref: np.ndarray) -> float:
    y = np.asarray(y, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(y - ref).max() / max(np.abs(ref).max(), 1e-30))


def oracle_faithful(w: W.Workload, block_size: int = 128) -> np.ndarray:
    A = w.arrays
    if w.kind == "gating":
        out = O.gating_attention_bf16(w.bits("x").reshape(-1, w.C), w.bits("wq"), w.bits("wk"), w.bits("wv"),
                                      w.bits("wg"), A["bg"], w.bits("wo"), A["bo"], w.bits("bias"),
                                      w.bits("nb") if w.has_nb else None, w.B, w.S, w.H, w.D, block_size=block_size)
    else:
        out = O.global_attention_bf16(w.bits("x"), w.bits("mask"), w.bits("wq"), w.bits("wk"), w.bits("wv"),
                                      w.bits("wg"), A["bg"], w.bits("wo"), A["bo"], w.B, w.S, w.H, w.D)
    return W.as_f32(out)


def oracle_exact(w: W.Workload) -> np.ndarray:
    A = w.arrays
    if w.kind == "gating":
        return O.gating_attention_exact(A["x"], A["wq"], A["wk"], A["wv"], A["wg"], A["bg"], A["wo"], A["bo"],
                                        A["bias"], A["nb"] if w.has_nb else None, w.B, w.S, w.H, w.D)
    return O.global_attention_exact(A["x"], A["mask"], A["wq"], A["wk"], A["wv"], A["wg"], A["bg"], A["wo"], A["bo"],
                                    w.B, w.S, w.H, w.D)
