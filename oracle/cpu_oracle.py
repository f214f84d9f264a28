"""ctypes front end of the CPU oracle (test infrastructure).

Arrays are numpy: bf16 data travels as uint16 bit patterns, fp32 as float32. Only tests, the
smoke check and the benchmark's CPU-baseline leg import this module.
"""
import ctypes as C
import os

import numpy as np

from . import build as _build

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = _build.LIB if os.path.exists(_build.LIB) else _build.build()
        _lib = C.CDLL(path)
        _lib.orc_fexpa_exp.restype = C.c_float
        _lib.orc_fexpa_exp.argtypes = [C.c_float]
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(C.c_int(int(n)))


def f32_to_bf16(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.empty(a.shape, dtype=np.uint16)
    lib().orc_f32_to_bf16(_p(a), _p(out), C.c_int64(a.size))
    return out


def bf16_to_f32(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint16)
    out = np.empty(a.shape, dtype=np.float32)
    lib().orc_bf16_to_f32(_p(a), _p(out), C.c_int64(a.size))
    return out


def fexpa_exp(x: float) -> float:
    return float(lib().orc_fexpa_exp(C.c_float(x)))


def gating_attention_bf16(x, wq, wk, wv, wg, bg, wo, bo, bias, nb, B, S, H, D, block_size=128, dumps=False):
    """Faithful mode. x [B*S,C] u16, w* [C,C] u16, bg/bo [C] f32, bias [B,S] u16, nb [H,S,S] u16 or None."""
    Cn = H * D
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty((B, S, Cn), dtype=np.uint16)
    bias = np.ascontiguousarray(bias, dtype=np.uint16)
    if nb is not None:
        nb = np.ascontiguousarray(nb, dtype=np.uint16)
    d = {}
    if dumps:
        for name in ("q", "k", "g", "avg"):
            d[name] = np.empty((B, S, H, D), dtype=np.uint16)
        d["v"] = np.empty((H, D, B, S), dtype=np.uint16)
    lib().orc_gating_attention_bf16(
        _p(x), _p(wq), _p(wk), _p(wv), _p(wg), _p(bg), _p(wo), _p(bo),
        _p(bias), C.c_int64(S), _p(nb), C.c_int64(S * S), C.c_int64(S),
        C.c_int64(B), C.c_int64(S), C.c_int64(H), C.c_int64(D), C.c_int64(block_size), _p(out),
        _p(d.get("q")), _p(d.get("k")), _p(d.get("v")), _p(d.get("g")), _p(d.get("avg")))
    return (out, d) if dumps else out


def gating_attention_exact(x, wq, wk, wv, wg, bg, wo, bo, bias, nb, B, S, H, D):
    """Exact mode: every array float32; double accumulation inside."""
    Cn = H * D
    f = lambda a: None if a is None else np.ascontiguousarray(a, dtype=np.float32)
    x, wq, wk, wv, wg, bg, wo, bo, bias, nb = map(f, (x, wq, wk, wv, wg, bg, wo, bo, bias, nb))
    out = np.empty((B, S, Cn), dtype=np.float32)
    lib().orc_gating_attention_exact(
        _p(x), _p(wq), _p(wk), _p(wv), _p(wg), _p(bg), _p(wo), _p(bo),
        _p(bias), C.c_int64(S), _p(nb), C.c_int64(S * S), C.c_int64(S),
        C.c_int64(B), C.c_int64(S), C.c_int64(H), C.c_int64(D), _p(out))
    return out


def global_attention_bf16(x, mask, wq, wk, wv, wg, bg, wo, bo, B, S, H, D):
    Cn = H * D
    out = np.empty((B, S, Cn), dtype=np.uint16)
    x = np.ascontiguousarray(x, dtype=np.uint16)
    mask = np.ascontiguousarray(mask, dtype=np.uint16)
    lib().orc_global_attention_bf16(_p(x), _p(mask), _p(wq), _p(wk), _p(wv), _p(wg), _p(bg), _p(wo), _p(bo),
                                    C.c_int64(B), C.c_int64(S), C.c_int64(H), C.c_int64(D), _p(out))
    return out


def global_attention_exact(x, mask, wq, wk, wv, wg, bg, wo, bo, B, S, H, D):
    Cn = H * D
    f = lambda a: np.ascontiguousarray(a, dtype=np.float32)
    x, mask, wq, wk, wv, wg, bg, wo, bo = map(f, (x, mask, wq, wk, wv, wg, bg, wo, bo))
    out = np.empty((B, S, Cn), dtype=np.float32)
    lib().orc_global_attention_exact(_p(x), _p(mask), _p(wq), _p(wk), _p(wv), _p(wg), _p(bg), _p(wo), _p(bo),
                                     C.c_int64(B), C.c_int64(S), C.c_int64(H), C.c_int64(D), _p(out))
    return out


def linear_bf16(act, w, bias, beta=0, result=None):
    """act [M,K] u16, w [N,K] u16, bias [N] f32 or None; returns [M,N] u16."""
    act = np.ascontiguousarray(act, dtype=np.uint16)
    w = np.ascontiguousarray(w, dtype=np.uint16)
    M, K = act.shape
    N = w.shape[0]
    res = np.zeros((M, N), dtype=np.uint16) if result is None else np.ascontiguousarray(result, dtype=np.uint16).copy()
    lib().orc_linear_bf16(_p(act), C.c_int64(K), _p(w), C.c_int64(K), _p(bias), C.c_int64(M), C.c_int64(N),
                          C.c_int64(K), C.c_int64(beta), _p(res))
    return res


def linear_exact(act, w, bias, beta=0, result=None):
    act = np.ascontiguousarray(act, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    M, K = act.shape
    N = w.shape[0]
    res = np.zeros((M, N), dtype=np.float32) if result is None else np.ascontiguousarray(result, dtype=np.float32).copy()
    lib().orc_linear_exact(_p(act), C.c_int64(K), _p(w), C.c_int64(K), _p(bias), C.c_int64(M), C.c_int64(N),
                           C.c_int64(K), C.c_int64(beta), _p(res))
    return res


def transition_bf16(x, w1, b1, w2, b2):
    """Transition MLP as src/attention/transition.cpp:31-38 runs it: two addmm calls with a row bias, the first
    with ReLU, the intermediate stored as bf16. x [M, c_o] u16, w1 [c_i, c_o] u16, w2 [c_o, c_i] u16, biases f32.
    (Where the closed GEMM applies the ReLU relative to its bf16 rounding cannot be seen; the two orders agree.)"""
    hid = linear_bf16(x, w1, b1)
    hid = np.where(hid & 0x8000, np.uint16(0), hid).astype(np.uint16)       # relu on bf16 bits (-0 -> +0)
    return linear_bf16(hid, w2, b2)


def transition_exact(x, w1, b1, w2, b2):
    hid = np.maximum(linear_exact(x, w1, b1), 0.0).astype(np.float32)
    return linear_exact(hid, w2, b2)


def tm_calc_proj_bf16(x, mask, pw, pb, gw, gb):
    """Triangle multiplication, projection step (src/attention/triangle_multiplication.cpp:25-70).
    x [n_res, n_gather, c_o] u16, mask [n_res, n_gather] u16, pw/gw [c_i, c_o] u16, pb/gb [c_i] f32.
    Returns (proj, gate), both [c_i, n_res, n_gather] u16: proj already multiplied by mask and sigmoid(gate)."""
    x = np.ascontiguousarray(x, dtype=np.uint16)
    n_res, n_gather, c_o = x.shape
    c_i = pw.shape[0]
    f16 = lambda a: np.ascontiguousarray(a, dtype=np.uint16)
    f32 = lambda a: np.ascontiguousarray(a, dtype=np.float32)
    mask, pw, gw, pb, gb = f16(mask), f16(pw), f16(gw), f32(pb), f32(gb)
    proj = np.empty((c_i, n_res, n_gather), dtype=np.uint16)
    gate = np.empty((c_i, n_res, n_gather), dtype=np.uint16)
    lib().orc_tm_calc_proj_bf16(_p(x), _p(mask), _p(pw), _p(pb), _p(gw), _p(gb), C.c_int64(n_res), C.c_int64(n_gather),
                                C.c_int64(c_o), C.c_int64(c_i), _p(proj), _p(gate))
    return proj, gate


def tm_calc_proj_exact(x, mask, pw, pb, gw, gb):
    f32 = lambda a: np.ascontiguousarray(a, dtype=np.float32)
    x, mask, pw, pb, gw, gb = map(f32, (x, mask, pw, pb, gw, gb))
    n_res, n_gather, c_o = x.shape
    c_i = pw.shape[0]
    proj = np.empty((c_i, n_res, n_gather), dtype=np.float32)
    lib().orc_tm_calc_proj_exact(_p(x), _p(mask), _p(pw), _p(pb), _p(gw), _p(gb), C.c_int64(n_res), C.c_int64(n_gather),
                                 C.c_int64(c_o), C.c_int64(c_i), _p(proj))
    return proj


def tm_equation_bf16(left, right, incoming):
    """center[ch] = left[ch] . right[ch]^T (outgoing) or right[ch]^T . left[ch] (incoming), per channel
    (triangle_multiplication.cpp:75-104). left, right [c_i, n, n] u16 -> [c_i, n, n] u16."""
    left = np.ascontiguousarray(left, dtype=np.uint16)
    right = np.ascontiguousarray(right, dtype=np.uint16)
    c_i, n, _ = left.shape
    center = np.empty((c_i, n, n), dtype=np.uint16)
    lib().orc_tm_equation_bf16(_p(left), _p(right), C.c_int64(c_i), C.c_int64(n), C.c_int(1 if incoming else 0), _p(center))
    return center


def tm_equation_exact(left, right, incoming):
    left = np.ascontiguousarray(left, dtype=np.float32)
    right = np.ascontiguousarray(right, dtype=np.float32)
    c_i, n, _ = left.shape
    center = np.empty((c_i, n, n), dtype=np.float32)
    lib().orc_tm_equation_exact(_p(left), _p(right), C.c_int64(c_i), C.c_int64(n), C.c_int(1 if incoming else 0), _p(center))
    return center


def tm_last_bf16(out, gate):
    """out = bf16(f32(out) * sigmoid(f32(gate))) element by element (triangle_multiplication.cpp:138-158)."""
    res = np.ascontiguousarray(out, dtype=np.uint16).copy()
    gate = np.ascontiguousarray(gate, dtype=np.uint16)
    lib().orc_tm_last_bf16(_p(res), _p(gate), C.c_int64(res.size))
    return res


def transpose_bytes(shards, m, n):
    """shards[r]: uint8 [chunk_r(m), n, len] (rows split over the ranks) -> list of uint8 [m, chunk_r(n), len]."""
    world = len(shards)
    ln = shards[0].shape[2]
    bn = (n + world - 1) // world
    shards = [np.ascontiguousarray(s_, dtype=np.uint8) for s_ in shards]
    outs = [np.zeros((m, max(0, min(bn, n - r * bn)), ln), dtype=np.uint8) for r in range(world)]
    keep = [o if o.size else np.zeros(1, dtype=np.uint8) for o in outs]
    src = (C.c_void_p * world)(*[s_.ctypes.data if s_.size else 0 for s_ in shards])
    dst = (C.c_void_p * world)(*[o.ctypes.data for o in keep])
    lib().orc_transpose_bytes(src, dst, C.c_int64(world), C.c_int64(m), C.c_int64(n), C.c_int64(ln))
    return outs


def layernorm_bf16(x, gamma, beta, eps):
    """x [rows, size] u16 (bf16 bits), gamma/beta [size] f32; returns [rows, size] u16."""
    x = np.ascontiguousarray(x, dtype=np.uint16)
    gamma = np.ascontiguousarray(gamma, dtype=np.float32)
    beta = np.ascontiguousarray(beta, dtype=np.float32)
    rows, size = x.shape
    out = np.empty_like(x)
    lib().orc_layernorm_bf16(_p(x), _p(gamma), _p(beta), C.c_int64(rows), C.c_int64(size), C.c_float(eps), _p(out))
    return out


def layernorm_exact(x, gamma, beta, eps):
    x = np.ascontiguousarray(x, dtype=np.float32)
    gamma = np.ascontiguousarray(gamma, dtype=np.float32)
    beta = np.ascontiguousarray(beta, dtype=np.float32)
    rows, size = x.shape
    out = np.empty_like(x)
    lib().orc_layernorm_exact(_p(x), _p(gamma), _p(beta), C.c_int64(rows), C.c_int64(size), C.c_float(eps), _p(out))
    return out


def all_gather_bytes(shards, out_shape, data_size0):
    """shards: list of contiguous uint8 arrays [a,b,len] (one per rank); returns gathered [m,n,len]."""
    world = len(shards)
    m, n, ln = out_shape
    out = np.zeros((m, n, ln), dtype=np.uint8)
    shards = [np.ascontiguousarray(s, dtype=np.uint8) for s in shards]
    ptrs = (C.c_void_p * world)(*[s.ctypes.data for s in shards])
    ds0 = (C.c_int64 * world)(*[s.shape[1] * ln for s in shards])
    ds1 = ln
    lib().orc_all_gather_bytes(ptrs, C.c_int64(world), C.c_int64(data_size0), ds0, C.c_int64(ds1),
                               _p(out), C.c_int64(m), C.c_int64(n), C.c_int64(ln), C.c_int64(n * ln), C.c_int64(ln))
    return out
