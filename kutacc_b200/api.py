"""Python front end of libkutacc.so: the reference's operator interface, bound with ctypes.

The function names, argument order and meaning follow the reference's public header
(include/kutacc.h:77-104, 297-307, 399-418): ``gating_attention(input, q_based, bias,
nonbatched_bias, weights, out, block_size)`` and so on. Tensors are passed as descriptors made by
:func:`tensor` from a torch tensor (CUDA or CPU), a numpy array, or a raw pointer.

There is no CPU implementation behind this module. If the shared library is missing the import
of any operator raises; build it with ``python -m kutacc_b200.build``.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("KUTACC_B200_LIB") or os.path.join(_HERE, "libkutacc.so")

DTYPE_INT64, DTYPE_BF16, DTYPE_FP32 = 0, 1, 2

EXPORTS = [
    # part 1: the reference's interface for this path
    "kutacc_get_version", "kutacc_comm_init", "kutacc_comm_fini", "kutacc_af2_all_gather", "kutacc_af2_transpose",
    "kutacc_af2_gating_attention", "kutacc_af2_global_attention", "kutacc_af2_linear",
    "kutacc_af2_linear_weight_prepack", "kutacc_af2_gemm_pack_get_size", "kutacc_af2_layernorm", "kutacc_af2_transition",
    "kutacc_af2_triangle_multiplication_calc_proj", "kutacc_af2_triangle_multiplication_equation",
    "kutacc_af2_triangle_multiplication_gate_and_out_linear", "kutacc_af2_triangle_multiplication_last",
    # part 2: additions
    "kutacc_b200_tensor_create", "kutacc_b200_tensor_destroy", "kutacc_b200_error_set", "kutacc_b200_last_error",
    "kutacc_b200_clear_error", "kutacc_b200_set_stream", "kutacc_b200_set_async", "kutacc_b200_set_sm_margin", "kutacc_b200_set_pair_bias_event", "kutacc_b200_synchronize",
    "kutacc_b200_device_malloc", "kutacc_b200_device_free", "kutacc_b200_memcpy_h2d", "kutacc_b200_memcpy_d2h",
    "kutacc_b200_workspace_bytes", "kutacc_b200_release_workspace", "kutacc_b200_launch_count",
    "kutacc_b200_set_profile", "kutacc_b200_profile_read", "kutacc_b200_comm_unique_id", "kutacc_b200_comm_init_with_id", "kutacc_b200_pair_bias",
    "kutacc_b200_global_attention_noalloc", "kutacc_b200_layernorm_rows", "kutacc_b200_selftest_wait_timeout",
    "kutacc_b200_gating_attention_ln", "kutacc_b200_pair_bias_ln",
]
EXPORTED_DATA = ["world_size", "rank"]


class KutaccError(RuntimeError):
    pass


class Version(C.Structure):
    _fields_ = [(n, C.c_char_p) for n in ("product_name", "product_version", "component_name", "component_version",
                                          "component_abi_version", "component_appendinfo")]


class AttentionWeights(C.Structure):
    """kutacc_af2_attention_weights_t (include/kutacc.h:77-89)."""
    _fields_ = [("nchannels", C.c_int64), ("nheads", C.c_int64), ("head_size", C.c_int64),
                ("query_w", C.c_void_p), ("key_w", C.c_void_p), ("value_w", C.c_void_p), ("gating_w", C.c_void_p),
                ("gating_b", C.c_void_p), ("output_w", C.c_void_p), ("output_b", C.c_void_p)]


class TransWeights(C.Structure):
    _fields_ = [("c_o", C.c_int64), ("c_i", C.c_int64), ("linear1_w", C.c_void_p), ("linear1_b", C.c_void_p),
                ("linear2_w", C.c_void_p), ("linear2_b", C.c_void_p)]


class TransInputs(C.Structure):
    _fields_ = [("batch", C.c_int64), ("n_res", C.c_int64), ("input_act", C.c_void_p), ("intermediate_act", C.c_void_p)]


class TmProjWeights(C.Structure):
    """kutacc_af2_tm_proj_weights_t (include/kutacc.h:154-162)."""
    _fields_ = [("c_o", C.c_int64), ("c_i", C.c_int64), ("proj_w", C.c_void_p), ("proj_b", C.c_void_p),
                ("gate_w", C.c_void_p), ("gate_b", C.c_void_p)]


class TmActInputs(C.Structure):
    """kutacc_af2_tm_act_inputs_t (include/kutacc.h:168-175)."""
    _fields_ = [("n_res", C.c_int64), ("n_res_gather", C.c_int64), ("proj_act", C.c_void_p), ("input_act", C.c_void_p),
                ("proj_act_gate", C.c_void_p)]


class TmLinearWeights(C.Structure):
    """kutacc_af2_tm_linear_weights_t (include/kutacc.h:181-189)."""
    _fields_ = [("c_o", C.c_int64), ("c_i", C.c_int64), ("gating_w", C.c_void_p), ("gating_b", C.c_void_p),
                ("output_proj_w", C.c_void_p), ("output_proj_b", C.c_void_p)]


class AttentionInputs(C.Structure):
    """kutacc_af2_attention_inputs_t (include/kutacc.h:95-104)."""
    _fields_ = [("batch", C.c_int64), ("seq_len", C.c_int64), ("q", C.c_void_p), ("k", C.c_void_p),
                ("v", C.c_void_p), ("gate", C.c_void_p), ("avg", C.c_void_p)]


_lib = None


def lib() -> C.CDLL:
    """Load libkutacc.so; raise if it has not been built. No fallback exists."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise KutaccError(f"{LIB_PATH} is missing: run `python -m kutacc_b200.build` (needs nvcc)")
    L = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
    vp, i64 = C.c_void_p, C.c_int64
    L.kutacc_get_version.restype = C.c_int
    L.kutacc_get_version.argtypes = [C.POINTER(Version)]
    L.kutacc_comm_init.argtypes = [i64, i64, i64]
    L.kutacc_comm_init.restype = None
    L.kutacc_comm_fini.restype = None
    L.kutacc_af2_all_gather.argtypes = [vp, vp]
    L.kutacc_af2_all_gather.restype = None
    L.kutacc_af2_transpose.argtypes = [vp, vp]
    L.kutacc_af2_transpose.restype = None
    L.kutacc_af2_gating_attention.argtypes = [vp, C.POINTER(AttentionInputs), vp, vp, C.POINTER(AttentionWeights), vp, i64]
    L.kutacc_af2_gating_attention.restype = None
    L.kutacc_af2_global_attention.argtypes = [C.POINTER(AttentionInputs), vp, vp, C.POINTER(AttentionWeights), vp]
    L.kutacc_af2_global_attention.restype = None
    L.kutacc_af2_linear.argtypes = [vp, vp, vp, vp, i64]
    L.kutacc_af2_linear.restype = None
    L.kutacc_af2_linear_weight_prepack.argtypes = [vp, vp, i64, i64, i64, i64]
    L.kutacc_af2_linear_weight_prepack.restype = None
    L.kutacc_af2_gemm_pack_get_size.argtypes = [C.c_char, C.c_char, C.c_char, C.c_int, C.c_int, C.c_int]
    L.kutacc_af2_gemm_pack_get_size.restype = C.c_size_t
    if hasattr(L, "kutacc_af2_triangle_multiplication_calc_proj"):
        L.kutacc_af2_triangle_multiplication_calc_proj.argtypes = [C.POINTER(TmActInputs), vp, C.POINTER(TmProjWeights), C.c_bool]
        L.kutacc_af2_triangle_multiplication_calc_proj.restype = None
        L.kutacc_af2_triangle_multiplication_equation.argtypes = [vp, vp, vp, i64, C.c_bool]
        L.kutacc_af2_triangle_multiplication_equation.restype = None
        L.kutacc_af2_triangle_multiplication_gate_and_out_linear.argtypes = [vp, vp, C.POINTER(TmActInputs), vp,
                                                                             C.POINTER(TmLinearWeights), C.c_bool]
        L.kutacc_af2_triangle_multiplication_gate_and_out_linear.restype = None
        L.kutacc_af2_triangle_multiplication_last.argtypes = [vp, vp, i64, i64, i64]
        L.kutacc_af2_triangle_multiplication_last.restype = None
    if hasattr(L, "kutacc_b200_gating_attention_ln"):
        L.kutacc_b200_gating_attention_ln.argtypes = [vp, C.POINTER(AttentionInputs), vp, vp, C.POINTER(AttentionWeights), vp, vp,
                                                      C.c_float, vp, i64]
        L.kutacc_b200_gating_attention_ln.restype = None
        L.kutacc_b200_pair_bias_ln.argtypes = [vp, vp, vp, C.c_float, vp, vp]
        L.kutacc_b200_pair_bias_ln.restype = None
    L.kutacc_b200_tensor_create.argtypes = [vp, i64, C.POINTER(i64), C.POINTER(i64), C.c_int]
    L.kutacc_b200_tensor_create.restype = vp
    L.kutacc_b200_tensor_destroy.argtypes = [vp]
    L.kutacc_b200_tensor_destroy.restype = None
    L.kutacc_b200_error_set.restype = C.c_int
    L.kutacc_b200_last_error.argtypes = [C.c_char_p, C.c_size_t]
    L.kutacc_b200_last_error.restype = C.c_int
    L.kutacc_b200_clear_error.restype = None
    L.kutacc_b200_set_stream.argtypes = [vp]
    L.kutacc_b200_set_stream.restype = None
    L.kutacc_b200_set_async.argtypes = [C.c_int]
    L.kutacc_b200_set_async.restype = None
    L.kutacc_b200_set_sm_margin.argtypes = [C.c_int]
    L.kutacc_b200_set_sm_margin.restype = None
    L.kutacc_b200_set_pair_bias_event.argtypes = [C.c_void_p]
    L.kutacc_b200_set_pair_bias_event.restype = None
    L.kutacc_b200_synchronize.restype = None
    L.kutacc_b200_device_malloc.argtypes = [C.c_size_t]
    L.kutacc_b200_device_malloc.restype = vp
    L.kutacc_b200_device_free.argtypes = [vp]
    L.kutacc_b200_device_free.restype = None
    L.kutacc_b200_memcpy_h2d.argtypes = [vp, vp, C.c_size_t]
    L.kutacc_b200_memcpy_h2d.restype = None
    L.kutacc_b200_memcpy_d2h.argtypes = [vp, vp, C.c_size_t]
    L.kutacc_b200_memcpy_d2h.restype = None
    L.kutacc_b200_workspace_bytes.restype = C.c_size_t
    L.kutacc_b200_release_workspace.restype = None
    L.kutacc_b200_launch_count.restype = C.c_uint64
    L.kutacc_b200_set_profile.argtypes = [C.c_int]
    L.kutacc_b200_set_profile.restype = None
    L.kutacc_b200_profile_read.argtypes = [C.c_char_p, C.c_size_t, C.POINTER(C.c_float), C.c_int]
    L.kutacc_b200_profile_read.restype = C.c_int
    L.kutacc_b200_comm_unique_id.argtypes = [vp]
    L.kutacc_b200_comm_unique_id.restype = None
    L.kutacc_b200_comm_init_with_id.argtypes = [i64, i64, vp]
    L.kutacc_b200_comm_init_with_id.restype = None
    L.kutacc_b200_global_attention_noalloc.argtypes = [vp] * 10 + [i64] * 5 + [vp]
    L.kutacc_b200_global_attention_noalloc.restype = C.c_int
    L.kutacc_b200_pair_bias.argtypes = [vp, vp, vp]
    L.kutacc_b200_pair_bias.restype = None
    L.kutacc_b200_selftest_wait_timeout.argtypes = [C.c_int64]
    L.kutacc_b200_selftest_wait_timeout.restype = C.c_int
    L.kutacc_af2_transition.argtypes = [C.POINTER(TransInputs), C.POINTER(TransWeights), vp]
    L.kutacc_af2_transition.restype = None
    L.kutacc_af2_layernorm.argtypes = [vp, vp, vp, C.c_int64, C.c_float, vp]
    L.kutacc_af2_layernorm.restype = None
    L.kutacc_b200_layernorm_rows.argtypes = [vp, vp, vp, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_float, vp]
    L.kutacc_b200_layernorm_rows.restype = None
    _lib = L
    return L


# ---- error convention ---------------------------------------------------------------------------
def error_set() -> bool:
    return bool(lib().kutacc_b200_error_set())


def last_error() -> str:
    buf = C.create_string_buffer(1024)
    lib().kutacc_b200_last_error(buf, 1024)
    return buf.value.decode(errors="replace")


def clear_error() -> None:
    lib().kutacc_b200_clear_error()


def raise_if_error() -> None:
    """Turn the library's sticky error flag into an exception (and clear it)."""
    if error_set():
        msg = last_error()
        clear_error()
        raise KutaccError(msg)


def version() -> dict:
    v = Version()
    rc = lib().kutacc_get_version(C.byref(v))
    if rc != 0:
        raise KutaccError("kutacc_get_version failed")
    return {n: getattr(v, n).decode() for n, _ in Version._fields_}


def launch_count() -> int:
    return int(lib().kutacc_b200_launch_count())


def set_profile(enabled: bool) -> None:
    lib().kutacc_b200_set_profile(1 if enabled else 0)


def profile_read(cap: int = 4096):
    """[(kernel name, ms), ...] of the launches recorded since the last read, in launch order."""
    names = C.create_string_buffer(cap * 24)
    ms = (C.c_float * cap)()
    n = lib().kutacc_b200_profile_read(names, len(names), ms, cap)
    nm = names.value.decode().split(";")[:n]
    return list(zip(nm, [float(ms[i]) for i in range(n)]))


def set_stream(stream_ptr: int) -> None:
    lib().kutacc_b200_set_stream(C.c_void_p(stream_ptr))


def set_async(enabled: bool) -> None:
    lib().kutacc_b200_set_async(1 if enabled else 0)


def set_sm_margin(sms: int) -> None:
    lib().kutacc_b200_set_sm_margin(int(sms))


def set_pair_bias_event(event) -> None:
    """The next gated-attention call waits for `event` (a torch.cuda.Event recorded on the stream that still
    produces its pair bias, or None) between its projections and its attention kernel."""
    lib().kutacc_b200_set_pair_bias_event(C.c_void_p(event.cuda_event) if event is not None else None)


def synchronize() -> None:
    lib().kutacc_b200_synchronize()


# ---- tensor descriptors -----------------------------------------------------------------------
class Tensor:
    """Owns a descriptor (not the data); keeps the backing object alive."""

    def __init__(self, ptr: int, sizes: Sequence[int], strides: Sequence[int], dtype: int, keep=None):
        self.sizes = [int(s) for s in sizes]
        self.strides = [int(s) for s in strides]
        self.dtype = int(dtype)
        self.ptr = int(ptr) if ptr else 0
        self._keep = keep
        n = len(self.sizes)
        arr = C.c_int64 * max(n, 1)
        self.handle = lib().kutacc_b200_tensor_create(C.c_void_p(self.ptr), n, arr(*self.sizes) if n else arr(0),
                                                      arr(*self.strides) if n else arr(0), self.dtype)
        if not self.handle:
            raise_if_error()
            raise KutaccError("tensor descriptor creation failed")

    def __del__(self):
        h = getattr(self, "handle", None)
        if h and _lib is not None:
            _lib.kutacc_b200_tensor_destroy(C.c_void_p(h))
            self.handle = None


def _is_torch(obj) -> bool:
    return type(obj).__module__.startswith("torch")


def tensor(obj, sizes: Optional[Sequence[int]] = None, strides: Optional[Sequence[int]] = None,
           dtype: Optional[int] = None) -> Tensor:
    """Descriptor for a torch tensor or numpy array. Strides are in elements. numpy uint16 arrays
    are taken as bf16 bit patterns. ``sizes``/``strides`` override the object's own view."""
    if isinstance(obj, Tensor):
        return obj
    if _is_torch(obj):
        import torch
        dt = {torch.bfloat16: DTYPE_BF16, torch.float32: DTYPE_FP32, torch.int64: DTYPE_INT64,
              torch.uint8: DTYPE_BF16, torch.int16: DTYPE_BF16}.get(obj.dtype)
        if dt is None:
            raise KutaccError(f"unsupported torch dtype {obj.dtype}")
        return Tensor(obj.data_ptr(), sizes if sizes is not None else list(obj.shape),
                      strides if strides is not None else list(obj.stride()), dtype if dtype is not None else dt, obj)
    if isinstance(obj, np.ndarray):
        dt = {np.dtype(np.uint16): DTYPE_BF16, np.dtype(np.float32): DTYPE_FP32, np.dtype(np.int64): DTYPE_INT64,
              np.dtype(np.uint8): DTYPE_BF16}.get(obj.dtype)
        if dt is None:
            raise KutaccError(f"unsupported numpy dtype {obj.dtype}")
        st = [s // obj.itemsize for s in obj.strides]
        return Tensor(obj.ctypes.data, sizes if sizes is not None else list(obj.shape),
                      strides if strides is not None else st, dtype if dtype is not None else dt, obj)
    raise KutaccError(f"cannot describe object of type {type(obj)}")


def empty_tensor(dtype: int = DTYPE_BF16) -> Tensor:
    """The 'absent pair bias' handle: a valid descriptor whose first size is 0."""
    return Tensor(0, [0], [1], dtype)


def _h(t) -> C.c_void_p:
    return C.c_void_p(t.handle if isinstance(t, Tensor) else (t or 0))


def make_weights(nchannels: int, nheads: int, head_size: int, query_w, key_w, value_w, gating_w, gating_b,
                 output_w, output_b):
    ts = [tensor(t) for t in (query_w, key_w, value_w, gating_w, gating_b, output_w, output_b)]
    w = AttentionWeights(nchannels, nheads, head_size, *[t.handle for t in ts])
    w._keep = ts
    return w


def make_inputs(batch: int, seq_len: int, q=None, k=None, v=None, gate=None, avg=None):
    ts = [None if t is None else tensor(t) for t in (q, k, v, gate, avg)]
    i = AttentionInputs(batch, seq_len, *[(t.handle if t is not None else None) for t in ts])
    i._keep = ts
    return i


# ---- operators (same names and argument order as the reference) -------------------------------
def gating_attention(input, q_based: AttentionInputs, bias, nonbatched_bias, weights: AttentionWeights, out,
                     block_size: int = 128, check: bool = True) -> None:
    lib().kutacc_af2_gating_attention(_h(input), C.byref(q_based) if q_based is not None else None, _h(bias),
                                      _h(nonbatched_bias), C.byref(weights) if weights is not None else None, _h(out),
                                      int(block_size))
    if check:
        raise_if_error()


def global_attention(q_based: AttentionInputs, q_data, q_mask, weights: AttentionWeights, out,
                     check: bool = True) -> None:
    lib().kutacc_af2_global_attention(C.byref(q_based) if q_based is not None else None, _h(q_data), _h(q_mask),
                                      C.byref(weights) if weights is not None else None, _h(out))
    if check:
        raise_if_error()


def gating_attention_ln(input, q_based: AttentionInputs, bias, nonbatched_bias, weights: AttentionWeights, gamma_ptr: int,
                        beta_ptr: int, eps: float, out, block_size: int = 128, check: bool = True) -> None:
    """kutacc_af2_gating_attention on LayerNorm(input); gamma/beta are raw fp32 pointers (host or device)."""
    lib().kutacc_b200_gating_attention_ln(_h(input), C.byref(q_based), _h(bias), _h(nonbatched_bias), C.byref(weights),
                                          C.c_void_p(gamma_ptr), C.c_void_p(beta_ptr), C.c_float(eps), _h(out), int(block_size))
    if check:
        raise_if_error()


def pair_bias_ln(z, gamma_ptr: int, beta_ptr: int, eps: float, wb, nb, check: bool = True) -> None:
    lib().kutacc_b200_pair_bias_ln(_h(z), C.c_void_p(gamma_ptr), C.c_void_p(beta_ptr), C.c_float(eps), _h(wb), _h(nb))
    if check:
        raise_if_error()


def linear(act, weight, bias_ptr: Optional[int], result, beta: int = 0, check: bool = True) -> None:
    lib().kutacc_af2_linear(_h(act), _h(weight), C.c_void_p(bias_ptr or 0), _h(result), int(beta))
    if check:
        raise_if_error()


def pair_bias(z, wb, nb, check: bool = True) -> None:
    lib().kutacc_b200_pair_bias(_h(z), _h(wb), _h(nb))
    if check:
        raise_if_error()


def transition(batch: int, n_res: int, c_o: int, c_i: int, input_act, w1, b1, w2, b2, out, check: bool = True) -> None:
    """out = relu(input_act . w1^T + b1) . w2^T + b2 (kutacc_af2_transition); arguments are api.Tensor objects."""
    wts = TransWeights(c_o, c_i, _h(w1), _h(b1), _h(w2), _h(b2))
    ins = TransInputs(batch, n_res, _h(input_act), None)
    lib().kutacc_af2_transition(C.byref(ins), C.byref(wts), _h(out))
    if check:
        raise_if_error()


# ---- triangle multiplication (include/kutacc.h:426-456) ------------------------------------------
def make_tm_acts(n_res: int, n_res_gather: int, proj_act, input_act, proj_act_gate) -> TmActInputs:
    ts = [None if t is None else tensor(t) for t in (proj_act, input_act, proj_act_gate)]
    a = TmActInputs(n_res, n_res_gather, *[(t.handle if t is not None else None) for t in ts])
    a._keep = ts
    return a


def make_tm_proj_weights(c_o: int, c_i: int, proj_w, proj_b, gate_w, gate_b) -> TmProjWeights:
    ts = [tensor(t) for t in (proj_w, proj_b, gate_w, gate_b)]
    w = TmProjWeights(c_o, c_i, *[t.handle for t in ts])
    w._keep = ts
    return w


def make_tm_linear_weights(c_o: int, c_i: int, gating_w, gating_b, output_proj_w, output_proj_b) -> TmLinearWeights:
    ts = [tensor(t) for t in (gating_w, gating_b, output_proj_w, output_proj_b)]
    w = TmLinearWeights(c_o, c_i, *[t.handle for t in ts])
    w._keep = ts
    return w


def tm_calc_proj(acts: TmActInputs, mask, weights: TmProjWeights, input_prepack: bool = False, check: bool = True) -> None:
    lib().kutacc_af2_triangle_multiplication_calc_proj(C.byref(acts), _h(mask), C.byref(weights), bool(input_prepack))
    if check:
        raise_if_error()


def tm_equation(center_act, left_proj_act, right_proj_act, n_res_gather: int, is_incoming: bool, check: bool = True) -> None:
    lib().kutacc_af2_triangle_multiplication_equation(_h(center_act), _h(left_proj_act), _h(right_proj_act),
                                                      int(n_res_gather), bool(is_incoming))
    if check:
        raise_if_error()


def tm_gate_and_out_linear(gate, out, acts: TmActInputs, center_act, weights: TmLinearWeights, input_prepack: bool = False,
                           check: bool = True) -> None:
    lib().kutacc_af2_triangle_multiplication_gate_and_out_linear(_h(gate), _h(out), C.byref(acts), _h(center_act),
                                                                 C.byref(weights), bool(input_prepack))
    if check:
        raise_if_error()


def tm_last(out, gate, n_res: int, n_res_gather: int, c_o: int, check: bool = True) -> None:
    lib().kutacc_af2_triangle_multiplication_last(_h(out), _h(gate), int(n_res), int(n_res_gather), int(c_o))
    if check:
        raise_if_error()


def transpose(data, out, check: bool = True) -> None:
    """Re-shard between row-split and column-split byte matrices (kutacc_af2_transpose)."""
    lib().kutacc_af2_transpose(_h(data), _h(out))
    if check:
        raise_if_error()


def layernorm_rows(data_ptr: int, gamma_ptr: int, beta_ptr: int, rows: int, size: int, eps: float, out_ptr: int,
                   row_stride: Optional[int] = None, out_row_stride: Optional[int] = None, check: bool = True) -> None:
    """LayerNorm of every row of a [rows, size] bf16 matrix (raw host or device addresses)."""
    lib().kutacc_b200_layernorm_rows(C.c_void_p(data_ptr), C.c_void_p(gamma_ptr), C.c_void_p(beta_ptr), int(rows),
                                     int(size), int(row_stride or size), int(out_row_stride or size), float(eps),
                                     C.c_void_p(out_ptr))
    if check:
        raise_if_error()


def layernorm(data_ptr: int, gamma_ptr: int, beta_ptr: int, size: int, eps: float, out_ptr: int, check: bool = True) -> None:
    """The reference's one-row entry point."""
    lib().kutacc_af2_layernorm(C.c_void_p(data_ptr), C.c_void_p(gamma_ptr), C.c_void_p(beta_ptr), int(size), float(eps),
                               C.c_void_p(out_ptr))
    if check:
        raise_if_error()


def all_gather(data, out, check: bool = True) -> None:
    lib().kutacc_af2_all_gather(_h(data), _h(out))
    if check:
        raise_if_error()


def comm_init(world_size: int, rank: int, buffer_size: int = 0, unique_id: Optional[bytes] = None) -> None:
    if unique_id is None:
        lib().kutacc_comm_init(world_size, rank, buffer_size)
    else:
        buf = C.create_string_buffer(unique_id, 128)
        lib().kutacc_b200_comm_init_with_id(world_size, rank, buf)
    raise_if_error()


def comm_unique_id() -> bytes:
    buf = C.create_string_buffer(128)
    lib().kutacc_b200_comm_unique_id(buf)
    raise_if_error()
    return buf.raw


def comm_fini() -> None:
    lib().kutacc_comm_fini()
    raise_if_error()


def gemm_pack_get_size(identifier: str, m: int, n: int, k: int) -> int:
    return int(lib().kutacc_af2_gemm_pack_get_size(identifier.encode(), b"N", b"N", m, n, k))
