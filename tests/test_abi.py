"""The C-ABI boundary without a GPU: exported symbols, argument validation, error convention.

The robustness cases follow the reference's own operator tests
(test/functest/cal/gating_attention_test.cpp:18-264, global_attention_test.cpp:18-189): one null
handle or one bad integer, every other "handle" a pointer to unrelated stack memory, and the call
must return without dereferencing anything.
"""
import ctypes as C
import os
import re

import numpy as np
import pytest

from kutacc_b200 import api

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "kutacc_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"#define[^\n]*", "", text)
    names = re.findall(r"KUTACC_B200_API\s+[\w\s\*]*?\b(\w+)\s*\(", text)
    data = re.findall(r"KUTACC_B200_API\s+extern\s+int64_t\s+(\w+)\s*;", text)
    return sorted(set(names)), sorted(set(data))


def test_library_exports_every_declared_symbol(kutacc_lib):
    funcs, data = _declared_functions()
    assert "kutacc_af2_gating_attention" in funcs and "kutacc_af2_global_attention" in funcs
    for name in funcs:
        if name in ("TensorWrapper",):
            continue
        assert hasattr(kutacc_lib, name), f"{name} declared in include/kutacc_b200.h but not exported"
    for name in data:
        C.c_int64.in_dll(kutacc_lib, name)
    for name in api.EXPORTS:
        assert name in funcs, f"{name} bound in api.py but not declared in the header"
    # C++ descriptor class with the reference's constructor signature (mangled, cxx11 ABI)
    assert hasattr(kutacc_lib, "_ZN6kutacc13TensorWrapperC1EPvOSt6vectorIlSaIlEES5_lNS_14TensorDataTypeE")
    assert hasattr(kutacc_lib, "_ZN6kutacc13TensorWrapperD1Ev")
    # entry points of the reference outside this path still resolve (they report "not built")
    for name in ("kutacc_af2_outer_product_mean_chunk",
                 "kutacc_af2_invariant_point", "kutacc_af2_triangle_multiplication_last"):
        assert hasattr(kutacc_lib, name)


def test_version(kutacc_lib):
    v = api.version()
    assert v["component_name"] == "KuTACC" and v["component_abi_version"] == "1"
    assert kutacc_lib.kutacc_get_version(None) == -1          # KUTACC_ERROR on null (version.cpp:30-32)


def test_rank_globals_default(kutacc_lib):
    assert C.c_int64.in_dll(kutacc_lib, "world_size").value == 1
    assert C.c_int64.in_dll(kutacc_lib, "rank").value == 0


class _Bogus:
    """'Handles' that point at unrelated memory, as the reference tests do."""

    def __init__(self):
        self.buf = (C.c_float * 8)(1.5, 2, 3, 4, 7, 8, 9, 10)
        self.p = C.cast(self.buf, C.c_void_p)

    def weights(self, nchannels=2, nheads=1, head_size=2):
        p = self.p.value
        return api.AttentionWeights(nchannels, nheads, head_size, p, p, p, p, p, p, p)

    def inputs(self, batch=2, seq_len=2):
        p = self.p.value
        return api.AttentionInputs(batch, seq_len, p, p, p, p, p)


@pytest.mark.parametrize("null_arg", range(6))
def test_gating_attention_null_arguments(kutacc_lib, capfd, null_arg):
    b = _Bogus()
    w, i = b.weights(), b.inputs()
    args = [b.p, C.byref(i), b.p, b.p, C.byref(w), b.p]
    args[null_arg] = None
    kutacc_lib.kutacc_af2_gating_attention(*args, 5)
    assert api.error_set()
    assert "nullptr" in api.last_error()
    err = capfd.readouterr().err
    assert err.startswith("KUTACC_CHECK fail in kutacc_af2_gating_attention at ")
    assert " , kutacc_af2_gating_attention: input args nullptr error" in err


@pytest.mark.parametrize("field,value", [("block_size", -5), ("batch", -2), ("seq_len", 0), ("nheads", -1),
                                         ("head_size", 0), ("nchannels", -64)])
def test_gating_attention_bad_integers(kutacc_lib, field, value):
    b = _Bogus()
    kw_w, kw_i, block = {}, {}, 5
    if field == "block_size":
        block = value
    elif field in ("batch", "seq_len"):
        kw_i[field] = value
    else:
        kw_w[field] = value
    w, i = b.weights(**kw_w), b.inputs(**kw_i)
    kutacc_lib.kutacc_af2_gating_attention(b.p, C.byref(i), b.p, b.p, C.byref(w), b.p, block)
    assert api.error_set()
    assert "input param <= 0 or overflow" in api.last_error()


@pytest.mark.parametrize("null_arg", range(5))
def test_global_attention_null_arguments(kutacc_lib, null_arg):
    b = _Bogus()
    w, i = b.weights(nchannels=64, nheads=8, head_size=8), b.inputs()
    args = [C.byref(i), b.p, b.p, C.byref(w), b.p]
    args[null_arg] = None
    kutacc_lib.kutacc_af2_global_attention(*args)
    assert api.error_set()


def test_global_attention_rejects_other_channel_counts(kutacc_lib):
    # nchannels != 64 is refused before any handle is touched (global_attention.cpp:171-173)
    b = _Bogus()
    w, i = b.weights(nchannels=2, nheads=1, head_size=2), b.inputs()
    kutacc_lib.kutacc_af2_global_attention(C.byref(i), b.p, b.p, C.byref(w), b.p)
    assert api.error_set()
    assert "invalid int value" in api.last_error()


def test_error_flag_is_sticky_and_clearable(kutacc_lib):
    kutacc_lib.kutacc_af2_all_gather(None, None)
    assert api.error_set()
    # while the flag is set every operator returns early, valid arguments or not
    x = np.zeros((4, 8), dtype=np.uint16)
    t = api.tensor(x)
    api.linear(t, t, None, t, 0, check=False)
    assert api.error_set()
    api.clear_error()
    assert not api.error_set() and api.last_error() == ""
    with pytest.raises(api.KutaccError):
        api.linear(None, t, None, t, 0)
    assert not api.error_set()         # raise_if_error clears


def test_not_built_entry_points_report(kutacc_lib):
    kutacc_lib.kutacc_af2_invariant_point()
    assert api.error_set() and "not part of" in api.last_error()
    api.clear_error()
    # the reference's robustness tests for the triangle multiplication: one null handle each
    # (test/functest/cal/triangle_multiplication_test.cpp)
    kutacc_lib.kutacc_af2_triangle_multiplication_last(None, None, 2, 2, 2)
    assert api.error_set() and "input args nullptr error" in api.last_error()
    api.clear_error()
    kutacc_lib.kutacc_af2_triangle_multiplication_equation(None, None, None, 4, False)
    assert api.error_set() and "nullptr" in api.last_error()
    api.clear_error()
    # null arguments of a built operator are reported in the reference's words, nothing is dereferenced
    kutacc_lib.kutacc_af2_transition(None, None, None)
    assert api.error_set() and "nullptr" in api.last_error()


def test_tensor_descriptor_checks(kutacc_lib):
    x = np.zeros((3, 5), dtype=np.float32)
    t = api.tensor(x)
    assert t.sizes == [3, 5] and t.strides == [5, 1] and t.dtype == api.DTYPE_FP32
    e = api.empty_tensor()
    assert e.sizes == [0]
    h = kutacc_lib.kutacc_b200_tensor_create(None, 2, None, None, 1)
    assert not h and api.error_set()


def test_pack_size_and_host_prepack(kutacc_lib):
    assert api.gemm_pack_get_size("A", 7, 9, 11) == 77
    assert api.gemm_pack_get_size("B", 7, 9, 11) == 99
    rng = np.random.default_rng(0)
    w = rng.integers(0, 65535, (40, 24), dtype=np.uint16)       # [n=40, k=16] with ldb=24
    packed = np.zeros((40, 16), dtype=np.uint16)
    kutacc_lib.kutacc_af2_linear_weight_prepack(w.ctypes.data, packed.ctypes.data, 40, 16, 24, 0)
    assert not api.error_set()
    assert np.array_equal(packed, w[:, :16])


def test_shape_mismatch_is_reported_before_any_launch(kutacc_lib):
    x = np.zeros((4, 8), dtype=np.uint16)
    wgt = np.zeros((8, 6), dtype=np.uint16)      # k mismatch
    r = np.zeros((4, 8), dtype=np.uint16)
    with pytest.raises(api.KutaccError, match="shape invalid"):
        api.linear(api.tensor(x), api.tensor(wgt), None, api.tensor(r), 0)
    i = api.make_inputs(2, 2)
    w = api.make_weights(8, 3, 2, x, x, x, x, np.zeros(8, np.float32), x, np.zeros(8, np.float32))
    with pytest.raises(api.KutaccError, match="nheads \\* head_size"):
        api.gating_attention(api.tensor(x), i, api.tensor(x), api.empty_tensor(), w, api.tensor(r), 4)
