"""Link-level boundary test: a C++ caller compiled against the reference's OWN public header
(include/kutacc.h of the reference, found through KUTACC_REFERENCE_INCLUDE or the build container's mount) and
linked with -lkutacc runs against this library.

The CPU part builds tests/link_caller.cpp and runs its null-handle path. The built program is kept beside the
library (tests/_built/, not tracked) so that the GPU part can run one small real call with it on a machine that
does not have the reference's header, and check the result against the CPU oracle.
"""
import os
import struct
import subprocess

import numpy as np
import pytest

from kutacc_b200 import api
from kutacc_b200 import workloads as W
from tests import helpers

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BUILT = os.path.join(ROOT, "tests", "_built")
BINARY = os.path.join(BUILT, "link_caller")


def _reference_include():
    for cand in (os.environ.get("KUTACC_REFERENCE_INCLUDE"), "/root/reference/include"):
        if cand and os.path.exists(os.path.join(cand, "kutacc.h")):
            return cand
    return None


def _env():
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = BUILT + ":" + env.get("LD_LIBRARY_PATH", "")
    return env


def test_caller_built_against_the_reference_header_links_and_reports_null_handles(kutacc_lib):
    inc = _reference_include()
    if inc is None:
        pytest.skip("the reference's include/kutacc.h is not on this machine")
    os.makedirs(BUILT, exist_ok=True)
    # the SONAME the reference's binaries ask for
    link = os.path.join(BUILT, "libkutacc.so.1")
    if os.path.islink(link) or os.path.exists(link):
        os.remove(link)
    os.symlink(api.LIB_PATH, link)
    # __bf16 in the header needs a recent g++; -include vector because the header uses std::vector without including it
    cmd = ["g++", "-std=c++17", "-O1", "-include", "vector", "-include", "cstdint", "-I", inc, os.path.join(ROOT, "tests", "link_caller.cpp"),
           "-o", BINARY, "-L", os.path.dirname(api.LIB_PATH), "-lkutacc", "-Wl,-rpath," + os.path.dirname(api.LIB_PATH)]
    subprocess.check_call(cmd)
    p = subprocess.run([BINARY, "null"], env=_env(), capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stdout + p.stderr
    assert "linked against" in p.stdout and "null handle reported" in p.stdout
    assert "KUTACC_CHECK fail in kutacc_af2_gating_attention" in p.stderr and "input args nullptr error" in p.stderr


@pytest.mark.gpu
def test_caller_built_against_the_reference_header_computes_the_oracle_result(kutacc_lib, tmp_path):
    if not os.path.exists(BINARY):
        pytest.skip("tests/_built/link_caller has not been built (needs the reference's header; the CPU test builds it)")
    w = W.random_gating_case(seed=41, B=2, S=72, H=2, D=32, with_nb=True, full_mask_rows=1)
    A = w.arrays
    blob = struct.pack("<5q", w.B, w.S, w.H, w.D, 1)
    blob += W.bf16_bits(A["x"]).tobytes()
    for k in ("wq", "wk", "wv", "wg", "wo"):
        blob += W.bf16_bits(A[k]).tobytes()
    blob += A["bg"].astype(np.float32).tobytes() + A["bo"].astype(np.float32).tobytes()
    blob += W.bf16_bits(A["bias"]).tobytes() + W.bf16_bits(A["nb"]).tobytes()
    src, dst = tmp_path / "in.bin", tmp_path / "out.bin"
    src.write_bytes(blob)
    p = subprocess.run([BINARY, "run", str(src), str(dst)], env=_env(), capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stdout + p.stderr
    got = W.as_f32(np.frombuffer(dst.read_bytes(), dtype=np.uint16)).reshape(w.B, w.S, w.C)
    assert helpers.rel_err(got, helpers.oracle_faithful(w)) <= helpers.BF16_TOL
