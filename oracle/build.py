"""Compile the CPU oracle (test infrastructure) into oracle/libkutacc_oracle.so.

The reference's own translation units for this path cannot be compiled on x86: they include
arm_sve.h / arm_neon.h (src/attention/gating_attention.cpp:16-18) and link a closed GEMM
(src/CMakeLists.txt:76-79). So there is no oracle/_ref build; the oracle is the restatement in
kutacc_oracle.cpp.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "kutacc_oracle.cpp")
LIB = os.path.join(HERE, "libkutacc_oracle.so")


def build(force: bool = False) -> str:
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    cmd = ["g++", "-O3", "-march=x86-64-v3", "-fopenmp", "-std=c++17", "-shared", "-fPIC", "-o", LIB, SRC]
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
