"""Parity of the five benchmark shapes against the CPU oracle, as a markdown table (run on a GPU box).

    python tests/parity_report.py [rows]

Each shape runs its full sequence length on the first `rows` batch rows (default 6; the oracle is a CPU
program) through libkutacc.so with device-resident tensors; the error is max|got - ref| / max|ref| against
the faithful oracle (every bf16 store of the reference) and against the exact oracle (fp32 in, double
accumulate). The tolerances are the ones the tests assert (tests/helpers.py).
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from kutacc_b200 import runner                     # noqa: E402
from kutacc_b200 import workloads as W             # noqa: E402
from tests import helpers                          # noqa: E402


def main():
    rows = int(sys.argv[1]) if len(sys.argv) > 1 else 6
    print("| workload | rows x S | dtype | err vs faithful oracle | err vs exact oracle | tolerance | mean abs err / max|ref| "
          "| share of elements beyond 2 bf16 ulps of the reference |")
    print("|---|---|---|---|---|---|---|---|")
    for name in W.NAMES:
        w = W.make(name, rows=rows)
        got = runner.out_to_f32(runner.DeviceCase(w).run())
        torch.cuda.synchronize()
        assert np.isfinite(got).all(), name
        exact = helpers.rel_err(got, helpers.oracle_exact(w))
        faithful = helpers.rel_err(got, helpers.oracle_faithful(w)) if w.dtype == "bf16" else float("nan")
        tol = helpers.BF16_TOL if w.dtype == "bf16" else helpers.FP32_TOL
        ref = helpers.oracle_faithful(w) if w.dtype == "bf16" else helpers.oracle_exact(w)
        diff = np.abs(got.astype(np.float64) - ref.astype(np.float64))
        mean_abs = float(diff.mean() / max(np.abs(ref).max(), 1e-30))
        ulp = np.maximum(np.abs(ref.astype(np.float64)), 2.0 ** -126) * 2.0 ** -7        # one bf16 ulp at |ref| (upper bound)
        beyond = float((diff > 2 * ulp).mean()) if w.dtype == "bf16" else float("nan")
        print(f"| {name} | {w.B} x {w.S} | {w.dtype} | {faithful:.2e} | {exact:.2e} | {tol:.0e} | {mean_abs:.2e} | {beyond:.4f} |")


if __name__ == "__main__":
    main()
