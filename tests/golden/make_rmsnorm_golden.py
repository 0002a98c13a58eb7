"""Generates ``rmsnorm_ref.npz`` with the REFERENCE's own ``llmops.rmsnorm`` (ops/op_misc.hpp:142-181), called
through its compiled Python module (oracle/build_ref_module.py): seeded inputs, weights, eps and the rows the
reference returns.  Run in the build container only:
    python tests/golden/make_rmsnorm_golden.py [--reference /path/to/llama.cl]
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("Q4FC_REFERENCE"))
    a = ap.parse_args()
    if not a.reference:
        raise SystemExit("give --reference /path/to/llama.cl (or set Q4FC_REFERENCE)")
    sys.path.insert(0, ROOT)
    from oracle import build_ref_module

    mod = build_ref_module.build(a.reference)
    if mod is None:
        raise SystemExit("the reference tree (or pybind11) is not available here")
    sys.path.insert(0, os.path.dirname(mod))
    import llmops

    rng = np.random.default_rng(20240611)
    out = {}
    for i, (rows, K, eps, spread) in enumerate([(3, 64, 1e-5, 1.0), (8, 1024, 1e-6, 3.0), (1, 4096, 1e-5, 0.02)]):
        x = (rng.standard_normal((1, rows, K)) * spread).astype(np.float32)
        w = (rng.random(K) + 0.5).astype(np.float32)
        y = x.copy()
        xt, wt = llmops.tensor(y), llmops.tensor(w)  # wraps the arrays: the op works in place on y
        llmops.rmsnorm(xt, wt, eps)
        out[f"x{i}"], out[f"w{i}"], out[f"eps{i}"], out[f"y{i}"] = x, w, np.float32(eps), y
    out["cases"] = np.int32(3)
    np.savez_compressed(os.path.join(HERE, "rmsnorm_ref.npz"), **out)
    print("written", os.path.join(HERE, "rmsnorm_ref.npz"))


if __name__ == "__main__":
    main()
