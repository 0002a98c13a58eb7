"""Generates ``silu_mul_ref.npz`` with the REFERENCE's own ``llmops.itrans(gate, "silu")`` and
``llmops.imul(up, gate)`` (ops/op_misc.hpp:83-138; the MLP glue of chatllama/main.py:365-368), called through
its compiled Python module (oracle/build_ref_module.py): seeded gate / up rows and the products the reference
returns.  Run in the build container only:
    python tests/golden/make_silu_golden.py --reference /path/to/llama.cl
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

    rng = np.random.default_rng(20240612)
    out = {}
    for i, (rows, K, spread) in enumerate([(3, 64, 1.0), (8, 1024, 4.0), (1, 11008, 2.0), (2, 256, 30.0)]):
        gate = (rng.standard_normal((1, rows, K)) * spread).astype(np.float32)
        up = (rng.standard_normal((1, rows, K)) * spread).astype(np.float32)
        g, u = gate.copy(), up.copy()
        gt, ut = llmops.tensor(g), llmops.tensor(u)  # wrap the arrays: the ops work in place
        llmops.itrans(gt, "silu")
        llmops.imul(ut, gt)
        out[f"gate{i}"], out[f"up{i}"], out[f"prod{i}"] = gate, up, u
    out["cases"] = np.int32(4)
    np.savez_compressed(os.path.join(HERE, "silu_mul_ref.npz"), **out)
    print("written", os.path.join(HERE, "silu_mul_ref.npz"))


if __name__ == "__main__":
    main()
