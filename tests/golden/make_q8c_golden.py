"""Generates ``q8c_ref.npz`` with the REFERENCE's own code: ``FC_quant_Q8C`` / ``FC_evaluate_Q8C`` of its older torch
extension (ext/llama_ext.cpp:56-113, 232-371; built by oracle/build_ref_ext.py) and ``embedding_q8c_quant_w`` /
``embedding_q8c`` of its ops module (ops/op_embedding.hpp:51-137; built by oracle/build_ref_module.py): seeded
inputs and what the reference returns.  Run in the build container only:
    python tests/golden/make_q8c_golden.py --reference /path/to/llama.cl
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
    import torch

    from oracle import build_ref_ext, build_ref_module

    build_ref_ext.build(a.reference)
    ext = build_ref_ext.load_module()
    mod = build_ref_module.build(a.reference)
    if ext is None or mod is None:
        raise SystemExit("the reference tree (or its build prerequisites) is not available here")
    sys.path.insert(0, os.path.dirname(mod))
    import llmops

    g = torch.Generator().manual_seed(20240613)
    out = {}
    # N % 32 == 0 throughout: the reference stores whole 32-column groups into a [B, M, N] output
    for i, (N, K, rows) in enumerate([(64, 128, 3), (96, 1024, 8), (32, 4096, 1), (64, 70, 2)]):
        W = torch.randn(N, K, generator=g) * 0.02
        x = torch.randn(1, rows, K, generator=g)
        wq, ws = ext.FC_quant_Q8C(W)
        y = ext.FC_evaluate_Q8C(x, wq, ws, N)
        out[f"W{i}"], out[f"x{i}"] = W.numpy(), x.numpy()
        out[f"wq{i}"], out[f"ws{i}"], out[f"y{i}"] = wq.numpy(), ws.numpy(), y.numpy()
    out["fc_cases"] = np.int32(4)
    rng = np.random.default_rng(20240614)
    for i, (V, E, n) in enumerate([(50, 64, 7), (16, 4096, 5), (20, 100, 4)]):
        table = rng.standard_normal((V, E)).astype(np.float32)
        ids = rng.integers(0, V, size=(1, n)).astype(np.int64)
        wt = llmops.tensor(table)
        codes, scales = llmops.embedding_q8c_quant_w(wt)
        res = np.zeros((1, n, E), dtype=np.float32)
        llmops.embedding_q8c(llmops.tensor(res), llmops.tensor(ids), codes, scales)
        out[f"table{i}"], out[f"ids{i}"] = table, ids
        out[f"codes{i}"], out[f"scales{i}"], out[f"emb{i}"] = np.array(codes.numpy()), np.array(scales.numpy()), res
    out["emb_cases"] = np.int32(3)
    np.savez_compressed(os.path.join(HERE, "q8c_ref.npz"), **out)
    print("written", os.path.join(HERE, "q8c_ref.npz"))


if __name__ == "__main__":
    main()
