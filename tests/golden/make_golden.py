"""Generate the golden fixtures in this folder from the COMPILED REFERENCE.

Run in a container that has the reference checkout (Q4FC_REFERENCE=/path/to/llama.cl):

    python oracle/build_oracle.py          # builds oracle/_ref from the reference sources
    python tests/golden/make_golden.py

Outputs (committed):
  q4fc_small_<variant>.npz   seeded small case per block variant: inputs and
                             the reference's packed bytes, dequantized weights,
                             Q8 codes / scales / group sums and FC output.
  known_answer_q4_1.npz      the reference's own lossless test construction
                             (ops/test_ops.py:106-149) at a reduced size, with
                             the reference's outputs.
  config1_sha256.json        SHA-256 of the reference's outputs on the
                             4096x4096 Q4_1/g32 seed-0 case.
"""
from __future__ import annotations

import hashlib
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import cpu  # noqa: E402


def sha(a) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def small_case(qtype: int, G: int) -> None:
    ref = cpu.compiled_reference(qtype, G, "vnni")
    g = torch.Generator().manual_seed(1000 * qtype + G)
    N, K, B, M = 96, 512, 2, 3
    W = (torch.randn(N, K, generator=g) * 0.02).numpy()
    x = torch.randn(B, M, K, generator=g).numpy()
    # a few exact ties and zeros to pin the rounding rules
    W[0, :8] = 0.0
    x[0, 0, :8] = [127, .5, 1.5, 2.5, -.5, -1.5, -2.5, 3.5]
    wq = ref.pack(W)
    codes, scales, gsums = ref.quant_x(x)
    np.savez_compressed(
        os.path.join(HERE, f"q4fc_small_{cpu.variant_name(qtype, G)}.npz"),
        W=W, x=x, N=N, packed=wq, dequant=ref.dequant(wq), codes=codes, scales=scales, gsums=gsums,
        y=ref.fc(x, wq, N))


def known_answer() -> None:
    # ops/test_ops.py:106-149 at N=K=256, B=2, M=5: exactly representable
    # weights / activations, so Q4_1 packing is lossless and the FC equals fp32 linear.
    g = torch.Generator().manual_seed(7)
    N, K, B, M = 256, 256, 2, 5
    w = torch.randint(-8, 8, (N, K), generator=g).float()
    x = torch.randint(-127, 128, (B, M, K), generator=g).float()
    for k in range(0, K, 32):
        w[:, k] = -8
        w[:, k + 1] = 7
        x[:, :, k] = -127
        x[:, :, k + 1] = 127
    w = (w * (1 / 128)).numpy()
    x = (x * (1 / 128)).numpy()
    out = {"W": w, "x": x, "linear": (torch.from_numpy(x) @ torch.from_numpy(w).T).numpy()}
    for G in (32, 128):
        ref = cpu.compiled_reference(1, G, "vnni")
        wq = ref.pack(w)
        out[f"packed_g{G}"] = wq
        out[f"y_g{G}"] = ref.fc(x, wq, N)
        assert np.array_equal(ref.dequant(wq), w)
        assert np.allclose(out[f"y_g{G}"], out["linear"])
    np.savez_compressed(os.path.join(HERE, "known_answer_q4_1.npz"), **out)


def config1() -> None:
    g = torch.Generator().manual_seed(0)
    W = (torch.randn(4096, 4096, generator=g) * 0.02).numpy()
    x = torch.randn(1, 1, 4096, generator=g).numpy()
    ref = cpu.compiled_reference(1, 32, "vnni")
    wq = ref.pack(W)
    codes, scales, gsums = ref.quant_x(x)
    y = ref.fc(x, wq, 4096)
    rec = {
        "recipe": "g=torch.Generator().manual_seed(0); W=randn(4096,4096,generator=g)*0.02; x=randn(1,1,4096,generator=g); Q4_1 group 32",
        "W_head": [float(v) for v in W[0, :3]], "x_head": [float(v) for v in x[0, 0, :3]],
        "packed": sha(wq), "codes": sha(codes), "scales": sha(scales), "gsums": sha(gsums), "y": sha(y),
        "y_head": [float(v) for v in y[0, 0, :4]], "y_sum_f64": float(y.astype(np.float64).sum()),
    }
    with open(os.path.join(HERE, "config1_sha256.json"), "w") as f:
        json.dump(rec, f, indent=1)


if __name__ == "__main__":
    for q in (0, 1):
        for G in (32, 128):
            small_case(q, G)
    known_answer()
    config1()
    print("golden fixtures written to", HERE)
