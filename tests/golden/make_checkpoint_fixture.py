"""Generates ``ref_checkpoint_tiny.pkl`` and ``ref_checkpoint_tiny.npz`` with the REFERENCE's own code:
its compiled ``llmops`` module (oracle/build_ref_module.py) and the op classes of its chatllama/main.py.

The pickle has the shape of what ``Model.save`` writes (chatllama/main.py:305-308): a dict holding
``op_dict`` (embedding, per-layer rmsnorm + FC ops, final norm, lm_head), ``configs`` and ``inv_freq``.
It is written as the script form of the reference writes it: the op classes are pickled under
``__main__`` (the reference is run as ``python main.py``).  Weights are seeded random, sizes tiny.
The npz holds what a reader needs to check itself against: the SHA-256 of the pickle, and per FC the fp32
weight, one input and the reference's output, so that the packed bytes can be re-derived and the FC re-run.

Needs the reference tree; run in the build container only:
    python tests/golden/make_checkpoint_fixture.py [--reference /path/to/llama.cl]
"""
from __future__ import annotations

import argparse
import hashlib
import os
import pickle
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("Q4FC_REFERENCE"), required="Q4FC_REFERENCE" not in os.environ)
    a = ap.parse_args()
    sys.path.insert(0, ROOT)
    from oracle import build_ref_module

    mod = build_ref_module.build(a.reference)
    if mod is None:
        raise SystemExit("the reference tree (or pybind11) is not available here")
    sys.path.insert(0, os.path.dirname(mod))
    sys.path.insert(0, os.path.join(a.reference, "chatllama"))
    import llmops  # the reference's compiled module
    import main as refmain  # the reference's model file (imported, not run)

    # the reference pickles its op classes under __main__ because it runs as a script
    main_mod = sys.modules["__main__"]
    for name in ("llmop_fc_q4a", "llmop_rmsnorm", "llmop_embedding_q8c"):
        cls = getattr(refmain, name)
        cls.__module__ = "__main__"
        setattr(main_mod, name, cls)

    torch.manual_seed(20240607)
    H, I, V, L = 64, 96, 64, 1  # hidden, intermediate, vocabulary (whole stripes: the reference writes 32 columns per stripe), layers
    lin = lambda n, k: torch.nn.Linear(k, n, bias=False)  # noqa: E731
    fcs = {}

    def fc(name, n, k):
        layer = lin(n, k)
        with torch.no_grad():
            layer.weight.mul_(0.5)
        fcs[name] = layer.weight.detach().clone()
        return refmain.llmop_fc_q4a(layer)

    layers = []
    for i in range(L):
        layers.append({
            "input_layernorm": refmain.llmop_rmsnorm(torch.rand(H) + 0.5, 1e-5),
            "post_attention_layernorm": refmain.llmop_rmsnorm(torch.rand(H) + 0.5, 1e-5),
            "self_attn.q_proj": fc(f"layers.{i}.self_attn.q_proj", H, H),
            "self_attn.k_proj": fc(f"layers.{i}.self_attn.k_proj", H, H),
            "self_attn.v_proj": fc(f"layers.{i}.self_attn.v_proj", H, H),
            "self_attn.o_proj": fc(f"layers.{i}.self_attn.o_proj", H, H),
            "mlp.gate_proj": fc(f"layers.{i}.mlp.gate_proj", I, H),
            "mlp.up_proj": fc(f"layers.{i}.mlp.up_proj", I, H),
            "mlp.down_proj": fc(f"layers.{i}.mlp.down_proj", H, I),
        })
    op_dict = {
        "model.embed_tokens": refmain.llmop_embedding_q8c(torch.randn(V, H)),
        "layers": layers,
        "model.norm": refmain.llmop_rmsnorm(torch.rand(H) + 0.5, 1e-5),
        "lm_head": fc("lm_head", V, H),
    }
    configs = {"layer_num": L, "head_num": 4, "head_size": H // 4, "hidden_size": H,
               "max_position_embeddings": 128, "rotary_dims": H // 4, "rms_norm_eps": 1e-5}
    inv_freq = 1.0 / (10000 ** (torch.arange(0, H // 4, 2).float() / (H // 4)))
    state = {"op_dict": op_dict, "configs": configs, "inv_freq": refmain.to_lt(inv_freq).clone()}

    path = os.path.join(HERE, "ref_checkpoint_tiny.pkl")
    with open(path, "wb") as f:
        pickle.dump(state, f)

    # companion facts, computed with the reference's ops
    facts = {"pickle_sha256": np.frombuffer(hashlib.sha256(open(path, "rb").read()).digest(), dtype=np.uint8),
             "names": np.array(sorted(fcs))}
    for name, W in fcs.items():
        parts = name.split(".")
        op = op_dict["lm_head"] if name == "lm_head" else op_dict["layers"][int(parts[1])][".".join(parts[2:])]
        xin = torch.randn(1, 3, W.shape[1], generator=torch.Generator().manual_seed(len(name)))
        xa = xin.numpy().copy()  # llmops.tensor wraps the memory without owning it: keep the array alive
        y = op(llmops.tensor(xa))
        facts[name + "/W"] = W.numpy()
        facts[name + "/x"] = xin.numpy()
        facts[name + "/y"] = y.numpy().copy()
        facts[name + "/packed"] = op.weight.numpy().copy()
    facts["inv_freq"] = state["inv_freq"].numpy().copy()
    facts["embed_weight"] = op_dict["model.embed_tokens"].weight.numpy().copy()
    np.savez_compressed(os.path.join(HERE, "ref_checkpoint_tiny.npz"), **facts)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
