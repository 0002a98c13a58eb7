"""A model saved by the reference runs on the GPU kernels as it is: packed weights go to the device byte for
byte (no repacking), outputs match what the reference's own fc_Q4A returned for the same inputs."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
PKL = os.path.join(HERE, "golden", "ref_checkpoint_tiny.pkl")
NPZ = os.path.join(HERE, "golden", "ref_checkpoint_tiny.npz")


def test_reference_checkpoint_runs_on_the_gpu(lib_built):
    import llama_cl_b200 as pkg
    from llama_cl_b200 import checkpoint

    facts = np.load(NPZ)
    model = checkpoint.load(PKL)
    ops = checkpoint.fc_ops(model, "cuda")
    assert sorted(ops) == ["op_dict." + n for n in facts["names"]]
    for name in facts["names"]:
        op = ops["op_dict." + name]
        W, x, y = facts[name + "/W"], facts[name + "/x"], facts[name + "/y"]
        # the device copy is the reference's bytes, and so is what the GPU packer makes of the fp32 weight
        assert np.array_equal(op.weight.cpu().numpy(), facts[name + "/packed"])
        repacked = pkg.llmops.offline_FC_quant_Q4A(torch.from_numpy(W).cuda(), qtype="q4_1", group_k=32)
        assert torch.equal(repacked, op.weight), name
        got = op(torch.from_numpy(x).cuda()).cpu().numpy()
        assert got.shape == y.shape
        assert np.allclose(got, y, rtol=1e-3, atol=1e-4), (name, float(np.abs(got - y).max()))
    # write-back: a weight repacked on the GPU lands in the model and the file stays loadable by either side
    first = "op_dict." + str(facts["names"][0])
    target = dict(checkpoint.walk_ops(model))[first]
    checkpoint.store_fc(target, ops[first])
    assert checkpoint.dumps(model) == open(PKL, "rb").read()


def test_reference_checkpoint_embedding_table_on_the_gpu(lib_built):
    """The quantized token table of a saved model (llmop_embedding_q8c: int8 codes, one scale per row) goes to the
    device as it is; a look-up returns scale * code, the reference's arithmetic, bit for bit."""
    from llama_cl_b200 import checkpoint

    model = checkpoint.load(PKL)
    embs = checkpoint.embedding_ops(model, "cuda")
    assert list(embs) == ["op_dict.model.embed_tokens"]
    op = embs["op_dict.model.embed_tokens"]
    host = dict(checkpoint.walk_ops(model))["op_dict.model.embed_tokens"]
    codes, scales = host.weight.numpy(), host.scales.numpy()
    V = codes.shape[0]
    ids = np.array([[0, V - 1, 3 % V, 1 % V]], dtype=np.int64)
    got = op(torch.from_numpy(ids)).cpu().numpy()
    want = scales[ids][..., None] * codes[ids].astype(np.float32)
    assert got.shape == (1, 4, codes.shape[1]) and np.array_equal(got, want)
