"""The CPU oracle against the reference's golden vectors (no GPU needed)."""
import hashlib
import json
import os

import numpy as np
import pytest
import torch

VARIANTS = [(0, 32), (0, 128), (1, 32), (1, 128)]


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.mark.parametrize("qtype,G", VARIANTS)
def test_restatement_matches_reference_fixture(oracle, golden_dir, qtype, G):
    """Fixtures were produced by the reference's own compiled code (make_golden.py)."""
    z = np.load(os.path.join(golden_dir, f"q4fc_small_{oracle.variant_name(qtype, G)}.npz"))
    W, x, N = z["W"], z["x"], int(z["N"])
    wq = oracle.restated.pack(W, qtype, G)
    assert wq.shape == z["packed"].shape and np.array_equal(wq, z["packed"])
    assert np.array_equal(oracle.restated.dequant(wq), z["dequant"])
    codes, scales, gsums = oracle.restated.quant_x(x, G, 1.0 if qtype else 1.0 / 16)
    assert np.array_equal(codes, z["codes"])
    assert np.array_equal(scales, z["scales"])
    assert np.array_equal(gsums, z["gsums"])
    y = oracle.restated.fc(x, wq, N)
    assert np.array_equal(y, z["y"])  # same fp32 operation order: bit-equal


def test_q8_rounding_rule(oracle, golden_dir):
    """Half-to-even on the 8-wide body (ops/utils.hpp:207): 0.5->0, 1.5->2, 2.5->2, 3.5->4."""
    z = np.load(os.path.join(golden_dir, "q4fc_small_q4_1_g32.npz"))
    assert list(z["codes"][0, 0, :8]) == [127, 0, 2, 2, 0, -2, -2, 4]


@pytest.mark.parametrize("G", [32, 128])
def test_reference_known_answer_construction(oracle, golden_dir, G):
    """ops/test_ops.py:106-149: lossless Q4_1 packing, FC equal to fp32 linear."""
    z = np.load(os.path.join(golden_dir, "known_answer_q4_1.npz"))
    W, x = z["W"], z["x"]
    wq = oracle.restated.pack(W, 1, G)
    assert np.array_equal(wq, z[f"packed_g{G}"])
    assert np.array_equal(oracle.restated.dequant(wq), W)
    y = oracle.restated.fc(x, wq, W.shape[0])
    assert np.array_equal(y, z[f"y_g{G}"])
    assert np.allclose(y, z["linear"])


def test_config1_known_answers(oracle, golden_dir):
    """4096x4096 Q4_1/g32, seed 0: SHA-256 of every stage equals the compiled reference's."""
    rec = json.load(open(os.path.join(golden_dir, "config1_sha256.json")))
    g = torch.Generator().manual_seed(0)
    W = (torch.randn(4096, 4096, generator=g) * 0.02).numpy()
    x = torch.randn(1, 1, 4096, generator=g).numpy()
    assert np.allclose(W[0, :3], rec["W_head"]) and np.allclose(x[0, 0, :3], rec["x_head"])
    wq = oracle.restated.pack(W, 1, 32)
    assert sha(wq) == rec["packed"]
    codes, scales, gsums = oracle.restated.quant_x(x, 32, 1.0)
    assert sha(codes) == rec["codes"] and sha(scales) == rec["scales"] and sha(gsums) == rec["gsums"]
    y = oracle.restated.fc(x, wq, 4096)
    assert sha(y) == rec["y"]
    assert abs(float(y.astype(np.float64).sum()) - rec["y_sum_f64"]) < 1e-9


@pytest.mark.parametrize("qtype,G", VARIANTS)
def test_restatement_matches_compiled_reference_live(oracle, qtype, G):
    """When oracle/_ref exists on this machine, compare on fresh seeded inputs."""
    if not oracle.have_compiled_reference(qtype, G):
        pytest.skip("compiled reference not built on this machine")
    ref = oracle.compiled_reference(qtype, G)
    g = torch.Generator().manual_seed(4242 + qtype * 7 + G)
    W = (torch.randn(160, 1024, generator=g) * 0.02).numpy()
    x = torch.randn(1, 8, 1024, generator=g).numpy()
    wq = oracle.restated.pack(W, qtype, G)
    assert np.array_equal(wq, ref.pack(W))
    for a, b in zip(oracle.restated.quant_x(x, G, 1.0 if qtype else 1 / 16), ref.quant_x(x)):
        assert np.array_equal(a.reshape(b.shape), b)
    if ref.exact_int_dot:
        assert np.array_equal(oracle.restated.fc(x, wq, 160), ref.fc(x, wq, 160))


def test_q4_0_reads_nibble_unsigned(oracle):
    """The reference's Q4_0 dequant / FC ignore the nibble's sign (ops/op_fc.hpp:95-106)."""
    g = torch.Generator().manual_seed(5)
    W = (torch.randn(32, 64, generator=g) * 0.02).numpy()
    wq = oracle.restated.pack(W, 0, 32)
    as_ref = oracle.restated.dequant(wq)
    signed = oracle.restated.dequant(wq, nibble_signed=True)
    assert np.abs(signed - W).max() < 0.01          # the corrected reading reconstructs W
    assert np.abs(as_ref - W).max() > 0.05          # the reference's does not
    assert (as_ref >= 0).all()


def test_fp16_conversion_round_to_nearest_even(oracle):
    vals = np.concatenate([np.float32([0, -0.0, 1, 65504, 65519.99, 65520, 1e-8, 5.96e-8, 6.1e-5, 3.0e-5]),
                           np.random.default_rng(0).standard_normal(2000).astype(np.float32) * 0.01])
    want = vals.astype(np.float16).view(np.uint16)
    got = np.array([oracle.restated.f16_bits(float(v)) for v in vals], dtype=np.uint16)
    assert np.array_equal(got, want)
    back = np.array([oracle.restated.f16_value(int(b)) for b in want], dtype=np.float32)
    assert np.array_equal(back, want.view(np.float16).astype(np.float32))


def test_ragged_shapes(oracle):
    """N not a multiple of 32 and K not a multiple of the group: padding is zero."""
    g = torch.Generator().manual_seed(9)
    N, K, G = 40, 72, 32
    W = (torch.randn(N, K, generator=g) * 0.02).numpy()
    x = torch.randn(1, 2, K, generator=g).numpy()
    wq = oracle.restated.pack(W, 1, G)
    assert wq.shape == (2, 3, 640)
    deq = oracle.restated.dequant(wq)
    assert np.abs(deq[:N, :K] - W).max() < 0.01
    assert np.all(deq[N:, :] == 0)
    codes, scales, gsums = oracle.restated.quant_x(x, G)
    assert codes.shape == (1, 2, 96) and np.all(codes[..., K:] == 0)
    y = oracle.restated.fc(x, wq, N)
    # same problem padded to full blocks: extra columns are independent; padding a K group
    # with the group's own minimum (and x with zeros) changes neither min/max, codes nor sums
    W2 = np.zeros((64, 96), np.float32)
    W2[:N, :K] = W
    W2[:N, K:] = W[:, 64:K].min(axis=1, keepdims=True)
    W2[N:] = 0.01
    x2 = np.zeros((1, 2, 96), np.float32)
    x2[..., :K] = x
    y2 = oracle.restated.fc(x2, oracle.restated.pack(W2, 1, G), 64)
    assert np.array_equal(y, y2[..., :N])


def test_empty_inputs(oracle):
    assert oracle.restated.pack(np.zeros((0, 64), np.float32), 1, 32).shape == (0, 2, 640)
    c, s, gs = oracle.restated.quant_x(np.zeros((0, 64), np.float32), 32)
    assert c.shape == (0, 64) and s.shape == (0, 2)


def test_rmsnorm_restatement_matches_the_reference_rows():
    """Rows returned by the reference's own llmops.rmsnorm (fixture from its compiled module): bit-equal."""
    import numpy as np

    from oracle import cpu

    f = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "rmsnorm_ref.npz"))
    for i in range(int(f["cases"])):
        got = cpu.restated.rmsnorm(f[f"x{i}"], f[f"w{i}"], float(f[f"eps{i}"]))
        assert np.array_equal(got, f[f"y{i}"]), i
    with pytest.raises(RuntimeError):
        cpu.restated.rmsnorm(np.zeros((1, 1, 12), np.float32), np.ones(12, np.float32), 1e-5)  # K % 8 != 0


def test_silu_mul_restatement_against_reference_rows(oracle, golden_dir):
    """up * silu(gate) as restated (polynomial exp of ops/utils.hpp:293-371, exact reciprocal) against the rows the
    reference's own module returned: its _mm256_rcp_ps is approximate, so the match is to tolerance, not bits."""
    d = np.load(os.path.join(golden_dir, "silu_mul_ref.npz"))
    for i in range(int(d["cases"])):
        got = oracle.restated.silu_mul(d[f"gate{i}"], d[f"up{i}"])
        ref = d[f"prod{i}"]
        assert np.allclose(got, ref, rtol=1e-3, atol=1e-4), (i, np.abs(got - ref).max())
        big = np.abs(ref) > 1e-3
        assert (np.abs(got - ref)[big] / np.abs(ref)[big]).max() < 5e-4


def test_q8c_restatement_is_bit_equal_to_the_reference(oracle, golden_dir):
    """FC_quant_Q8C / FC_evaluate_Q8C (ext/llama_ext.cpp:56-113, 232-371) and embedding_q8c_quant_w / embedding_q8c
    (ops/op_embedding.hpp:51-137) as restated, against what the reference's own compiled code returned."""
    d = np.load(os.path.join(golden_dir, "q8c_ref.npz"))
    r = oracle.restated
    for i in range(int(d["fc_cases"])):
        wq, ws = r.q8c_pack(d[f"W{i}"])
        assert np.array_equal(wq, d[f"wq{i}"]) and np.array_equal(ws, d[f"ws{i}"]), i
        y = r.q8c_fc(d[f"x{i}"], wq, ws, d[f"W{i}"].shape[0])
        assert np.array_equal(y, d[f"y{i}"]), (i, np.abs(y - d[f"y{i}"]).max())
    for i in range(int(d["emb_cases"])):
        codes, scales = r.emb_q8c_quant(d[f"table{i}"])
        assert np.array_equal(codes, d[f"codes{i}"]) and np.array_equal(scales, d[f"scales{i}"].ravel()), i
        assert np.array_equal(r.emb_q8c(d[f"ids{i}"], codes, scales), d[f"emb{i}"]), i


def test_q8c_edges_of_the_restatement(oracle):
    r = oracle.restated
    rng = np.random.default_rng(5)
    # a zero column has scale 0 and codes 0; N and K need not fill their last block
    W = rng.standard_normal((40, 70)).astype(np.float32)
    W[7] = 0
    wq, ws = r.q8c_pack(W)
    assert wq.shape == (2, 3, 1024) and ws.shape == (64,)
    assert ws[7] == 0 and np.all(ws[40:] == 0)
    x = rng.standard_normal((1, 2, 70)).astype(np.float32)
    y = r.q8c_fc(x, wq, ws, 40)
    ref = x.reshape(2, 70) @ W.T
    assert np.all(y[0, :, 7] == 0) and np.abs(y[0] - ref).max() < 0.05 * np.abs(ref).max()
    # the table: ties round to even in the 8-wide body and away from zero in the tail
    t = np.array([[127, 0.5, 1.5, 2.5, -0.5, -1.5, 3, 4, 0.5, 2.5, -2.5]], dtype=np.float32)
    codes, scales = r.emb_q8c_quant(t)
    assert scales[0] == 1.0
    assert codes[0].tolist() == [127, 0, 2, 2, 0, -2, 3, 4, 1, 3, -3]
