"""CUDA path vs the CPU oracle and the reference's golden vectors, through the C-ABI.

Bars: bit-exact for packed weights, dequantized weights, Q8 codes, scales and
group sums; FC outputs within rtol 1e-3 / atol 1e-4 of the reference's CPU FC
(the tolerance stated for this path), in practice ~1e-6.
"""
import hashlib
import json
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

VARIANTS = [(0, 32), (0, 128), (1, 32), (1, 128)]
QNAME = {0: "q4_0", 1: "q4_1"}
RTOL, ATOL = 1e-3, 1e-4


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.fixture(scope="module")
def pkg(lib_built):
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    import llama_cl_b200

    return llama_cl_b200


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def close(y, ref):
    return np.allclose(y, ref, rtol=RTOL, atol=ATOL)


# ---------------------------------------------------------------- packer ----
@pytest.mark.parametrize("qtype,G", VARIANTS)
def test_pack_golden(pkg, oracle, golden_dir, qtype, G):
    z = np.load(os.path.join(golden_dir, f"q4fc_small_{oracle.variant_name(qtype, G)}.npz"))
    wq = pkg.llmops.offline_FC_quant_Q4A(dev(z["W"]), qtype=QNAME[qtype], group_k=G)
    assert np.array_equal(wq.cpu().numpy(), z["packed"])
    deq = pkg.llmops.offline_FC_dequant_Q4A(wq)
    assert np.array_equal(deq.cpu().numpy(), z["dequant"])


def test_pack_config1_sha(pkg, oracle, golden_dir):
    rec = json.load(open(os.path.join(golden_dir, "config1_sha256.json")))
    g = torch.Generator().manual_seed(0)
    W = torch.randn(4096, 4096, generator=g) * 0.02
    x = torch.randn(1, 1, 4096, generator=g)
    wq = pkg.llmops.offline_FC_quant_Q4A(W.cuda())
    assert tuple(wq.shape) == (128, 128, 640)
    assert sha(wq.cpu().numpy()) == rec["packed"]
    codes, scales, gsums = pkg.llmops.FC_dynamic_quantize_x(x.cuda(), 32, 1.0)
    assert sha(codes.cpu().numpy()) == rec["codes"]
    assert sha(scales.cpu().numpy()) == rec["scales"]
    assert sha(gsums.cpu().numpy()) == rec["gsums"]
    y = pkg.llmops.fc_Q4A(x.cuda(), wq, 4096).cpu().numpy()
    want = oracle.restated.fc(x.numpy(), wq.cpu().numpy(), 4096)
    assert sha(want) == rec["y"]
    assert close(y, want) and np.allclose(y[0, 0, :4], rec["y_head"], rtol=RTOL, atol=ATOL)
    assert abs(float(y.astype(np.float64).sum()) - rec["y_sum_f64"]) < 1e-2


@pytest.mark.parametrize("qtype,G", VARIANTS)
@pytest.mark.parametrize("N,K", [(32, 128), (96, 640), (40, 200), (33, 36), (1000, 4096 + 128)])
def test_pack_vs_oracle_shapes(pkg, oracle, qtype, G, N, K):
    g = torch.Generator().manual_seed(N * 31 + K)
    W = torch.randn(N, K, generator=g) * 0.02
    W[0, : min(K, 40)] = 0.0          # an all-zero group
    if N > 1:
        W[1, :8] = torch.tensor([0.0, -0.0, 0.0, 0.0, -0.0, 0.0, 0.0, 0.0])  # zero-sign ties
        W[1, 8:G] = 0.0
    want = oracle.restated.pack(W.numpy(), qtype, G)
    got = pkg.llmops.offline_FC_quant_Q4A(W.cuda(), qtype=QNAME[qtype], group_k=G).cpu().numpy()
    assert got.shape == want.shape
    assert np.array_equal(got, want)
    for signed in (False, True):
        d_want = oracle.restated.dequant(want, nibble_signed=signed)
        d_got = pkg.llmops.offline_FC_dequant_Q4A(dev(want), nibble_signed=signed).cpu().numpy()
        assert np.array_equal(d_got, d_want)


def test_pack_negative_zero_minimum(pkg, oracle):
    """get_min_max keeps the FIRST of equal values: a group of (-0, +0, ...) stores m = -0."""
    W = np.zeros((32, 32), np.float32)
    W[0, 0] = -0.0
    W[1, 1] = -0.0          # +0 first, -0 later: m = +0
    W[2, :] = -0.0
    for q in (0, 1):
        want = oracle.restated.pack(W, q, 32)
        got = pkg.llmops.offline_FC_quant_Q4A(dev(W), qtype=QNAME[q], group_k=32).cpu().numpy()
        assert np.array_equal(got, want)


def test_known_answer_construction(pkg, golden_dir):
    """ops/test_ops.py:106-149: Q4_1 packing lossless, FC == fp32 linear, zero tolerance."""
    z = np.load(os.path.join(golden_dir, "known_answer_q4_1.npz"))
    W, x = dev(z["W"]), dev(z["x"])
    for G in (32, 128):
        wq = pkg.llmops.offline_FC_quant_Q4A(W, group_k=G)
        assert np.array_equal(wq.cpu().numpy(), z[f"packed_g{G}"])
        assert np.array_equal(pkg.llmops.offline_FC_dequant_Q4A(wq).cpu().numpy(), z["W"])
        y = pkg.llmops.fc_Q4A(x, wq, W.shape[0]).cpu().numpy()      # rows = 10 -> prefill path
        assert np.array_equal(y, z["linear"])
        y8 = pkg.llmops.fc_Q4A(x[:, :4].contiguous(), wq, W.shape[0]).cpu().numpy()  # rows = 8 -> decode
        assert np.array_equal(y8, z["linear"][:, :4])


def test_known_answer_full_size(pkg):
    """Same construction at the reference's own test size B=2, M=17, N=K=4096 (all sums exact in fp32)."""
    g = torch.Generator().manual_seed(11)
    N = K = 4096
    w = torch.randint(-8, 8, (N, K), generator=g).float()
    x = torch.randint(-127, 128, (2, 17, K), generator=g).float()
    w[:, 0::32] = -8
    w[:, 1::32] = 7
    x[:, :, 0::32] = -127
    x[:, :, 1::32] = 127
    w, x = (w / 128).cuda(), (x / 128).cuda()
    ref = torch.nn.functional.linear(x.double(), w.double()).float()
    for G in (32, 128):
        wq = pkg.llmops.offline_FC_quant_Q4A(w, group_k=G)
        assert torch.equal(pkg.llmops.offline_FC_dequant_Q4A(wq), w)
        assert torch.equal(pkg.llmops.fc_Q4A(x, wq, N), ref)
        assert torch.equal(pkg.llmops.fc_Q4A(x[:1, :5].contiguous(), wq, N), ref[:1, :5])


# ------------------------------------------------------------- quantizer ----
@pytest.mark.parametrize("G", [32, 128])
@pytest.mark.parametrize("rows,K", [(1, 4096), (8, 11008), (5, 200), (3, 36), (64, 1024), (1, 32)])
def test_quant_x_bit_exact(pkg, oracle, G, rows, K):
    g = torch.Generator().manual_seed(rows * 131 + K + G)
    x = torch.randn(1, rows, K, generator=g)
    x[0, 0, : min(K, 8)] = torch.tensor([127, .5, 1.5, 2.5, -.5, -1.5, -2.5, 3.5])[: min(K, 8)]
    if rows > 1:
        x[0, 1, :G] = 0.0
    for scale in (1.0, 1.0 / 16):
        c0, s0, g0 = oracle.restated.quant_x(x.numpy(), G, scale)
        c1, s1, g1 = pkg.llmops.FC_dynamic_quantize_x(x.cuda(), G, scale)
        assert np.array_equal(c1.cpu().numpy(), c0)
        assert np.array_equal(s1.cpu().numpy(), s0)
        assert np.array_equal(g1.cpu().numpy(), g0)


@pytest.mark.parametrize("qtype,G", VARIANTS)
def test_quant_x_golden(pkg, oracle, golden_dir, qtype, G):
    z = np.load(os.path.join(golden_dir, f"q4fc_small_{oracle.variant_name(qtype, G)}.npz"))
    c, s, gs = pkg.llmops.FC_dynamic_quantize_x(dev(z["x"]), G, 1.0 if qtype else 1.0 / 16)
    assert np.array_equal(c.cpu().numpy(), z["codes"])
    assert np.array_equal(s.cpu().numpy(), z["scales"])
    assert np.array_equal(gs.cpu().numpy(), z["gsums"])


# -------------------------------------------------------------------- FC ----
@pytest.mark.parametrize("qtype,G", VARIANTS)
def test_fc_golden(pkg, oracle, golden_dir, qtype, G):
    z = np.load(os.path.join(golden_dir, f"q4fc_small_{oracle.variant_name(qtype, G)}.npz"))
    y = pkg.llmops.fc_Q4A(dev(z["x"]), dev(z["packed"]), int(z["N"])).cpu().numpy()
    assert y.shape == z["y"].shape
    assert close(y, z["y"])
    assert np.abs(y - z["y"]).max() < 2e-5


@pytest.mark.parametrize("path", ["decode", "streamk"])
@pytest.mark.parametrize("qtype,G", VARIANTS)
@pytest.mark.parametrize("rows", [1, 2, 3, 4, 7, 8])
@pytest.mark.parametrize("N,K", [(32, 128), (4096, 4096), (160, 1280), (352, 11008), (2080, 640)])
def test_fc_decode_vs_oracle(pkg, oracle, path, qtype, G, rows, N, K):
    g = torch.Generator().manual_seed(N + 7 * K + rows)
    W = torch.randn(N, K, generator=g) * 0.02
    x = torch.randn(1, rows, K, generator=g)
    wq = oracle.restated.pack(W.numpy(), qtype, G)
    want = oracle.restated.fc(x.numpy(), wq, N)
    got = pkg.llmops.fc_Q4A(x.cuda(), dev(wq), N, path=path).cpu().numpy()
    assert close(got, want), np.abs(got - want).max()
    assert np.abs(got - want).max() <= 1e-5 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("K,N", [(4096, 4096), (4096, 11008), (11008, 4096), (4096, 32000)])
@pytest.mark.parametrize("rows", [1, 2, 4, 8])
def test_fc_decode_llama7b_shapes_q4_1_g128(pkg, oracle, K, N, rows):
    """The decode sweep the benchmark runs: Q4_1 group 128 over the Llama-7B FC shapes."""
    g = torch.Generator().manual_seed(K * 3 + N + rows)
    W = torch.randn(N, K, generator=g) * 0.02
    x = torch.randn(1, rows, K, generator=g)
    wq_gpu = pkg.llmops.offline_FC_quant_Q4A(W.cuda(), group_k=128)
    wq = oracle.restated.pack(W.numpy(), 1, 128)
    assert np.array_equal(wq_gpu.cpu().numpy(), wq)
    want = oracle.restated.fc(x.numpy(), wq, N)
    got = pkg.llmops.fc_Q4A(x.cuda(), wq_gpu, N).cpu().numpy()
    assert close(got, want), np.abs(got - want).max()


@pytest.mark.parametrize("qtype,G", [(0, 32), (0, 128)])
def test_fc_q4_0_signed_option(pkg, oracle, qtype, G):
    g = torch.Generator().manual_seed(77 + G)
    W = torch.randn(64, 512, generator=g) * 0.02
    x = torch.randn(1, 3, 512, generator=g)
    wq = oracle.restated.pack(W.numpy(), qtype, G)
    want = oracle.restated.fc(x.numpy(), wq, 64, nibble_signed=True)
    got = pkg.llmops.fc_Q4A(x.cuda(), dev(wq), 64, nibble_signed=True).cpu().numpy()
    assert close(got, want)
    # and the corrected reading is the one that approximates the fp32 product
    lin = x.numpy() @ W.numpy().T
    assert np.abs(got - lin).max() < 0.15 * np.abs(lin).max()


def test_fc_repeatable_and_workspace_reuse(pkg, oracle):
    """Back-to-back calls share one workspace; results are bit-identical run to run."""
    g = torch.Generator().manual_seed(3)
    W = torch.randn(4096, 4096, generator=g) * 0.02
    wq = pkg.llmops.offline_FC_quant_Q4A(W.cuda(), group_k=128)
    x = torch.randn(1, 4, 4096, generator=g).cuda()
    for path in ("decode", "streamk"):
        y0 = pkg.llmops.fc_Q4A(x, wq, 4096, path=path)
        for _ in range(5):
            assert torch.equal(pkg.llmops.fc_Q4A(x, wq, 4096, path=path), y0)
    # an explicit workspace, reused by calls of both kernels one after the other: every call must leave it
    # ready for the next (the stream-K kernel returns its stripe counters to zero), or results would drift
    ws = pkg.llmops.Workspace(pkg._cabi.lib().q4fc_fc_workspace_bytes(4, 4096, 4096, 1, 128), x.device)
    for i in range(6):
        path = ("streamk", "decode")[i & 1]
        assert torch.equal(pkg.llmops.fc_Q4A(x, wq, 4096, path=path, workspace=ws),
                           pkg.llmops.fc_Q4A(x, wq, 4096, path=path))
    ws.check()


def test_fc_workspace_shared_between_shapes(pkg, oracle):
    """One workspace serves interleaved calls of different N (fixed layout)."""
    g = torch.Generator().manual_seed(4)
    shapes = [(64, 256), (4096, 4096), (32, 128), (11008, 4096)]
    ws = pkg.llmops.Workspace(pkg._cabi.lib().q4fc_fc_workspace_bytes(8, 4096, 11008, 1, 128), torch.device("cuda"))
    cases = []
    for N, K in shapes:
        W = torch.randn(N, K, generator=g) * 0.02
        x = torch.randn(1, 3, K, generator=g)
        wq = oracle.restated.pack(W.numpy(), 1, 128)
        cases.append((x.cuda(), dev(wq), N, oracle.restated.fc(x.numpy(), wq, N)))
    for _ in range(2):
        for x, wq, N, want in cases:
            got = pkg.llmops.fc_Q4A(x, wq, N, workspace=ws, path="streamk").cpu().numpy()
            assert close(got, want), (N, np.abs(got - want).max())


def test_fc_pdl_chain(pkg, oracle):
    """A chain launched with programmatic stream serialization gives the same results."""
    g = torch.Generator().manual_seed(21)
    Ws = [(torch.randn(4096, 4096, generator=g) * 0.02).cuda() for _ in range(3)]
    wqs = [pkg.llmops.offline_FC_quant_Q4A(w, group_k=128) for w in Ws]
    x = torch.randn(1, 1, 4096, generator=g).cuda()
    plain = []
    h = x
    for wq in wqs:
        h = pkg.llmops.fc_Q4A(h, wq, 4096)
        plain.append(h)
    # under programmatic serialization the kernel takes half of the CTA slots, so its fp32 sums are
    # ordered differently: each layer, fed the plain chain's input, agrees within tolerance, and the
    # PDL chain is bit-equal from run to run
    inputs = [x] + plain[:-1]
    first = None
    for _ in range(3):
        outs = []
        for i, wq in enumerate(wqs):   # back-to-back PDL launches, each reading the previous launch's output buffer
            outs.append(pkg.llmops.fc_Q4A(inputs[i], wq, 4096, pdl=True))
        for i in range(3):
            assert close(outs[i].cpu().numpy(), plain[i].cpu().numpy())
        h = x
        chain = []
        for wq in wqs:
            h = pkg.llmops.fc_Q4A(h, wq, 4096, pdl=True)
            chain.append(h)
        if first is None:
            first = chain
        else:
            assert all(torch.equal(a, b) for a, b in zip(chain, first))
    for i, wq in enumerate(wqs):
        got = pkg.llmops.fc_Q4A(inputs[i], wq, 4096, pdl=True, path="streamk")
        assert close(got.cpu().numpy(), plain[i].cpu().numpy())


@pytest.mark.parametrize("qtype,G", VARIANTS)
def test_fc_many_rows(pkg, oracle, qtype, G):
    g = torch.Generator().manual_seed(5 + G)
    N, K = 320, 1024
    W = torch.randn(N, K, generator=g) * 0.02
    x = torch.randn(2, 17, K, generator=g)
    wq = oracle.restated.pack(W.numpy(), qtype, G)
    want = oracle.restated.fc(x.numpy(), wq, N)
    got = pkg.llmops.fc_Q4A(x.cuda(), dev(wq), N).cpu().numpy()
    assert got.shape == (2, 17, N)
    assert close(got, want), np.abs(got - want).max()


@pytest.mark.parametrize("qtype,G", VARIANTS)
@pytest.mark.parametrize("rows,N,K", [(9, 32, 128), (130, 416, 1024), (256, 128, 4096), (300, 1000, 640), (5, 96, 256)])
def test_fc_prefill_vs_oracle(pkg, oracle, qtype, G, rows, N, K):
    """The tensor-core kernel on tile edges: partial row / column tiles, few and many K stages."""
    g = torch.Generator().manual_seed(rows + 3 * N + 7 * K + G)
    W = torch.randn(N, K, generator=g) * 0.02
    x = torch.randn(1, rows, K, generator=g)
    wq = oracle.restated.pack(W.numpy(), qtype, G)
    want = oracle.restated.fc(x.numpy(), wq, N)
    got = pkg.llmops.fc_Q4A(x.cuda(), dev(wq), N, path="prefill").cpu().numpy()
    assert close(got, want), np.abs(got - want).max()
    assert np.abs(got - want).max() <= 2e-5 * max(1.0, np.abs(want).max())
    pkg.llmops.fc_workspace(rows, K, N, qtype, G, torch.device("cuda")).check()   # no wait ran out


def test_fc_prefill_q4_0_signed(pkg, oracle):
    g = torch.Generator().manual_seed(78)
    W = torch.randn(160, 512, generator=g) * 0.02
    x = torch.randn(1, 40, 512, generator=g)
    for G in (32, 128):
        wq = oracle.restated.pack(W.numpy(), 0, G)
        want = oracle.restated.fc(x.numpy(), wq, 160, nibble_signed=True)
        got = pkg.llmops.fc_Q4A(x.cuda(), dev(wq), 160, nibble_signed=True, path="prefill").cpu().numpy()
        assert close(got, want), np.abs(got - want).max()


def test_fc_prefill_config3_q4_0_g32(pkg, oracle):
    """The prefill configuration of the baseline: Q4_0 group 32, M=512, K=4096, N=11008 (reference semantics)."""
    g = torch.Generator().manual_seed(33)
    N, K, M = 11008, 4096, 512
    W = torch.randn(N, K, generator=g) * 0.02
    x = torch.randn(1, M, K, generator=g)
    wq_gpu = pkg.llmops.offline_FC_quant_Q4A(W.cuda(), qtype="q4_0", group_k=32)
    wq = oracle.restated.pack(W.numpy(), 0, 32)
    assert np.array_equal(wq_gpu.cpu().numpy(), wq)
    got = pkg.llmops.fc_Q4A(x.cuda(), wq_gpu, N).cpu().numpy()
    rows = [0, 1, 127, 128, 300, 511]          # the oracle on a sample of rows keeps the test short
    want = oracle.restated.fc(x.numpy()[:, rows], wq, N)
    assert close(got[:, rows], want), np.abs(got[:, rows] - want).max()
    # every row against the decode kernel (same arithmetic, different machinery)
    for r0 in range(0, M, 8):
        ref8 = pkg.llmops.fc_Q4A(x[:, r0:r0 + 8].cuda().contiguous(), wq_gpu, N, path="decode").cpu().numpy()
        assert close(got[:, r0:r0 + 8], ref8)


def test_fc_ragged_n_and_k(pkg, oracle):
    g = torch.Generator().manual_seed(9)
    N, K, G = 40, 72, 32
    W = torch.randn(N, K, generator=g) * 0.02
    x = torch.randn(1, 2, K, generator=g)
    wq = pkg.llmops.offline_FC_quant_Q4A(W.cuda(), group_k=G)
    assert np.array_equal(wq.cpu().numpy(), oracle.restated.pack(W.numpy(), 1, G))
    want = oracle.restated.fc(x.numpy(), wq.cpu().numpy(), N)
    got = pkg.llmops.fc_Q4A(x.cuda(), wq, N).cpu().numpy()
    assert close(got, want)


def test_scaling_by_power_of_two_is_exact(pkg):
    """Size-independent property at a full Llama-7B shape: y(4x) == 4 y(x) bit for bit."""
    g = torch.Generator().manual_seed(1)
    W = (torch.randn(11008, 4096, generator=g) * 0.02).cuda()
    wq = pkg.llmops.offline_FC_quant_Q4A(W, group_k=128)
    x = torch.randn(1, 8, 4096, generator=g).cuda()
    assert torch.equal(pkg.llmops.fc_Q4A(x * 4, wq, 11008), pkg.llmops.fc_Q4A(x, wq, 11008) * 4)


def test_wrappers(pkg, oracle):
    """Old-extension names and the per-Linear callable of the reference model."""
    g = torch.Generator().manual_seed(2)
    lin = torch.nn.Linear(256, 96, bias=True)
    with torch.no_grad():
        lin.weight.copy_(torch.randn(96, 256, generator=g) * 0.02)
        lin.bias.copy_(torch.randn(96, generator=g))
    x = torch.randn(1, 3, 256, generator=g)
    wq = oracle.restated.pack(lin.weight.detach().numpy(), 1, 32)
    want = oracle.restated.fc(x.numpy(), wq, 96)
    op = pkg.llmop_fc_q4a(lin)
    assert op.N == 96 and repr(op) == "llmop_fc_q4a(weight: [3, 8, 640])"
    assert op.weight_size() == 3 * 8 * 640 + 96 * 4
    assert close(op(x.cuda()).cpu().numpy(), want + lin.bias.detach().numpy())
    fc = pkg.c_ext.FCQ4A(lin.weight.detach().cuda())
    assert repr(fc) == "FCQ4A()" and fc._N == 96
    assert np.array_equal(fc._weight.cpu().numpy(), wq)
    assert close(fc.forward(x.cuda()).cpu().numpy(), want)
    assert close(pkg.c_ext.FC_evaluate_Q4A(x.cuda(), pkg.c_ext.FC_quant_Q4A(lin.weight.detach().cuda()), 96)
                 .cpu().numpy(), want)


def test_errors_on_gpu(pkg):
    x = torch.zeros(1, 1, 64, device="cuda")
    wq = torch.zeros(1, 2, 640, dtype=torch.int8, device="cuda")
    with pytest.raises(RuntimeError, match="does not match"):
        pkg.llmops.fc_Q4A(torch.zeros(1, 1, 100, device="cuda"), wq, 32)
    with pytest.raises(RuntimeError, match="exceeds"):
        pkg.llmops.fc_Q4A(x, wq, 64)
    with pytest.raises(RuntimeError, match="none of"):
        pkg.llmops.fc_Q4A(x, torch.zeros(1, 2, 600, dtype=torch.int8, device="cuda"), 32)
    with pytest.raises(RuntimeError, match="contiguous"):
        pkg.llmops.fc_Q4A(torch.zeros(1, 64, 2, device="cuda").transpose(1, 2), wq, 32)
    assert pkg.llmops.fc_Q4A(x[:, :0], wq, 32).shape == (1, 0, 32)


def test_full_layer_pack_matches_oracle(pkg, oracle):
    """One Llama-7B layer's FC set at full size, group 32 and 128: packed bytes bit-equal."""
    shapes = [(4096, 4096)] * 4 + [(11008, 4096)] * 2 + [(4096, 11008)]
    for i, (N, K) in enumerate(shapes):
        g = torch.Generator().manual_seed(100 + i)
        W = torch.randn(N, K, generator=g) * 0.02
        Wd = W.cuda()
        for G in (32, 128):
            got = pkg.llmops.offline_FC_quant_Q4A(Wd, group_k=G).cpu().numpy()
            assert sha(got) == sha(oracle.restated.pack(W.numpy(), 1, G))


def test_host_fc_graph_and_streams(lib_built):
    """HostFC: host buffers in and out; the captured-graph form and the eager form give the same bytes as
    the device-side call, for every row count, across repeated calls with fresh inputs."""
    import llama_cl_b200 as pkg
    from llama_cl_b200.host import HostFC

    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(5)
    N, K = 1000, 1024
    W = (torch.randn(N, K, generator=g) * 0.02).to(dev)
    wq = pkg.llmops.offline_FC_quant_Q4A(W, qtype="q4_1", group_k=128)
    hg = HostFC(wq, N, max_rows=8, path="decode")
    he = HostFC(wq, N, max_rows=8, graph=False, path="decode", stream=torch.cuda.Stream(dev))
    for it in range(3):
        for M in (1, 3, 8):
            x = torch.randn(1, M, K, generator=g)
            want = pkg.llmops.fc_Q4A(x.to(dev), wq, N, path="decode").cpu()
            assert torch.equal(hg(x).clone(), want)
            assert torch.equal(he(x.pin_memory()).clone(), want)
            stage = hg.x_staging(M)
            stage.copy_(x * 2)
            y = hg(stage, sync=False)
            hg.stream.synchronize()
            assert torch.equal(y, pkg.llmops.fc_Q4A((x * 2).to(dev), wq, N, path="decode").cpu())
    with pytest.raises(RuntimeError):
        hg(torch.zeros(1, 9, K))


@pytest.mark.parametrize("qname,q,G,signed", [("q4_1", 1, 128, False), ("q4_1", 1, 32, False), ("q4_0", 0, 32, False),
                                              ("q4_0", 0, 128, True)])
def test_decode_prequantized_path_equals_fused_quantizer(lib_built, qname, q, G, signed):
    """For large rows x K the decode entry point quantizes the activations in a launch of its own (when the
    workspace has room for the codes) instead of inside the FC kernel.  Both quantizers follow the same
    rules in the same order, so the outputs are bit-identical; without a workspace the fused one runs."""
    import llama_cl_b200 as pkg

    L = pkg._cabi.lib()
    g = torch.Generator().manual_seed(77)
    s = torch.cuda.current_stream().cuda_stream
    flags = 1 if signed else 0
    for (N, K, rows) in [(4096, 11008, 8), (1000, 11008, 4), (640, 6152, 8), (96, 8192, 6)]:
        W = (torch.randn(N, K, generator=g) * 0.02).cuda()
        wq = pkg.llmops.offline_FC_quant_Q4A(W, qtype=qname, group_k=G)
        Ng, Kg, _ = wq.shape
        x = torch.randn(1, rows, K, generator=g).cuda()
        nbytes = int(L.q4fc_fc_workspace_bytes(rows, K, N, q, G))
        ws = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        outs = []
        for w in (None, ws, ws):  # the second pass over the same scratch finds it used
            y = torch.full((1, rows, N), float("nan"), device="cuda")
            rc = L.q4fc_fc_decode(x.data_ptr(), rows, K, K, wq.data_ptr(), Ng, Kg, q, G, N, y.data_ptr(), N,
                                  w.data_ptr() if w is not None else None, nbytes if w is not None else 0, flags, s)
            assert rc == 0, L.q4fc_last_error()
            outs.append(y)
        torch.cuda.synchronize()
        assert rows * K >= 40 * 1024  # the sizes above are meant to take the separate launch
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2]), (N, K, rows)
        want = pkg.llmops.fc_Q4A(x, wq, N, path="streamk", nibble_signed=signed)
        assert torch.allclose(outs[1], want, rtol=1e-3, atol=1e-4)


def test_host_fc_group(lib_built):
    """Several host-buffer FCs submitted as one replayed graph over their own streams: same bytes as the
    one-by-one calls, for changing inputs and for a second combination of row counts."""
    import llama_cl_b200 as pkg
    from llama_cl_b200.host import HostFC, HostFCGroup

    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(6)
    shapes = [(1000, 1024), (512, 2048), (96, 1024)]
    wqs = [pkg.llmops.offline_FC_quant_Q4A((torch.randn(N, K, generator=g) * 0.02).to(dev), qtype="q4_1", group_k=128)
           for N, K in shapes]
    streams = [torch.cuda.Stream(dev), torch.cuda.Stream(dev)]
    members = [HostFC(wq, N, max_rows=8, path="decode", stream=streams[i % 2],
                      workspace=pkg.llmops.Workspace(pkg._cabi.lib().q4fc_fc_workspace_bytes(8, K, N, 1, 128), dev))
               for i, (wq, (N, K)) in enumerate(zip(wqs, shapes))]
    group = HostFCGroup(members)
    for Ms in [(1, 4, 8), (1, 4, 8), (2, 2, 1), (1, 4, 8)]:
        xs = [torch.randn(1, M, K, generator=g) for M, (N, K) in zip(Ms, shapes)]
        ys = [y.clone() for y in group(xs)]
        for y, x, wq, (N, K) in zip(ys, xs, wqs, shapes):
            assert torch.equal(y, pkg.llmops.fc_Q4A(x.to(dev), wq, N, path="decode").cpu())
    with pytest.raises(RuntimeError):
        group([torch.zeros(1, 1, 1024)])


@pytest.mark.parametrize("qname,G,signed", [("q4_1", 128, False), ("q4_1", 32, False), ("q4_0", 32, True)])
def test_quantize_once_then_several_fcs(lib_built, qname, G, signed):
    """quantize_activations + fc_Q4A_q8: codes and scales bit-equal to the oracle's quantizer, FC outputs the
    same bytes as fc_Q4A on the fp32 input, for several FCs sharing one quantized input."""
    import llama_cl_b200 as pkg
    from oracle import cpu

    g = torch.Generator().manual_seed(31)
    for rows, K in [(1, 4096), (8, 1024), (3, 1160)]:  # the last: ragged final group
        x = torch.randn(1, rows, K, generator=g)
        xq = pkg.llmops.quantize_activations(x.cuda(), G, nibble_signed=signed)
        scale = 1.0 if qname == "q4_1" else 1 / 16
        c0, s0, g0 = cpu.restated.quant_x(x.numpy(), G, 1.0)
        assert np.array_equal(xq.codes().cpu().numpy(), c0.reshape(rows, -1))
        sc, gs = xq.scales_and_sums()
        assert np.array_equal(sc.cpu().numpy(), s0.reshape(rows, -1))
        if not signed:
            assert np.allclose(gs.cpu().numpy(), g0.reshape(rows, -1), rtol=1e-5, atol=1e-5)  # tree-ordered sums
        for N in (96, 1000):
            W = (torch.randn(N, K, generator=g) * 0.02).cuda()
            wq = pkg.llmops.offline_FC_quant_Q4A(W, qtype=qname, group_k=G)
            want = pkg.llmops.fc_Q4A(x.cuda(), wq, N, path="decode", nibble_signed=signed,
                                     workspace=pkg.llmops.Workspace(4096, torch.device("cuda")))
            got = pkg.llmops.fc_Q4A_q8(xq, wq, N)
            assert torch.equal(got, want), (rows, K, N, scale)
    with pytest.raises(RuntimeError):
        pkg.llmops.quantize_activations(torch.zeros(1, 9, 256, device="cuda"), G)


def test_rmsnorm_quantize_matches_the_reference_rows(lib_built):
    """rmsnorm fused with the quantizer: normalized rows bit-equal to the reference's llmops.rmsnorm (fixture
    from its compiled module), codes and scales bit-equal to quantizing those rows, and the FC behind it the
    same bytes as the two-step path."""
    import llama_cl_b200 as pkg
    from oracle import cpu

    f = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "rmsnorm_ref.npz"))
    g = torch.Generator().manual_seed(32)
    for i in range(int(f["cases"])):
        x, w, eps, y = f[f"x{i}"], f[f"w{i}"], float(f[f"eps{i}"]), f[f"y{i}"]
        rows, K = x.shape[1], x.shape[2]
        for G in (32, 128):
            if K % G:
                continue
            xd = torch.from_numpy(x).cuda()
            normalized = torch.empty_like(xd)
            xq = pkg.llmops.rmsnorm_quantize(xd, torch.from_numpy(w).cuda(), eps, G, normalized=normalized)
            assert torch.equal(xd.cpu(), torch.from_numpy(x))  # the input is left alone
            assert np.array_equal(normalized.cpu().numpy(), y), (i, G)
            c0, s0, _ = cpu.restated.quant_x(y, G, 1.0)
            assert np.array_equal(xq.codes().cpu().numpy(), c0.reshape(rows, -1))
            assert np.array_equal(xq.scales_and_sums()[0].cpu().numpy(), s0.reshape(rows, -1))
            # without the normalized output the quantized result is the same
            xq2 = pkg.llmops.rmsnorm_quantize(xd, torch.from_numpy(w).cuda(), eps, G)
            assert torch.equal(xq2.codes(), xq.codes())  # (the buffers' padding bytes are never written)
            assert all(torch.equal(a, b) for a, b in zip(xq2.scales_and_sums(), xq.scales_and_sums()))
            W = (torch.randn(160, K, generator=g) * 0.02).cuda()
            wq = pkg.llmops.offline_FC_quant_Q4A(W, qtype="q4_1", group_k=G)
            want = pkg.llmops.fc_Q4A(torch.from_numpy(y).cuda(), wq, 160, path="decode",
                                     workspace=pkg.llmops.Workspace(4096, torch.device("cuda")))
            assert torch.equal(pkg.llmops.fc_Q4A_q8(xq, wq, 160), want)
    # residual addition in front of the norm (llmops.iadd + clone + rmsnorm in the reference's layer)
    x, w, eps = f["x1"], f["w1"], float(f["eps1"])
    res = torch.randn(x.shape, generator=g).numpy()
    summed = (x + res).astype(np.float32)
    want_rows = cpu.restated.rmsnorm(summed, w, eps)
    xd, rd = torch.from_numpy(x).cuda(), torch.from_numpy(res).cuda()
    normalized, sum_out = torch.empty_like(xd), torch.empty_like(xd)
    xq = pkg.llmops.rmsnorm_quantize(xd, torch.from_numpy(w).cuda(), eps, 128, residual=rd, sum_out=sum_out,
                                     normalized=normalized)
    assert np.array_equal(sum_out.cpu().numpy(), summed) and np.array_equal(normalized.cpu().numpy(), want_rows)
    c0, _, _ = cpu.restated.quant_x(want_rows, 128, 1.0)
    assert np.array_equal(xq.codes().cpu().numpy(), c0.reshape(x.shape[1], -1))
    pkg.llmops.rmsnorm_quantize(xd, torch.from_numpy(w).cuda(), eps, 128, residual=rd, sum_out=rd)  # in place
    assert np.array_equal(rd.cpu().numpy(), summed)
    with pytest.raises(RuntimeError):
        pkg.llmops.rmsnorm_quantize(torch.zeros(1, 1, 12, device="cuda"), torch.ones(12, device="cuda"), 1e-5, 32)


@pytest.mark.parametrize("qname,G", [("q4_1", 128), ("q4_0", 32)])
def test_fc_decode_with_addend(lib_built, qname, G):
    """Bias or residual folded into the decode kernel: the same bytes as the FC followed by one fp32 add
    (the reference's llmops.iadd), also in place on the output and behind the separate quantizing launch."""
    import llama_cl_b200 as pkg

    g = torch.Generator().manual_seed(41)
    for rows, K, N in [(1, 4096, 1000), (8, 1024, 96), (4, 11008, 160)]:
        W = (torch.randn(N, K, generator=g) * 0.02).cuda()
        wq = pkg.llmops.offline_FC_quant_Q4A(W, qtype=qname, group_k=G)
        x = torch.randn(1, rows, K, generator=g).cuda()
        bias = torch.randn(N, generator=g).cuda()
        res = torch.randn(1, rows, N, generator=g).cuda()
        plain = pkg.llmops.fc_Q4A(x, wq, N, path="decode")
        assert torch.equal(pkg.llmops.fc_Q4A(x, wq, N, addend=bias), plain + bias)
        assert torch.equal(pkg.llmops.fc_Q4A(x, wq, N, addend=res), plain + res)
        inplace = res.clone()
        pkg.llmops.fc_Q4A(x, wq, N, addend=inplace, out=inplace)  # hidden = fc(x) + hidden
        assert torch.equal(inplace, plain + res)

        import types

        lin = types.SimpleNamespace(weight=W, bias=bias)  # what llmop_fc_q4a takes: .weight, .bias
        op = pkg.ops.llmop_fc_q4a(lin, qtype=qname, group_k=G)
        assert torch.equal(op(x), plain + bias)
    with pytest.raises(RuntimeError):
        pkg.llmops.fc_Q4A(x, wq, N, addend=torch.zeros(N + 1, device="cuda"))
