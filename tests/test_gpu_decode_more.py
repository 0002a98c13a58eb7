"""Decode-path entry points beyond the single call: several weights per launch, batches of independent FCs,
silu(gate) * up fused with the quantizer, the per-token FC schedule, and a few argument checks.  Everything goes
through the C-ABI (ctypes) on a B200 and is compared with the CPU oracle."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pkg(lib_built):
    assert torch.cuda.is_available(), "these tests need a CUDA device; there is no CPU path"
    import llama_cl_b200 as p

    p._cabi.lib()
    return p


def close(y, ref):
    # the tolerance the task states for fp32 outputs against the reference's CPU FC
    return np.allclose(y, ref, rtol=1e-3, atol=1e-4)


@pytest.mark.parametrize("qname,G", [("q4_1", 128), ("q4_1", 32), ("q4_0", 32), ("q4_0", 128)])
@pytest.mark.parametrize("rows", [1, 3, 8])
def test_several_weights_on_one_input(pkg, oracle, qname, G, rows):
    """q4fc_fc_decode_multi: the q/k/v (or gate/up) pattern -- one input, several weight tensors, one launch --
    on fp32 input and on pre-quantized input, with a bias on one job; every output against the oracle."""
    ops = pkg.llmops
    g = torch.Generator().manual_seed(11 * rows + G)
    K, Ns = 1024, [4096, 1000, 96, 40]
    Ws = [torch.randn(N, K, generator=g) * 0.02 for N in Ns]
    wqs = [ops.offline_FC_quant_Q4A(W.cuda(), qtype=qname, group_k=G) for W in Ws]
    x = torch.randn(1, rows, K, generator=g)
    bias = torch.randn(Ns[1], generator=g)
    want = [oracle.restated.fc(x.numpy(), w.cpu().numpy(), N) for w, N in zip(wqs, Ns)]
    want[1] = want[1] + bias.numpy()
    outs = ops.fc_Q4A_multi(x.cuda(), wqs, Ns, addends=[None, bias.cuda(), None, None])
    xq = ops.quantize_activations(x.cuda(), G)
    outs_q = ops.fc_Q4A_multi(xq, wqs, Ns, addends=[None, bias.cuda(), None, None], pdl=True)
    torch.cuda.synchronize()
    for i in range(len(Ns)):
        assert close(outs[i].cpu().numpy(), want[i]), (i, np.abs(outs[i].cpu().numpy() - want[i]).max())
        assert close(outs_q[i].cpu().numpy(), want[i]), i


def test_batch_of_independent_fcs(pkg, oracle):
    """q4fc_fc_decode_batch: calls with different inputs, K, row counts and widths in one launch; two calls share
    an input.  Every output against the oracle, twice in a row (the launch leaves nothing behind)."""
    ops = pkg.llmops
    g = torch.Generator().manual_seed(5)
    spec = [(4096, 4096, 1), (1024, 11008, 8), (11008, 320, 4), (4096, 1000, 2), (256, 32, 3), (4096, 2080, 1)]
    calls, wants = [], []
    shared = None
    for i, (K, N, rows) in enumerate(spec):
        W = torch.randn(N, K, generator=g) * 0.02
        wq = ops.offline_FC_quant_Q4A(W.cuda(), qtype="q4_1", group_k=128)
        if i == 5:
            xq, x = shared  # the same input as call 0
        else:
            x = torch.randn(1, rows, K, generator=g)
            xq = ops.quantize_activations(x.cuda(), 128)
            if i == 0:
                shared = (xq, x)
        calls.append((xq, wq, N))
        wants.append(oracle.restated.fc(x.numpy(), wq.cpu().numpy(), N))
    fb = ops.FCBatch(calls, pdl=True)
    for _ in range(2):
        for o in fb.outs:
            o.fill_(float("nan"))
        outs = fb.run()
        torch.cuda.synchronize()
        for i, (o, w) in enumerate(zip(outs, wants)):
            assert close(o.cpu().numpy(), w), (i, np.abs(o.cpu().numpy() - w).max())
    L = pkg._cabi.lib()
    assert L.q4fc_fc_check_status(None, torch.cuda.current_stream().cuda_stream) == 0, L.q4fc_last_error()


def test_batch_of_the_sweep_shapes(pkg, oracle):
    """The decode sweep of the baseline as four launches (one per row count): Llama-7B shapes, Q4_1 group 128."""
    ops = pkg.llmops
    g = torch.Generator().manual_seed(6)
    shapes = [(4096, 4096), (4096, 11008), (11008, 4096), (4096, 32000)]
    wqs = {sh: ops.offline_FC_quant_Q4A((torch.randn(sh[1], sh[0], generator=g) * 0.02).cuda(), qtype="q4_1", group_k=128)
           for sh in shapes}
    wq_np = {sh: w.cpu().numpy() for sh, w in wqs.items()}
    for M in (1, 2, 4, 8):
        xs = {sh: torch.randn(1, M, sh[0], generator=g) for sh in shapes}
        fb = ops.FCBatch([(ops.quantize_activations(xs[sh].cuda(), 128), wqs[sh], sh[1]) for sh in shapes])
        outs = fb.run()
        torch.cuda.synchronize()
        for sh, o in zip(shapes, outs):
            want = oracle.restated.fc(xs[sh].numpy(), wq_np[sh], sh[1])
            assert close(o.cpu().numpy(), want), (sh, M)


def test_silu_mul_quantize(pkg, oracle, golden_dir):
    """silu(gate) * up + quantizer: products within the output tolerance of the rows the REFERENCE's own module
    returned (fixture) and of the oracle; codes, scales and sums exactly those of the quantizer on the products."""
    ops = pkg.llmops
    d = np.load(os.path.join(golden_dir, "silu_mul_ref.npz"))
    for i in range(int(d["cases"])):
        gate, up, ref = d[f"gate{i}"], d[f"up{i}"], d[f"prod{i}"]
        for G in (32, 128):
            prod = torch.empty(gate.shape, device="cuda")
            xq = ops.silu_mul_quantize(torch.from_numpy(gate).cuda(), torch.from_numpy(up).cuda(), G, product=prod)
            torch.cuda.synchronize()
            got = prod.cpu().numpy()
            assert np.allclose(got, ref, rtol=1e-3, atol=1e-4), (i, G, np.abs(got - ref).max())
            assert np.allclose(got, oracle.restated.silu_mul(gate, up), rtol=1e-3, atol=1e-4)
            # exact quantization of the GPU's own products
            codes, scales, _ = oracle.restated.quant_x(got, G)
            assert np.array_equal(xq.codes().cpu().numpy().reshape(codes.shape), codes)
            sc, _ = xq.scales_and_sums()
            assert np.array_equal(sc.cpu().numpy().reshape(scales.shape), scales)
            # and the same bytes as quantizing those products with the stand-alone quantizer
            xq2 = ops.quantize_activations(prod, G)
            assert torch.equal(xq.codes(), xq2.codes())
            for a, b in zip(xq.scales_and_sums(), xq2.scales_and_sums()):
                assert torch.equal(a, b)


@pytest.mark.parametrize("rows", [1, 4])
def test_token_schedule_against_the_oracle(pkg, oracle, rows):
    """stack.DecodeFCStack: the chained per-token pass (rmsnorm, q/k/v, o + residual, rmsnorm, gate/up, silu*up,
    down + residual, ..., final norm, lm_head).  Quantization is a step function, so a difference of one ulp in
    an FC's input can flip a code and move the next FC's output by far more than the FC tolerance: a chain cannot
    be compared end to end at 1e-3.  So the eager pass records every buffer, and EACH step is checked against the
    CPU oracle fed with the GPU's own inputs of that step, in the chain's order; the replayed graph must then
    reproduce the eager pass bit for bit, and the whole chain must stay near the all-oracle chain."""
    from llama_cl_b200.stack import DecodeFCStack

    ops, r = pkg.llmops, oracle.restated
    H, I, V, L_, G, eps = 512, 1408, 1000, 3, 128, 1e-5
    g = torch.Generator().manual_seed(77)

    def mk(N, K):
        return ops.offline_FC_quant_Q4A((torch.randn(N, K, generator=g) * 0.05).cuda(), qtype="q4_1", group_k=G)

    layers = [dict(q=mk(H, H), k=mk(H, H), v=mk(H, H), o=mk(H, H), gate=mk(I, H), up=mk(I, H), down=mk(H, I))
              for _ in range(L_)]
    lm = mk(V, H)
    norms = [dict(input=(torch.rand(H, generator=g) + 0.5).cuda(), post=(torch.rand(H, generator=g) + 0.5).cuda())
             for _ in range(L_)]
    fin = (torch.rand(H, generator=g) + 0.5).cuda()
    lnp = [{k: v.cpu().numpy() for k, v in l.items()} for l in layers]
    nnp = [{k: v.cpu().numpy() for k, v in n.items()} for n in norms]
    seen = {}
    st = DecodeFCStack(layers, lm, hidden=H, intermediate=I, vocab=V, rows=rows, glue="llama", norms=norms,
                       final_norm=fin, eps=eps, graph=False, tap=lambda n, i, t: seen.__setitem__((n, i), t.cpu().numpy()))
    x = torch.randn(1, rows, H, generator=g)
    logits = st.forward(x.cuda(), sync=True).cpu().numpy()
    for i in range(L_):
        xin = seen[("x", i)]
        a = r.rmsnorm(xin, nnp[i]["input"], eps)
        for n in ("q", "k", "v"):
            assert close(seen[(n, i)], r.fc(a, lnp[i][n], H)), (n, i)
        assert close(seen[("h1", i)], r.fc(seen[("q", i)], lnp[i]["o"], H) + xin), ("o", i)
        b = r.rmsnorm(seen[("h1", i)], nnp[i]["post"], eps)
        assert close(seen[("gate", i)], r.fc(b, lnp[i]["gate"], I)), ("gate", i)
        assert close(seen[("up", i)], r.fc(b, lnp[i]["up"], I)), ("up", i)
        m = r.silu_mul(seen[("gate", i)], seen[("up", i)])
        # silu * up agrees with the reference's formula to ~4e-4 relative (its reciprocal is approximate); codes that
        # sit on a rounding boundary may differ by one step, which the down projection turns into a few 1e-3 of
        # its output scale
        want = r.fc(m, lnp[i]["down"], H) + seen[("h1", i)]
        assert np.abs(seen[("h2", i)] - want).max() <= 5e-3 * np.abs(want).max(), ("down", i)
    want = r.fc(r.rmsnorm(seen[("h2", L_ - 1)], fin.cpu().numpy(), eps), lm.cpu().numpy(), V)
    assert close(logits, want)
    # the replayed graph (programmatic launches, fixed buffers) reproduces the eager pass bit for bit, on fresh inputs
    stg = DecodeFCStack(layers, lm, hidden=H, intermediate=I, vocab=V, rows=rows, glue="llama", norms=norms,
                        final_norm=fin, eps=eps)
    for step in range(3):
        xs = torch.randn(1, rows, H, generator=g).cuda()
        a_ = st.forward(xs, sync=True).clone()
        b_ = stg.forward(xs, sync=True).clone()
        assert torch.equal(a_, b_), step
    # the whole chain stays near the chain computed by the oracle alone (codes flipped by one-ulp differences move
    # it by a few percent of the logits' scale, no more)
    h = x.numpy()
    for l, nw in zip(lnp, nnp):
        q = r.fc(r.rmsnorm(h, nw["input"], eps), l["q"], H)
        o = r.fc(q, l["o"], H) + h
        b = r.rmsnorm(o, nw["post"], eps)
        h = r.fc(r.silu_mul(r.fc(b, l["gate"], I), r.fc(b, l["up"], I)), l["down"], H) + o
    chain = r.fc(r.rmsnorm(h, fin.cpu().numpy(), eps), lm.cpu().numpy(), V)
    assert np.abs(logits - chain).max() <= 0.15 * np.abs(chain).max()
    # the FC-only schedule: with one layer every buffer survives the pass, and each FC is checked on its own input
    st2 = DecodeFCStack(layers[:1], lm, hidden=H, intermediate=I, vocab=V, rows=rows, glue="none")
    xx = torch.randn(1, rows, H, generator=g).cuda()
    got = st2.forward(xx, sync=True).cpu().numpy()
    l0 = lnp[0]
    for n in ("q", "k", "v"):
        assert close(getattr(st2, n).cpu().numpy(), r.fc(xx.cpu().numpy(), l0[n], H)), n
    assert close(st2.h1.cpu().numpy(), r.fc(st2.q.cpu().numpy(), l0["o"], H))
    assert close(st2.gate.cpu().numpy(), r.fc(st2.h1.cpu().numpy(), l0["gate"], I))
    assert close(st2.up.cpu().numpy(), r.fc(st2.h1.cpu().numpy(), l0["up"], I))
    assert close(st2.h2.cpu().numpy(), r.fc(st2.gate.cpu().numpy(), l0["down"], H))
    assert close(got, r.fc(st2.h2.cpu().numpy(), lm.cpu().numpy(), V))


def test_host_fc_batch(pkg, oracle):
    """host.HostFCBatch: one copy in, quantizers, grouped FCs, one copy out; fresh inputs on every replay."""
    from llama_cl_b200.host import HostFCBatch

    ops = pkg.llmops
    g = torch.Generator().manual_seed(9)
    spec = [(1024, 4096, 1), (1024, 352, 8), (2048, 96, 1), (4096, 640, 4)]
    wqs = [ops.offline_FC_quant_Q4A((torch.randn(N, K, generator=g) * 0.02).cuda(), qtype="q4_1", group_k=128)
           for K, N, _ in spec]
    hb = HostFCBatch([(w, N, rows) for w, (K, N, rows) in zip(wqs, spec)])
    for step in range(3):
        xs = [torch.randn(1, rows, K, generator=g) for K, N, rows in spec]
        ys = hb(xs)
        for x, y, w, (K, N, rows) in zip(xs, ys, wqs, spec):
            assert close(y.numpy(), oracle.restated.fc(x.numpy(), w.cpu().numpy(), N)), (step, K, N, rows)
    assert hb.h2d_bytes() == 4 * sum(r * K for K, _, r in spec) and hb.d2h_bytes() == 4 * sum(r * N for _, N, r in spec)


def test_prefill_config3_m2048(pkg, oracle):
    """The larger prefill configuration of the baseline: Q4_0 group 32, M=2048, K=4096, N=11008 (reference
    semantics: unsigned nibble).  Rows from every one of the sixteen 128-row tiles against the oracle, every row
    against the decode kernel."""
    g = torch.Generator().manual_seed(34)
    N, K, M = 11008, 4096, 2048
    W = torch.randn(N, K, generator=g) * 0.02
    x = torch.randn(1, M, K, generator=g)
    wq_gpu = pkg.llmops.offline_FC_quant_Q4A(W.cuda(), qtype="q4_0", group_k=32)
    wq = wq_gpu.cpu().numpy()
    got = pkg.llmops.fc_Q4A(x.cuda(), wq_gpu, N).cpu().numpy()
    rows = sorted({128 * t + o for t in range(16) for o in (0, 127)} | {5, 1000, 2047})
    want = oracle.restated.fc(x.numpy()[:, rows], wq, N)
    assert close(got[:, rows], want), np.abs(got[:, rows] - want).max()
    xg = x.cuda()
    for r0 in range(0, M, 8):
        ref8 = pkg.llmops.fc_Q4A(xg[:, r0:r0 + 8].contiguous(), wq_gpu, N, path="decode").cpu().numpy()
        assert close(got[:, r0:r0 + 8], ref8), r0


def test_signed_activations_only_serve_q4_0(pkg):
    ops = pkg.llmops
    x = torch.randn(1, 2, 256, device="cuda")
    w1 = ops.offline_FC_quant_Q4A(torch.randn(64, 256, device="cuda"), qtype="q4_1", group_k=32)
    xq = ops.quantize_activations(x, 32, nibble_signed=True)
    with pytest.raises(RuntimeError, match="Q4_0 weights only"):
        ops.fc_Q4A_q8(xq, w1, 64)
    with pytest.raises(RuntimeError, match="Q4_0 weights only"):
        ops.fc_Q4A_multi(xq, [w1], [64])


def test_streamk_counts_the_stripes_of_the_packed_tensor(pkg, oracle):
    """The first N columns of a wider packed tensor (Ng > ceil(N/32)), N not a multiple of 32: the stream-K kernel
    keeps a counter per stripe of the tensor, so the workspace is sized and checked from Ng."""
    ops, L = pkg.llmops, pkg._cabi.lib()
    g = torch.Generator().manual_seed(3)
    W = torch.randn(320, 512, generator=g) * 0.02
    wq = ops.offline_FC_quant_Q4A(W.cuda(), qtype="q4_1", group_k=32)
    x = torch.randn(1, 3, 512, generator=g)
    N = 72
    want = oracle.restated.fc(x.numpy(), wq.cpu().numpy()[:3], N)
    y = torch.empty((1, 3, N), device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    small = torch.zeros(int(L.q4fc_fc_workspace_bytes(3, 512, N, 1, 32)), dtype=torch.uint8, device="cuda")
    big = torch.zeros(int(L.q4fc_fc_workspace_bytes(3, 512, 320, 1, 32)), dtype=torch.uint8, device="cuda")
    args = (x.cuda().data_ptr(), 3, 512, 512, wq.data_ptr(), 10, 16, 1, 32, N, y.data_ptr(), N)
    xg = x.cuda()
    args = (xg.data_ptr(), 3, 512, 512, wq.data_ptr(), 10, 16, 1, 32, N, y.data_ptr(), N)
    assert L.q4fc_fc_decode(*args, big.data_ptr(), big.numel(), 4, s) == 0, L.q4fc_last_error()
    torch.cuda.synchronize()
    assert close(y.cpu().numpy(), want)
    if small.numel() < big.numel():
        assert L.q4fc_fc_decode(*args, small.data_ptr(), small.numel(), 4, s) == 4  # Q4FC_EWORKSPACE
    got = torch.empty_like(y)
    args2 = (xg.data_ptr(), 3, 512, 512, wq.data_ptr(), 10, 16, 1, 32, N, got.data_ptr(), N)
    assert L.q4fc_fc_decode_noalloc(*args2, 0, s) == 0, L.q4fc_last_error()
    torch.cuda.synchronize()
    assert close(got.cpu().numpy(), want)


def test_quantize_batch_equals_single_launches(pkg):
    """q4fc_quant_x_q8_batch: several inputs quantized by one launch -- codes, scales and sums bit-equal to one
    q4fc_quant_x_q8 launch per input, for both group sizes, ragged K and different row counts."""
    ops = pkg.llmops
    g = torch.Generator().manual_seed(31)
    for G in (32, 128):
        xs = [torch.randn(1, M, K, generator=g).cuda() for M, K in ((1, 4096), (8, 11008), (3, 72), (2, 1000), (5, 128))]
        outs = [ops.QuantizedActivations(1, x.shape[1], x.shape[2], G, False, x.device) for x in xs]
        for o in outs:
            o.buf.fill_(0x55)
        qb = ops.QuantizeBatch(list(zip(xs, outs)))
        qb.run()
        for x, o in zip(xs, outs):
            ref = ops.quantize_activations(x, G)
            assert torch.equal(o.codes(), ref.codes())
            a, b = o.scales_and_sums(), ref.scales_and_sums()
            assert all(torch.equal(p, q) for p, q in zip(a, b)) if isinstance(a, (tuple, list)) else torch.equal(a, b)
    with pytest.raises(RuntimeError):
        ops.QuantizeBatch([])
    with pytest.raises(RuntimeError):
        ops.QuantizeBatch([(xs[0], outs[1])])  # shapes do not fit
