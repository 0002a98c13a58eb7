"""The chain of dependent decode FCs as one persistent launch (q4fc_fc_chain_*), through the C-ABI on a B200.

Quantization is a step function: a one-ulp difference in an FC's input can flip a code and move the next FC's output
by more than the FC tolerance.  So a chain is checked step by step: every step of the test chain writes buffers of its
own, and after the launch EACH step's outputs are compared with the CPU oracle fed with the GPU's own inputs of that
step.  The per-token stack built on the chain is then compared with the stack of separate launches."""
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
    # the tolerance stated for fp32 FC outputs against the reference's CPU result
    return np.allclose(y, ref, rtol=1e-3, atol=1e-4)


def _layer_chain(ops, g, H, I, V, L_, rows, qname, G):
    """A Llama-shaped chain in which every step has buffers of its own.  Returns (steps, records): records hold, per
    step, what the oracle needs to recompute it."""
    dev = "cuda"

    def mk(N, K):
        return ops.offline_FC_quant_Q4A((torch.randn(N, K, generator=g) * 0.05).cuda(), qtype=qname, group_k=G)

    def buf(N):
        return torch.full((1, rows, N), float("nan"), device=dev)

    x0 = torch.randn(1, rows, H, generator=g).cuda()
    steps, rec = [], []
    h = x0
    for _ in range(L_):
        wn1, wn2 = (torch.rand(H, generator=g) + 0.5).cuda(), (torch.rand(H, generator=g) + 0.5).cuda()
        wq_, wk_, wv_, wo_ = mk(H, H), mk(H, H), mk(H, H), mk(H, H)
        wg_, wu_, wd_ = mk(I, H), mk(I, H), mk(H, I)
        bias = torch.randn(H, generator=g).cuda()
        q, k, v, h1, gate, up, h2 = buf(H), buf(H), buf(H), buf(H), buf(I), buf(I), buf(H)
        steps.append(dict(x=h, transform="rmsnorm", aux=wn1, eps=1e-5, jobs=[(wq_, H, q), (wk_, H, k, bias), (wv_, H, v)]))
        rec.append(("rmsnorm", h, wn1, [(wq_, H, q, None), (wk_, H, k, bias), (wv_, H, v, None)]))
        steps.append(dict(x=q, jobs=[(wo_, H, h1, h)]))
        rec.append(("plain", q, None, [(wo_, H, h1, h)]))
        steps.append(dict(x=h1, transform="rmsnorm", aux=wn2, eps=1e-5, jobs=[(wg_, I, gate), (wu_, I, up)]))
        rec.append(("rmsnorm", h1, wn2, [(wg_, I, gate, None), (wu_, I, up, None)]))
        steps.append(dict(x=gate, transform="silu_mul", aux=up, jobs=[(wd_, H, h2, h1)]))
        rec.append(("silu_mul", gate, up, [(wd_, H, h2, h1)]))
        h = h2
    wl, logits = mk(V, H), buf(V)
    steps.append(dict(x=h, jobs=[(wl, V, logits)]))
    rec.append(("plain", h, None, [(wl, V, logits, None)]))
    return steps, rec, x0, logits


@pytest.mark.parametrize("qname,G", [("q4_1", 128), ("q4_1", 32), ("q4_0", 32), ("q4_0", 128)])
@pytest.mark.parametrize("rows", [1, 3, 8])
def test_chain_steps_against_the_oracle(pkg, oracle, qname, G, rows):
    ops, r = pkg.llmops, oracle.restated
    g = torch.Generator().manual_seed(1000 + rows + G)
    H, I, V = 512, 1408, 5000  # 16, 44 and 157 stripes: fewer than, and more than, one per SM
    steps, rec, x0, logits = _layer_chain(ops, g, H, I, V, 2, rows, qname, G)
    chain = ops.FCChain(steps)
    chain.run()
    chain.check()
    for si, (kind, x, aux, jobs) in enumerate(rec):
        xin = x.cpu().numpy()
        assert np.isfinite(xin).all(), si
        loose = False
        if kind == "rmsnorm":
            a = r.rmsnorm(xin, aux.cpu().numpy(), 1e-5)
        elif kind == "silu_mul":
            # agrees with the reference's formula to ~4e-4 relative (its reciprocal is approximate): codes on a
            # rounding boundary may differ by one step
            a, loose = r.silu_mul(xin, aux.cpu().numpy()), True
        else:
            a = xin
        for (w, N, out, addend) in jobs:
            want = r.fc(a, w.cpu().numpy(), N)
            if addend is not None:
                want = want + addend.cpu().numpy()
            got = out.cpu().numpy()
            if loose:
                assert np.abs(got - want).max() <= 5e-3 * np.abs(want).max(), (si, N)
            else:
                assert close(got, want), (si, N, np.abs(got - want).max())
    # a second launch on a new input: the barrier words, the ring and the buffers start over cleanly, and a launch
    # repeats itself bit for bit
    first = logits.clone()
    x0.copy_(torch.randn(x0.shape, generator=g).cuda())
    chain.run()
    second = logits.clone()
    chain.run()
    chain.check()
    assert torch.equal(second, logits) and not torch.equal(first, second)
    chain.close()


@pytest.mark.parametrize("rows", [1, 4])
def test_stack_on_the_chain(pkg, oracle, rows):
    """DecodeFCStack(chain=True): the per-token schedule as one launch instead of 4 or 8 per layer.  With one layer
    every buffer survives the pass, so each step is checked on its own input; with three layers the logits must stay
    near those of the separate launches (codes flipped by rounding-level differences move a chain by a few percent of
    the logits' scale, no more), and the replayed graph must repeat the eager chain bit for bit."""
    from llama_cl_b200.stack import DecodeFCStack

    ops, r = pkg.llmops, oracle.restated
    H, I, V, L_, G, eps = 512, 1408, 1000, 3, 128, 1e-5
    g = torch.Generator().manual_seed(5 + rows)

    def mk(N, K):
        return ops.offline_FC_quant_Q4A((torch.randn(N, K, generator=g) * 0.05).cuda(), qtype="q4_1", group_k=G)

    layers = [dict(q=mk(H, H), k=mk(H, H), v=mk(H, H), o=mk(H, H), gate=mk(I, H), up=mk(I, H), down=mk(H, I))
              for _ in range(L_)]
    lm = mk(V, H)
    norms = [dict(input=(torch.rand(H, generator=g) + 0.5).cuda(), post=(torch.rand(H, generator=g) + 0.5).cuda())
             for _ in range(L_)]
    fin = (torch.rand(H, generator=g) + 0.5).cuda()
    l0 = {k: v.cpu().numpy() for k, v in layers[0].items()}
    lmn = lm.cpu().numpy()
    n = lambda t: t.cpu().numpy()  # noqa: E731

    # ---- one layer, FC-only schedule
    st = DecodeFCStack(layers[:1], lm, hidden=H, intermediate=I, vocab=V, rows=rows, glue="none", chain=True)
    assert st.launches_per_token == 1
    xx = torch.randn(1, rows, H, generator=g).cuda()
    got = n(st.forward(xx, sync=True))
    st.check()
    for k in ("q", "k", "v"):
        assert close(n(getattr(st, k)), r.fc(n(xx), l0[k], H)), k
    assert close(n(st.h1), r.fc(n(st.q), l0["o"], H))
    assert close(n(st.gate), r.fc(n(st.h1), l0["gate"], I))
    assert close(n(st.up), r.fc(n(st.h1), l0["up"], I))
    assert close(n(st.h2), r.fc(n(st.gate), l0["down"], H))
    assert close(got, r.fc(n(st.h2), lmn, V))

    # ---- one layer, with the norms, the residual adds and silu * up
    st = DecodeFCStack(layers[:1], lm, hidden=H, intermediate=I, vocab=V, rows=rows, glue="llama", norms=norms[:1],
                       final_norm=fin, eps=eps, chain=True)
    got = n(st.forward(xx, sync=True))
    st.check()
    a = r.rmsnorm(n(xx), n(norms[0]["input"]), eps)
    for k in ("q", "k", "v"):
        assert close(n(getattr(st, k)), r.fc(a, l0[k], H)), k
    assert close(n(st.h1), r.fc(n(st.q), l0["o"], H) + n(xx))
    b = r.rmsnorm(n(st.h1), n(norms[0]["post"]), eps)
    assert close(n(st.gate), r.fc(b, l0["gate"], I)) and close(n(st.up), r.fc(b, l0["up"], I))
    want = r.fc(r.silu_mul(n(st.gate), n(st.up)), l0["down"], H) + n(st.h1)
    assert np.abs(n(st.h2) - want).max() <= 5e-3 * np.abs(want).max()
    assert close(got, r.fc(r.rmsnorm(n(st.h2), n(fin), eps), lmn, V))

    # ---- three layers: eager chain == replayed chain, both near the separate launches
    kw = dict(hidden=H, intermediate=I, vocab=V, rows=rows, glue="llama", norms=norms, final_norm=fin, eps=eps)
    ref = DecodeFCStack(layers, lm, graph=False, **kw)
    one = DecodeFCStack(layers, lm, graph=False, chain=True, **kw)
    rep = DecodeFCStack(layers, lm, graph=True, chain=True, **kw)
    for step in range(3):
        x = torch.randn(1, rows, H, generator=g).cuda()
        a_ = ref.forward(x, sync=True).clone()
        b_ = one.forward(x, sync=True).clone()
        c_ = rep.forward(x, sync=True).clone()
        one.check()
        rep.check()
        assert torch.equal(b_, c_), step
        scale = a_.abs().max().item()
        assert (a_ - b_).abs().max().item() <= 0.15 * scale, (step, (a_ - b_).abs().max().item(), scale)

    # ---- with an attention callable the chain is cut in front of every attention call
    def att(q, k, v, layer):
        return q * 0.5 + v * 0.25 + k * 0.125

    ref2 = DecodeFCStack(layers, lm, graph=False, attention=att, **kw)
    cut = DecodeFCStack(layers, lm, graph=True, chain=True, attention=att, **kw)
    assert cut.launches_per_token == L_ + 1
    for step in range(2):
        x = torch.randn(1, rows, H, generator=g).cuda()
        a_ = ref2.forward(x, sync=True).clone()
        b_ = cut.forward(x, sync=True).clone()
        cut.check()
        scale = a_.abs().max().item()
        assert (a_ - b_).abs().max().item() <= 0.15 * scale, (step, (a_ - b_).abs().max().item(), scale)
    # one layer with attention: o reads the attention output, checked on its own input
    c1 = DecodeFCStack(layers[:1], lm, graph=False, chain=True, attention=att, hidden=H, intermediate=I, vocab=V,
                       rows=rows, glue="llama", norms=norms[:1], final_norm=fin, eps=eps)
    c1.forward(xx, sync=True)
    c1.check()
    assert close(n(c1.h1), r.fc(n(att(c1.q, c1.k, c1.v, 0)), l0["o"], H) + n(xx))


def test_chain_argument_checks(pkg):
    ops = pkg.llmops
    W = ops.offline_FC_quant_Q4A(torch.randn(64, 64).cuda(), qtype="q4_1", group_k=32)
    W2 = ops.offline_FC_quant_Q4A(torch.randn(64, 64).cuda(), qtype="q4_0", group_k=32)
    x = torch.randn(1, 2, 64).cuda()
    y = torch.empty(1, 2, 64).cuda()
    with pytest.raises(RuntimeError):
        ops.FCChain([])
    with pytest.raises(RuntimeError):
        ops.FCChain([dict(x=x, jobs=[(W, 64, x)])])  # a job writes the input of its own step
    with pytest.raises(RuntimeError):
        ops.FCChain([dict(x=x, jobs=[(W, 64, y), (W2, 64, y)])])  # two block types
    with pytest.raises(RuntimeError):
        ops.FCChain([dict(x=x, transform="rmsnorm", jobs=[(W, 64, y)])])  # no weight for the norm
    with pytest.raises(RuntimeError):
        ops.FCChain([dict(x=torch.randn(1, 9, 64).cuda(), jobs=[(W, 64, torch.empty(1, 9, 64).cuda())])])  # rows > 8
    W3 = ops.offline_FC_quant_Q4A(torch.randn(64, 36).cuda(), qtype="q4_1", group_k=32)
    with pytest.raises(RuntimeError):
        ops.FCChain([dict(x=torch.randn(1, 2, 36).cuda(), jobs=[(W3, 64, y)])])  # K % 8 != 0
    c = ops.FCChain([dict(x=x, jobs=[(W, 64, y)])])  # a chain of one step is a plain FC
    c.run()
    c.check()
    assert np.allclose(y.cpu().numpy(), ops.fc_Q4A(x, W, 64).cpu().numpy(), rtol=1e-5, atol=1e-6)
