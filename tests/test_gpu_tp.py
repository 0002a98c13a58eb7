"""N-split tensor parallelism on real GPUs: NCCL ranks (two, and -- for boxes with one GPU -- a world of one, where
the peer stores go to the rank's own buffers), outputs checked against the CPU oracle and the single-GPU FC."""
import os
import sys
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, initfile, result_q):
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"file://{initfile}", rank=rank, world_size=world, device_id=dev)
    try:
        import llama_cl_b200 as pkg

        ok = True
        for (N, K, rows, qname, G) in [(4096, 4096, 1, "q4_1", 128), (11008, 4096, 4, "q4_1", 128),
                                       (4096, 11008, 8, "q4_1", 32), (32000, 4096, 1, "q4_0", 32),
                                       (11008, 4096, 192, "q4_0", 32)]:  # the last: prefill kernel per shard
            g = torch.Generator().manual_seed(N + K + rows)
            W = (torch.randn(N, K, generator=g) * 0.02).to(dev)
            x = torch.randn(1, rows, K, generator=g).to(dev)
            full = pkg.llmops.offline_FC_quant_Q4A(W, qtype=qname, group_k=G)
            layer = pkg.tp.TPLinearQ4.from_full_weight(W, qtype=qname, group_k=G)
            # packing only this rank's rows reproduces this rank's slice of the full packed tensor
            ok &= torch.equal(layer.weight, pkg.tp.shard_packed(full, world, rank))
            y = layer(x)
            # every stripe is computed by the same kernel arithmetic wherever it lives: compare with the
            # single-GPU result column by column within the FC tolerance, and across ranks bit for bit
            want = pkg.llmops.fc_Q4A(x, full, N)
            ok &= bool(torch.allclose(y, want, rtol=1e-3, atol=1e-4))
            other = [torch.empty_like(y) for _ in range(world)]
            dist.all_gather(other, y.contiguous())
            ok &= all(torch.equal(o, y) for o in other)
        result_q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_tp_two_gpus_nccl(lib_built):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        procs = [ctx.Process(target=_worker, args=(r, world, os.path.join(d, "init"), q)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(300)
            assert p.exitcode == 0
    assert sorted(q.get(timeout=5) for _ in range(world)) == [(0, True), (1, True)]


def _fused_worker(rank, world, initfile, result_q):
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"file://{initfile}", rank=rank, world_size=world, device_id=dev)
    notes = []
    try:
        import llama_cl_b200 as pkg
        from llama_cl_b200 import tp
        from oracle import build_oracle, cpu

        build_oracle.build_restatement()

        def expect(cond, what):
            if not bool(cond):
                notes.append(what)

        arena = tp.TPArena(32 << 20, dev)
        sched = tp.TPSchedule(arena)
        H, I, NR = 4096, 11008, 4100  # NR: ragged tail (129 stripes: 65 + 64, last one 4 columns wide)
        specs = {"q": (H, H, "q4_1", 128), "k": (H, H, "q4_1", 128), "up": (I, H, "q4_1", 128),
                 "down": (H, I, "q4_1", 32), "last": (NR, H, "q4_0", 32)}
        full, lay = {}, {}
        for i, (name, (N, K, qname, G)) in enumerate(specs.items()):
            g = torch.Generator().manual_seed(100 + i)
            W = (torch.randn(N, K, generator=g) * 0.02).to(dev)
            full[name] = pkg.llmops.offline_FC_quant_Q4A(W, qtype=qname, group_k=G)
            n0, n1 = tp.shard_rows(N, world, rank)
            shard = pkg.llmops.offline_FC_quant_Q4A(W[n0:n1].contiguous(), qtype=qname, group_k=G)
            expect(torch.equal(shard, tp.shard_packed(full[name], world, rank)), f"{name}: shard bytes")
            lay[name] = tp.FusedTPLinearQ4(sched, shard, N, pdl=True)

        def chain(x):
            """q, k side by side -> up(q) -> down -> last; every consumer waits inside its own kernel,
            the unpacking kernels at the end wait for whatever is still in flight."""
            sched.step_begin()
            q = lay["q"](x)
            k = lay["k"](x)
            up = lay["up"](q)
            down = lay["down"](up)
            last = lay["last"](down)
            return {n: o.tensor() for n, o in (("q", q), ("k", k), ("up", up), ("down", down), ("last", last))}

        full_np = {n: w.cpu().numpy() for n, w in full.items()}

        def verify(x, outs, tag, with_oracle=False):
            got = {n: o.clone() for n, o in outs.items()}
            ins = {"q": x, "k": x, "up": got["q"], "down": got["up"], "last": got["down"]}
            for name, (N, K, _, _) in specs.items():
                if with_oracle:
                    # the CPU restatement of the reference's fc_Q4A on the same inputs
                    ref = torch.from_numpy(cpu.restated.fc(ins[name].cpu().numpy(), full_np[name], N)).to(dev)
                    expect(torch.allclose(got[name], ref, rtol=1e-3, atol=1e-4), f"{tag} {name}: differs from the oracle")
                want = pkg.llmops.fc_Q4A(ins[name].contiguous(), full[name], N)
                expect(got[name].shape == want.shape, f"{tag} {name}: shape {tuple(got[name].shape)}")
                expect(torch.allclose(got[name], want, rtol=1e-3, atol=1e-4), f"{tag} {name}: differs from one GPU")
                # a column is computed by exactly one rank and stored everywhere: ranks agree bit for bit
                other = [torch.empty_like(got[name]) for _ in range(world)]
                dist.all_gather(other, got[name].contiguous())
                expect(all(torch.equal(o, got[name]) for o in other), f"{tag} {name}: ranks differ")

        for rows in (1, 4):
            for step in range(3):  # fresh input every step: stale data from the step before would show
                g = torch.Generator().manual_seed(7 * rows + step)
                x = torch.randn(1, rows, H, generator=g).to(dev)
                outs = chain(x)
                torch.cuda.synchronize()
                verify(x, outs, f"rows={rows} step={step}", with_oracle=(step == 0))

        # the same chain replayed as a CUDA graph: the epoch lives on the device, so replays advance it
        xg = torch.zeros(1, 1, H, device=dev)
        side = torch.cuda.Stream(dev)
        with torch.cuda.stream(side):
            chain(xg)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                outs_g = chain(xg)
        torch.cuda.synchronize()
        for step in range(3):
            g = torch.Generator().manual_seed(900 + step)
            xg.copy_(torch.randn(1, 1, H, generator=g))
            graph.replay()
            torch.cuda.synchronize()
            verify(xg, outs_g, f"graph step={step}", with_oracle=(step == 2))
        expect(arena.status() == 0, f"status {arena.status():#x} after the chains")

        # a wait that nothing satisfies gives up after its limit, flags it, and leaves the context usable
        ghost = tp.FusedTPLinearQ4(sched, tp.shard_packed(full["q"], world, rank), H)  # never run
        tp.StampedOutput(ghost, 1, 1).tensor()
        expect(arena.status() == 0x54505754, "the unsatisfied wait did not set the status word")
        arena.tensor(arena.STATUS, (1,), torch.int32).zero_()
        outs = chain(xg)
        torch.cuda.synchronize()
        verify(xg, outs, "after the timed-out wait")
        expect(arena.status() == 0, "status after recovery")

        # a second schedule in the same arena keeps its own step count: a stand-alone FC run twice
        solo = tp.TPSchedule(arena)
        one = tp.FusedTPLinearQ4(solo, tp.shard_packed(full["q"], world, rank), H)
        for step in range(2):
            solo.step_begin()
            y = one(xg).tensor()
            torch.cuda.synchronize()
            want = pkg.llmops.fc_Q4A(xg, full["q"], H)
            expect(torch.allclose(y, want, rtol=1e-3, atol=1e-4), f"solo schedule step {step}")
        # a layer that quantizes its plain input once in front of the kernel: same codes and scales; its kernel
        # splits K over clusters of 4 instead of 8, so the fp32 sums differ in the last bits only
        sq = tp.TPSchedule(arena)
        la = tp.FusedTPLinearQ4(sq, tp.shard_packed(full["up"], world, rank), I, pdl=True)
        lb = tp.FusedTPLinearQ4(sq, tp.shard_packed(full["up"], world, rank), I, pdl=True, prequant=True)
        for M in (1, 8):
            g = torch.Generator().manual_seed(500 + M)
            xm = torch.randn(1, M, H, generator=g).to(dev)
            sq.step_begin()
            ya, yb = la(xm).tensor(), lb(xm).tensor()
            torch.cuda.synchronize()
            expect(torch.allclose(ya, yb, rtol=1e-4, atol=1e-5), f"prequant layer M={M}")

        # several layers per launch: q and k on one (stamped or plain) input, and a batch on pre-quantized inputs,
        # gathered by one unpacking launch
        sm = tp.TPSchedule(arena)
        lq = tp.FusedTPLinearQ4(sm, tp.shard_packed(full["q"], world, rank), H, pdl=True)
        lk = tp.FusedTPLinearQ4(sm, tp.shard_packed(full["k"], world, rank), H, pdl=True)
        lu = tp.FusedTPLinearQ4(sm, tp.shard_packed(full["up"], world, rank), I, pdl=True)
        for M in (1, 3):
            g = torch.Generator().manual_seed(700 + M)
            xm = torch.randn(1, M, H, generator=g).to(dev)
            sm.step_begin()
            oq, ok_ = tp.fused_multi([lq, lk], xm)
            (ou,) = tp.fused_multi([lu], oq)  # reads the stamped output of q
            yq, yk, yu = (torch.empty((1, M, n), device=dev) for n in (H, H, I))
            tp.collect_many([oq, ok_, ou], [yq, yk, yu])
            torch.cuda.synchronize()
            for name, y, xin in (("q", yq, xm), ("k", yk, xm), ("up", yu, yq)):
                ref = torch.from_numpy(cpu.restated.fc(xin.cpu().numpy(), full_np[name], y.shape[-1])).to(dev)
                expect(torch.allclose(y, ref, rtol=1e-3, atol=1e-4), f"fused_multi {name} M={M}: differs from the oracle")
        xqa = pkg.llmops.quantize_activations(torch.randn(1, 2, H, generator=torch.Generator().manual_seed(801)).to(dev), 128)
        xqb = pkg.llmops.quantize_activations(torch.randn(1, 2, H, generator=torch.Generator().manual_seed(802)).to(dev), 128)
        fb = tp.FusedTPBatch([lq, lu], [xqa, xqb])
        for step in range(2):
            sm.step_begin()
            outs_b = fb.run()
            ya, yb = torch.empty((1, 2, H), device=dev), torch.empty((1, 2, I), device=dev)
            tp.collect_many(outs_b, [ya, yb])
            torch.cuda.synchronize()
            expect(torch.allclose(ya, pkg.llmops.fc_Q4A_q8(xqa, full["q"], H), rtol=1e-3, atol=1e-4), f"FusedTPBatch q step {step}")
            expect(torch.allclose(yb, pkg.llmops.fc_Q4A_q8(xqb, full["up"], I), rtol=1e-3, atol=1e-4), f"FusedTPBatch up step {step}")
        expect(arena.status() == 0, f"status {arena.status():#x} after the batched launches")

        # host buffers in and out over the N-split FC, as a replayed graph, two row counts, fresh inputs
        hf = tp.HostFusedFC(arena, tp.shard_packed(full["up"], world, rank), I, max_rows=4, pdl=True)
        for step in range(3):
            for M in (1, 4):
                g = torch.Generator().manual_seed(300 + 10 * step + M)
                xh = torch.randn(1, M, H, generator=g)
                y = hf(xh).clone()
                want = pkg.llmops.fc_Q4A(xh.to(dev), full["up"], I).cpu()
                expect(torch.allclose(y, want, rtol=1e-3, atol=1e-4), f"HostFusedFC step {step} M={M}")
        # a fixed batch of host-buffer FCs over one pinned block each way (copies pipelined per launch), three row
        # counts, five members in two of them: every output against the oracle, replayed with fresh inputs
        mem = [("q", 1), ("up", 1), ("k", 3), ("q", 8), ("up", 8), ("k", 8), ("down", 8), ("last", 8)]
        same = [m for m in mem if specs[m[0]][2:] == ("q4_1", 128)]  # one block type per batch object
        hb = tp.HostFusedBatch(arena, [(tp.shard_packed(full[nm], world, rank), specs[nm][0], M) for nm, M in same])
        for step in range(2):
            xs = []
            for i, (nm, M) in enumerate(same):
                g = torch.Generator().manual_seed(900 + 20 * step + i)
                xs.append(torch.randn(1, M, specs[nm][1], generator=g))
            ys = hb(xs)
            for (nm, M), xh, y in zip(same, xs, ys):
                ref = torch.from_numpy(cpu.restated.fc(xh.numpy(), full_np[nm], specs[nm][0]))
                expect(torch.allclose(y, ref, rtol=1e-3, atol=1e-4), f"HostFusedBatch {nm} M={M} step {step}")
        # the per-token FC schedule over N-split weights as a package class: one layer + lm_head, replayed as a graph,
        # against the single-GPU stack on the full weights (same codes; the sums may meet in another order)
        from llama_cl_b200.stack import DecodeFCStack, FusedTPDecodeFCStack

        Hs, Is, Vs = 512, 1408, 1000
        gs_ = torch.Generator().manual_seed(4242)
        fullw = {k: pkg.llmops.offline_FC_quant_Q4A((torch.randn(n_, k_, generator=gs_) * 0.05).to(dev), qtype="q4_1",
                                                    group_k=128)
                 for k, (n_, k_) in dict(q=(Hs, Hs), k=(Hs, Hs), v=(Hs, Hs), o=(Hs, Hs), gate=(Is, Hs), up=(Is, Hs),
                                         down=(Hs, Is), lm=(Vs, Hs)).items()}
        shard = {k: tp.shard_packed(w, world, rank) for k, w in fullw.items()}
        ref_stack = DecodeFCStack([{k: fullw[k] for k in ("q", "k", "v", "o", "gate", "up", "down")}], fullw["lm"],
                                  hidden=Hs, intermediate=Is, vocab=Vs, rows=2, glue="none")
        tp_stack = FusedTPDecodeFCStack(arena, [{k: shard[k] for k in ("q", "k", "v", "o", "gate", "up", "down")}],
                                        shard["lm"], hidden=Hs, intermediate=Is, vocab=Vs, rows=2)
        for step in range(3):
            xt = torch.randn(1, 2, Hs, generator=gs_).to(dev)
            want_l = ref_stack.forward(xt, sync=True)
            got_l = tp_stack.forward(xt, sync=True)
            scale_l = want_l.abs().max().item()
            expect((want_l - got_l).abs().max().item() <= 0.02 * scale_l, f"FusedTPDecodeFCStack step {step}")
        outs = chain(xg)  # and the first schedule is undisturbed by it
        torch.cuda.synchronize()
        verify(xg, outs, "after the solo schedule")
        expect(arena.status() == 0, "status at the end")
        arena.close()
        result_q.put((rank, notes))
    except Exception as e:  # report instead of leaving the parent to time out
        import traceback

        result_q.put((rank, notes + [traceback.format_exc()]))
    finally:
        dist.destroy_process_group()


def test_tp_two_gpus_fused_peer_stores(lib_built):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        procs = [ctx.Process(target=_fused_worker, args=(r, world, os.path.join(d, "init"), q)) for r in range(world)]
        for p in procs:
            p.start()
        results = sorted(q.get(timeout=280) for _ in range(world))
        for p in procs:
            p.join(60)
            if p.exitcode is None:
                p.kill()  # exactly the processes started above
    assert results == [(0, []), (1, [])], results


def test_tp_fused_world_of_one(lib_built):
    """The whole fused N-split path on ONE GPU: arena, step barrier, stamped peer stores (to the rank's own
    buffers), stamped inputs, unpacking kernel, graph replay, and a bounded wait that runs out and recovers --
    each FC checked against the CPU oracle."""
    assert torch.cuda.is_available()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        p = ctx.Process(target=_fused_worker, args=(0, 1, os.path.join(d, "init"), q))
        p.start()
        results = [q.get(timeout=280)]
        p.join(60)
        if p.exitcode is None:
            p.kill()  # exactly the process started above
    assert results == [(0, [])], results
