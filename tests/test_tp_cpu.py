"""N-split tensor parallelism of one FC: sharding and gathering logic on CPU ranks (gloo, world size 2)."""
import os
import sys
import tempfile

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_bounds_cover_every_stripe_once():
    import llama_cl_b200 as pkg

    tp = pkg.tp
    for Ng in (1, 2, 7, 128, 344, 1000, 1001):
        for world in (1, 2, 3, 4, 8):
            seen = []
            for r in range(world):
                a, b = tp.shard_bounds(Ng, world, r)
                assert 0 <= a <= b <= Ng
                seen += list(range(a, b))
            assert seen == list(range(Ng))
    # the Llama-7B widths split evenly over 1/2/4/8 GPUs
    for N in (4096, 11008, 32000):
        for world in (1, 2, 4, 8):
            assert ((N + 31) // 32) % world == 0
            sizes = {tp.shard_rows(N, world, r)[1] - tp.shard_rows(N, world, r)[0] for r in range(world)}
            assert sizes == {N // world}


def _worker(rank, world, initfile, N, K, rows, qtype, G, result_q):
    sys.path.insert(0, ROOT)
    dist.init_process_group("gloo", init_method=f"file://{initfile}", rank=rank, world_size=world)
    try:
        import llama_cl_b200 as pkg
        from oracle import cpu

        g = torch.Generator().manual_seed(1234)
        W = torch.randn(N, K, generator=g) * 0.02
        x = torch.randn(1, rows, K, generator=g)
        full = cpu.restated.pack(W.numpy(), qtype, G)
        want = cpu.restated.fc(x.numpy(), full, N)
        # packing only this rank's rows gives this rank's slice of the full packed tensor
        n0, n1 = pkg.tp.shard_rows(N, world, rank)
        mine = cpu.restated.pack(W.numpy()[n0:n1], qtype, G) if n1 > n0 else full[:0]
        shard = pkg.tp.shard_packed(torch.from_numpy(full), world, rank)
        assert np.array_equal(shard.numpy()[: mine.shape[0]], mine[: shard.shape[0]])

        def cpu_fc(inp, wq, n_local, **kw):  # stand-in for the CUDA FC: the CPU checker on this rank's shard
            return torch.from_numpy(cpu.restated.fc(inp.numpy(), wq.numpy(), n_local))

        layer = pkg.tp.TPLinearQ4(shard, N, local_fc=cpu_fc)
        y = layer(x)
        assert y.shape == (1, rows, N)
        # no summation order changes: the gathered output is bit-equal to the unsharded one
        result_q.put((rank, bool(np.array_equal(y.numpy(), want))))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("N,K,rows,qtype,G", [(256, 128, 1, 1, 32), (320, 256, 3, 1, 128), (96, 128, 2, 0, 32),
                                              (100, 64, 2, 1, 32)])
def test_tp_two_ranks_gloo(oracle, N, K, rows, qtype, G):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        initfile = os.path.join(d, "init")
        procs = [ctx.Process(target=_worker, args=(r, world, initfile, N, K, rows, qtype, G, q)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
    got = sorted(q.get(timeout=5) for _ in range(world))
    assert got == [(0, True), (1, True)]
