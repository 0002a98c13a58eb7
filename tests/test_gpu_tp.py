"""N-split tensor parallelism on real GPUs: two NCCL ranks, outputs bit-equal to the single-GPU FC."""
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
                                       (4096, 11008, 8, "q4_1", 32), (32000, 4096, 1, "q4_0", 32)]:
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
