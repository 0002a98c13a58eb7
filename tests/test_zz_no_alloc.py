"""The allocation-free decode entry point, checked against the ordinary one.

Collected last on purpose (file name): a run that stops at the first failure
has then already run every other test.

Who needs this entry point: a host program that has given all device memory
to its own arena (or works under a fixed memory budget) cannot obtain the FC
workspace with cudaMalloc.  ``q4fc_fc_decode_noalloc`` keeps the reduction
scratch in an array inside the library image instead.  The test calls it
through the C-ABI twice in a row -- the second call finds the scratch as the
first one left it -- and expects bit-identical outputs to ``q4fc_fc_decode``
run with the same (stream-K) kernel and a caller-provided workspace, whose
reduction order is deterministic; that is well inside the rtol 1e-3 /
atol 1e-4 bar the other FC tests use, which is also checked against the
default decode kernel.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(L, fn_noalloc, x, wq, N, y, q, G, ws=None):
    rows, K = x.shape[1], x.shape[2]
    Ng, Kg, _ = wq.shape
    s = torch.cuda.current_stream().cuda_stream
    if fn_noalloc:
        return L.q4fc_fc_decode_noalloc(x.data_ptr(), rows, K, K, wq.data_ptr(), Ng, Kg, q, G, N, y.data_ptr(), N, 0, s)
    flags = 4 if ws is not None else 0  # Q4FC_FLAG_STREAMK: the kernel the allocation-free entry point runs
    return L.q4fc_fc_decode(x.data_ptr(), rows, K, K, wq.data_ptr(), Ng, Kg, q, G, N, y.data_ptr(), N,
                            ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0, flags, s)


@pytest.mark.parametrize("qname,q,G", [("q4_1", 1, 128), ("q4_1", 1, 32), ("q4_0", 0, 32)])
def test_noalloc_matches_workspace_entry_point(lib_built, qname, q, G):
    assert torch.cuda.is_available()
    import llama_cl_b200 as pkg

    L = pkg._cabi.lib()
    g = torch.Generator().manual_seed(123)
    for (N, K, rows) in [(4096, 4096, 1), (11008, 4096, 8), (96, 512, 3), (72, 256, 2)]:
        W = (torch.randn(N, K, generator=g) * 0.02).cuda()
        wq = pkg.llmops.offline_FC_quant_Q4A(W, qtype=qname, group_k=G)
        ws = torch.zeros(int(L.q4fc_fc_workspace_bytes(rows, K, N, q, G)), dtype=torch.uint8, device="cuda")
        want = torch.empty((1, rows, N), device="cuda")
        for call in range(2):  # two calls in a row share the built-in scratch
            x = torch.randn(1, rows, K, generator=g).cuda()
            assert _call(L, False, x, wq, N, want, q, G, ws) == 0, L.q4fc_last_error()
            got = torch.full((1, rows, N), float("nan"), device="cuda")
            assert _call(L, True, x, wq, N, got, q, G) == 0, L.q4fc_last_error()
            torch.cuda.synchronize()
            assert torch.equal(got, want), (N, K, rows, call, float((got - want).abs().max()))
            default = torch.empty_like(want)
            assert _call(L, False, x, wq, N, default, q, G, None) == 0, L.q4fc_last_error()
            assert torch.allclose(got, default, rtol=1e-3, atol=1e-4)


def test_noalloc_rejects_sizes_beyond_the_scratch(lib_built):
    import llama_cl_b200 as pkg

    L = pkg._cabi.lib()
    N = 262144 + 32
    rc = L.q4fc_fc_decode_noalloc(16, 1, 128, 128, 16, N // 32, 1, 1, 128, N, 16, N, 0, None)
    assert rc == 7 and b"exceeds the built-in scratch" in L.q4fc_last_error()
    # more rows than the entry point takes: a stated limit, reported as such
    assert L.q4fc_fc_decode_noalloc(16, 9, 128, 128, 16, 1, 1, 1, 128, 32, 16, 32, 0, None) == 7
    # a packed tensor with more stripes than the scratch has counters for, even though N itself is small
    assert L.q4fc_fc_decode_noalloc(16, 1, 128, 128, 16, 8193, 1, 1, 128, 64, 16, 64, 0, None) == 7
