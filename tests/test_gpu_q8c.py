"""Per-channel int8 FC (FC_quant_Q8C / FC_evaluate_Q8C of the reference's older extension) and the quantized
embedding table (embedding_q8c_quant_w / embedding_q8c of its ops module) on a B200, through the C-ABI, against the
CPU oracle and the rows the reference's own compiled code returned."""
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
    # the tolerance stated for fp32 FC outputs against the reference's CPU result
    return np.allclose(y, ref, rtol=1e-3, atol=1e-4)


def test_q8c_against_reference_rows(pkg, golden_dir):
    d = np.load(os.path.join(golden_dir, "q8c_ref.npz"))
    ext = pkg.c_ext
    for i in range(int(d["fc_cases"])):
        W = torch.from_numpy(d[f"W{i}"]).cuda()
        wq, ws = ext.FC_quant_Q8C(W)
        assert np.array_equal(wq.cpu().numpy(), d[f"wq{i}"]), i
        assert np.array_equal(ws.cpu().numpy(), d[f"ws{i}"]), i
        y = ext.FC_evaluate_Q8C(torch.from_numpy(d[f"x{i}"]).cuda(), wq, ws, W.shape[0]).cpu().numpy()
        assert close(y, d[f"y{i}"]), (i, np.abs(y - d[f"y{i}"]).max())
    ops = pkg.llmops
    for i in range(int(d["emb_cases"])):
        codes, scales = ops.embedding_q8c_quant_w(torch.from_numpy(d[f"table{i}"]).cuda())
        assert np.array_equal(codes.cpu().numpy(), d[f"codes{i}"]), i
        assert np.array_equal(scales.cpu().numpy(), d[f"scales{i}"].ravel()), i
        ids = torch.from_numpy(d[f"ids{i}"]).cuda()
        out = torch.empty(tuple(ids.shape) + (codes.shape[1],), dtype=torch.float32, device="cuda")
        ops.embedding_q8c(out, ids, codes, scales)
        assert np.array_equal(out.cpu().numpy(), d[f"emb{i}"]), i
        out32 = torch.full_like(out, -1.0)
        ops.embedding_q8c(out32, ids.to(torch.int32), codes, scales)
        assert torch.equal(out, out32)


@pytest.mark.parametrize("N,K", [(4096, 4096), (96, 1024), (40, 70), (1000, 11008), (32, 32), (33, 8200)])
@pytest.mark.parametrize("rows", [1, 3, 8, 9, 40])
def test_q8c_fc_against_oracle(pkg, oracle, N, K, rows):
    """Pack bit-equal to the oracle; FC within the stated tolerance, for decode and wider row counts, few and many
    stripes (with and without the K split over a cluster), ragged N and K, and twice the same bits."""
    ops = pkg.llmops
    g = torch.Generator().manual_seed(N + 7 * K + rows)
    W = torch.randn(N, K, generator=g) * 0.02
    W[N // 2] = 0
    x = torch.randn(1, rows, K, generator=g)
    wq, ws = ops.FC_quant_Q8C(W.cuda())
    rq, rs = oracle.restated.q8c_pack(W.numpy())
    assert np.array_equal(wq.cpu().numpy(), rq) and np.array_equal(ws.cpu().numpy(), rs)
    want = oracle.restated.q8c_fc(x.numpy(), rq, rs, N)
    y = ops.FC_evaluate_Q8C(x.cuda(), wq, ws, N)
    assert close(y.cpu().numpy(), want), np.abs(y.cpu().numpy() - want).max()
    y2 = torch.full_like(y, 7.0)
    ops.FC_evaluate_Q8C(x.cuda(), wq, ws, N, out=y2)
    assert torch.equal(y, y2)


def test_q8c_fc_batched_input_and_large_rows(pkg, oracle):
    ops = pkg.llmops
    g = torch.Generator().manual_seed(3)
    N, K = 256, 512
    W = torch.randn(N, K, generator=g)
    x = torch.randn(3, 50, K, generator=g) * 4
    wq, ws = ops.FC_quant_Q8C(W.cuda())
    want = oracle.restated.q8c_fc(x.numpy(), wq.cpu().numpy(), ws.cpu().numpy(), N)
    y = ops.FC_evaluate_Q8C(x.cuda(), wq, ws, N).cpu().numpy()
    assert y.shape == (3, 50, N)
    assert np.allclose(y, want, rtol=1e-3, atol=1e-3 * np.abs(want).max())


def test_q8c_argument_checks(pkg):
    ops = pkg.llmops
    W = torch.randn(64, 64).cuda()
    wq, ws = ops.FC_quant_Q8C(W)
    x = torch.randn(1, 1, 64).cuda()
    with pytest.raises(RuntimeError):
        ops.FC_evaluate_Q8C(x, wq, ws, 65)  # more columns than the weights hold
    with pytest.raises(RuntimeError):
        ops.FC_evaluate_Q8C(torch.randn(1, 1, 96).cuda(), wq, ws, 64)  # K does not match Kg
    with pytest.raises(RuntimeError):
        ops.FC_evaluate_Q8C(x, wq[:, :, :640].contiguous(), ws, 64)  # not a q8_c_block
    with pytest.raises(RuntimeError):
        ops.FC_evaluate_Q8C(x.cpu(), wq, ws, 64)  # no CPU path
    L = pkg._cabi.lib()
    assert L.q4fc_q8c_fc(x.data_ptr(), 1, 64, 64, wq.data_ptr(), ws.data_ptr(), 2, 2, 64, x.data_ptr(), 64, None, 0,
                         None) == 4  # Q4FC_EWORKSPACE
    # empty inputs are accepted and do nothing
    assert L.q4fc_q8c_fc(None, 0, 64, 64, wq.data_ptr(), ws.data_ptr(), 2, 2, 64, None, 64, None, 0, None) == 0
    assert L.q4fc_q8c_pack(None, 0, 64, None, None, None) == 0


@pytest.mark.parametrize("V,E", [(1000, 4096), (37, 100), (5, 8), (3, 5000)])
def test_embedding_q8c_against_oracle(pkg, oracle, V, E):
    ops = pkg.llmops
    rng = np.random.default_rng(V + E)
    table = rng.standard_normal((V, E)).astype(np.float32)
    table[V // 2] = 0
    table[0, :4] = [0.5, 1.5, 2.5, -0.5]
    codes, scales = ops.embedding_q8c_quant_w(torch.from_numpy(table).cuda())
    rc, rs = oracle.restated.emb_q8c_quant(table)
    assert np.array_equal(codes.cpu().numpy(), rc) and np.array_equal(scales.cpu().numpy(), rs)
    ids = rng.integers(0, V, size=(2, 9)).astype(np.int64)
    out = torch.empty((2, 9, E), dtype=torch.float32, device="cuda")
    ops.embedding_q8c(out, torch.from_numpy(ids).cuda(), codes, scales)
    assert np.array_equal(out.cpu().numpy(), oracle.restated.emb_q8c(ids, rc, rs))
    ops.check_device_status()


def test_embedding_q8c_checks(pkg):
    ops = pkg.llmops
    codes, scales = ops.embedding_q8c_quant_w(torch.randn(10, 64).cuda())
    ids = torch.tensor([[1, 2, 10]], device="cuda")
    out = torch.full((1, 3, 64), 5.0, device="cuda")
    with pytest.raises(RuntimeError):
        ops.embedding_q8c(out[:, :2], ids, codes, scales)  # shape of the output
    with pytest.raises(RuntimeError):
        ops.embedding_q8c(out, ids.float(), codes, scales)  # ids must be integers
    ops.check_device_status()
    ops.embedding_q8c(out, ids, codes, scales)  # id 10 is outside the table: zeros, and the status word says so
    assert torch.all(out[0, 2] == 0) and not torch.all(out[0, 1] == 0)
    with pytest.raises(RuntimeError, match="embedding id"):
        ops.check_device_status()
    ops.check_device_status()  # reading it cleared it
