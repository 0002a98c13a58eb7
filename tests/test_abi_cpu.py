"""The C-ABI library loads and exports what include/q4fc_b200.h declares (no GPU compute)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "q4fc_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(q4fc_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(lib_built):
    lib = C.CDLL(lib_built)
    names = declared_functions()
    assert len(names) >= 14
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"


def test_python_binding_lists_every_symbol(lib_built):
    import llama_cl_b200 as pkg

    assert sorted(pkg._cabi.SYMBOLS) == declared_functions()
    assert pkg._cabi.lib().q4fc_version() >= 100


def test_variant_tables(lib_built):
    import llama_cl_b200 as pkg

    L = pkg._cabi.lib()
    for (q, G), bs in {(0, 32): 576, (0, 128): 2112, (1, 32): 640, (1, 128): 2176}.items():
        assert L.q4fc_block_bytes(q, G) == bs
        qq, gg = C.c_int(-1), C.c_int(-1)
        assert L.q4fc_infer_variant(bs, C.byref(qq), C.byref(gg)) == 0
        assert (qq.value, gg.value) == (q, G)
        assert pkg._cabi.infer_variant(bs) == (q, G)
    assert L.q4fc_block_bytes(1, 64) == -1
    assert L.q4fc_infer_variant(600, None, None) == 2
    with pytest.raises(RuntimeError):
        pkg._cabi.infer_variant(600)


def test_argument_errors_without_gpu(lib_built):
    """Validation happens before any CUDA call, so it can be checked here."""
    import llama_cl_b200 as pkg

    L = pkg._cabi.lib()
    assert L.q4fc_pack(None, 32, 32, 1, 64, None, None) == 2           # bad group
    assert L.q4fc_pack(None, -1, 32, 1, 32, None, None) == 1           # negative size
    assert L.q4fc_pack(None, 32, 32, 1, 32, None, None) == 1           # null pointers
    assert L.q4fc_pack(None, 0, 32, 1, 32, None, None) == 0            # empty is fine
    assert L.q4fc_quant_x(None, 0, 0, 0, 32, 1.0, None, None, None, None) == 0
    assert L.q4fc_quant_x(None, 1, 32, 32, 48, 1.0, None, None, None, None) == 2
    # K does not match Kg
    assert L.q4fc_fc_decode(16, 1, 100, 100, 16, 1, 2, 1, 32, 32, 16, 32, None, 0, 0, None) == 1
    # N beyond the packed columns
    assert L.q4fc_fc_decode(16, 1, 64, 64, 16, 1, 2, 1, 32, 64, 16, 64, None, 0, 0, None) == 1
    # rows beyond the decode limit
    assert L.q4fc_fc_decode(16, 9, 64, 64, 16, 1, 2, 1, 32, 32, 16, 32, None, 0, 0, None) == 7
    # misaligned packed pointer
    assert L.q4fc_fc_decode(16, 1, 64, 64, 8, 1, 2, 1, 32, 32, 16, 32, None, 0, 0, None) == 3
    assert b"alignment" in L.q4fc_last_error()
    assert L.q4fc_strerror(4) == b"workspace missing or too small"


def test_wrappers_reject_cpu_tensors(lib_built):
    """There is no CPU path: CPU tensors are an error, not a fallback."""
    import torch

    import llama_cl_b200 as pkg

    with pytest.raises(RuntimeError, match="CUDA"):
        pkg.llmops.offline_FC_quant_Q4A(torch.zeros(32, 32))
    with pytest.raises(RuntimeError, match=r"is<float32>\(3\)"):
        pkg.llmops.fc_Q4A(torch.zeros(32, 32), torch.zeros(1, 1, 640, dtype=torch.int8), 32)
    with pytest.raises(RuntimeError, match=r"is<int8>\(3\)"):
        pkg.llmops.offline_FC_dequant_Q4A(torch.zeros(1, 640))
    with pytest.raises(RuntimeError):
        pkg.llmops.fc_Q4A2(None, None, 0)
