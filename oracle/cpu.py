"""numpy front-ends for the two CPU checkers (TEST INFRASTRUCTURE ONLY).

``restated``  -- the plain-C restatement in ``q4fc_oracle.c``.
``compiled_reference(variant)`` -- the reference's own ``ops/op_fc.hpp``
compiled by ``build_oracle.py`` into ``oracle/_ref`` (one library per block
variant, because the variant is a compile-time alias in the reference).

Only ``tests/``, the smoke check and the benchmark's CPU-baseline leg may
import this module.  The shipped CUDA path never does.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
Q4_0, Q4_1 = 0, 1

_VARIANT_OF_BS = {576: (Q4_0, 32), 2112: (Q4_0, 128), 640: (Q4_1, 32), 2176: (Q4_1, 128)}


def block_bytes(qtype: int, G: int) -> int:
    return 16 * G + (128 if qtype == Q4_1 else 64)


def infer_variant(bs: int) -> tuple[int, int]:
    return _VARIANT_OF_BS[int(bs)]


def variant_name(qtype: int, G: int) -> str:
    return f"q4_{qtype}_g{G}"


def _p(a: np.ndarray, t):
    return a.ctypes.data_as(C.POINTER(t))


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a), dtype=np.float32)


class _Restated:
    """ctypes binding of oracle/libq4fc_oracle.so."""

    def __init__(self) -> None:
        self._lib = None

    @property
    def lib(self):
        if self._lib is None:
            path = os.path.join(HERE, "libq4fc_oracle.so")
            if not os.path.exists(path):
                from . import build_oracle

                build_oracle.build_restatement()
            lib = C.CDLL(path)
            i64, i32, f32 = C.c_int64, C.c_int, C.c_float
            u8p, i8p, fp = C.POINTER(C.c_uint8), C.POINTER(C.c_int8), C.POINTER(C.c_float)
            lib.oracle_pack.argtypes = [fp, i64, i64, i32, i32, u8p]
            lib.oracle_dequant.argtypes = [u8p, i64, i64, i32, i32, i32, fp]
            lib.oracle_quant_x.argtypes = [fp, i64, i64, i32, f32, i8p, fp, fp]
            lib.oracle_fc.argtypes = [fp, i64, i64, u8p, i64, i64, i32, i32, i64, i32, fp, i64]
            lib.oracle_rmsnorm.argtypes = [fp, i64, i64, fp, f32]
            lib.oracle_silu_mul.argtypes = [fp, fp, i64, fp]
            lib.oracle_q8c_pack.argtypes = [fp, i64, i64, i8p, fp]
            lib.oracle_q8c_fc.argtypes = [fp, i64, i64, i8p, fp, i64, i64, i64, fp, i64]
            lib.oracle_emb_q8c_quant.argtypes = [fp, i64, i64, i8p, fp]
            lib.oracle_emb_q8c.argtypes = [C.POINTER(C.c_int64), i64, i8p, fp, i64, fp]
            lib.oracle_f32_to_f16.argtypes = [f32]
            lib.oracle_f32_to_f16.restype = C.c_uint16
            lib.oracle_f16_to_f32.argtypes = [C.c_uint16]
            lib.oracle_f16_to_f32.restype = f32
            lib.oracle_max_threads.restype = i32
            self._lib = lib
        return self._lib

    def threads(self) -> int:
        return int(self.lib.oracle_max_threads())

    def pack(self, w, qtype: int = Q4_1, G: int = 32) -> np.ndarray:
        w = _f32(w)
        N, K = w.shape
        Ng, Kg = (N + 31) // 32, (K + G - 1) // G
        out = np.empty((Ng, Kg, block_bytes(qtype, G)), dtype=np.int8)
        rc = self.lib.oracle_pack(_p(w, C.c_float), N, K, qtype, G, _p(out, C.c_uint8))
        if rc:
            raise RuntimeError(f"oracle_pack failed ({rc})")
        return out

    def dequant(self, wq, nibble_signed: bool = False) -> np.ndarray:
        wq = np.ascontiguousarray(wq, dtype=np.int8)
        Ng, Kg, bs = wq.shape
        qtype, G = infer_variant(bs)
        out = np.empty((Ng * 32, Kg * G), dtype=np.float32)
        rc = self.lib.oracle_dequant(_p(wq, C.c_uint8), Ng, Kg, qtype, G, int(nibble_signed), _p(out, C.c_float))
        if rc:
            raise RuntimeError(f"oracle_dequant failed ({rc})")
        return out

    def quant_x(self, x, G: int, scale: float = 1.0):
        x = _f32(x)
        K = x.shape[-1]
        rows = x.size // K if K else 0
        Kg = (K + G - 1) // G
        codes = np.empty(x.shape[:-1] + (Kg * G,), dtype=np.int8)
        scales = np.empty(x.shape[:-1] + (Kg,), dtype=np.float32)
        gsums = np.empty(x.shape[:-1] + (Kg,), dtype=np.float32)
        rc = self.lib.oracle_quant_x(_p(x, C.c_float), rows, K, G, scale, _p(codes, C.c_int8),
                                     _p(scales, C.c_float), _p(gsums, C.c_float))
        if rc:
            raise RuntimeError(f"oracle_quant_x failed ({rc})")
        return codes, scales, gsums

    def fc(self, x, wq, N: int, nibble_signed: bool = False) -> np.ndarray:
        x = _f32(x)
        wq = np.ascontiguousarray(wq, dtype=np.int8)
        Ng, Kg, bs = wq.shape
        qtype, G = infer_variant(bs)
        K = x.shape[-1]
        rows = x.size // K
        y = np.zeros(x.shape[:-1] + (N,), dtype=np.float32)
        rc = self.lib.oracle_fc(_p(x, C.c_float), rows, K, _p(wq, C.c_uint8), Ng, Kg, qtype, G, N,
                                int(nibble_signed), _p(y, C.c_float), N)
        if rc:
            raise RuntimeError(f"oracle_fc failed ({rc})")
        return y

    def rmsnorm(self, x, weight, eps: float) -> np.ndarray:
        """llmops.rmsnorm (ops/op_misc.hpp:142-181) on a copy of ``x`` [..., K]."""
        y = _f32(x).copy()
        w = _f32(weight)
        K = y.shape[-1]
        rc = self.lib.oracle_rmsnorm(_p(y, C.c_float), y.size // K, K, _p(w, C.c_float), eps)
        if rc:
            raise RuntimeError(f"oracle_rmsnorm failed ({rc})")
        return y

    def silu_mul(self, gate, up) -> np.ndarray:
        """up * silu(gate) as the reference's itrans("silu") + imul compute it (ops/op_misc.hpp:83-138), with an
        exact reciprocal in place of its approximate one."""
        g, u = _f32(gate), _f32(up)
        out = np.empty_like(g)
        rc = self.lib.oracle_silu_mul(_p(g, C.c_float), _p(u, C.c_float), g.size, _p(out, C.c_float))
        if rc:
            raise RuntimeError(f"oracle_silu_mul failed ({rc})")
        return out

    def q8c_pack(self, w):
        """FC_quant_Q8C (ext/llama_ext.cpp:56-113): -> (int8 [Ng][Kg][1024], fp32 scales [Ng*32])."""
        w = _f32(w)
        N, K = w.shape
        Ng, Kg = (N + 31) // 32, (K + 31) // 32
        wq = np.empty((Ng, Kg, 1024), dtype=np.int8)
        sc = np.empty((Ng * 32,), dtype=np.float32)
        if self.lib.oracle_q8c_pack(_p(w, C.c_float), N, K, _p(wq, C.c_int8), _p(sc, C.c_float)):
            raise RuntimeError("oracle_q8c_pack failed")
        return wq, sc

    def q8c_fc(self, x, wq, wscales, N: int) -> np.ndarray:
        """FC_evaluate_Q8C (ext/llama_ext.cpp:232-371)."""
        x = _f32(x)
        wq = np.ascontiguousarray(wq, dtype=np.int8)
        ws = _f32(wscales)
        Ng, Kg, _ = wq.shape
        K = x.shape[-1]
        rows = x.size // K
        y = np.zeros(x.shape[:-1] + (N,), dtype=np.float32)
        rc = self.lib.oracle_q8c_fc(_p(x, C.c_float), rows, K, _p(wq, C.c_int8), _p(ws, C.c_float), Ng, Kg, N,
                                    _p(y, C.c_float), N)
        if rc:
            raise RuntimeError(f"oracle_q8c_fc failed ({rc})")
        return y

    def emb_q8c_quant(self, w):
        """embedding_q8c_quant_w (ops/op_embedding.hpp:51-78): -> (int8 [V][E], fp32 scales [V])."""
        w = _f32(w)
        V, E = w.shape
        codes = np.empty((V, E), dtype=np.int8)
        sc = np.empty((V,), dtype=np.float32)
        if self.lib.oracle_emb_q8c_quant(_p(w, C.c_float), V, E, _p(codes, C.c_int8), _p(sc, C.c_float)):
            raise RuntimeError("oracle_emb_q8c_quant failed")
        return codes, sc

    def emb_q8c(self, ids, codes, scales) -> np.ndarray:
        """embedding_q8c (ops/op_embedding.hpp:80-137)."""
        ids = np.ascontiguousarray(ids, dtype=np.int64)
        codes = np.ascontiguousarray(codes, dtype=np.int8)
        sc = _f32(scales)
        E = codes.shape[1]
        out = np.empty(ids.shape + (E,), dtype=np.float32)
        if self.lib.oracle_emb_q8c(_p(ids, C.c_int64), ids.size, _p(codes, C.c_int8), _p(sc, C.c_float), E,
                                   _p(out, C.c_float)):
            raise RuntimeError("oracle_emb_q8c failed")
        return out

    def f16_bits(self, v: float) -> int:
        return int(self.lib.oracle_f32_to_f16(v))

    def f16_value(self, bits: int) -> float:
        return float(self.lib.oracle_f16_to_f32(bits))


restated = _Restated()


def _cpu_flags() -> set[str]:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


class CompiledReference:
    """ctypes binding of one oracle/_ref/libref_<variant>_<isa>.so."""

    def __init__(self, qtype: int, G: int, isa: str | None = None) -> None:
        flags = _cpu_flags()
        if isa is None:
            isa = "vnni" if "avx_vnni" in flags else "avx2"
        if isa == "avx2" and not {"avx2", "fma", "f16c"} <= flags:
            raise OSError("host CPU lacks AVX2/FMA/F16C: compiled reference cannot run")
        path = os.path.join(HERE, "_ref", f"libref_{variant_name(qtype, G)}_{isa}.so")
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.qtype, self.G, self.isa, self.path = qtype, G, isa, path
        lib = C.CDLL(path)
        i64, i32 = C.c_int64, C.c_int
        i8p, fp = C.POINTER(C.c_int8), C.POINTER(C.c_float)
        lib.ref_pack.argtypes = [fp, i64, i64, i8p]
        lib.ref_dequant.argtypes = [i8p, i64, i64, fp]
        lib.ref_quant_x.argtypes = [fp, i64, i64, i64, i8p, fp, fp]
        lib.ref_fc.argtypes = [fp, i64, i64, i64, i8p, i64, i64, i32, fp]
        assert lib.ref_block_bytes() == block_bytes(qtype, G)
        assert lib.ref_group_k() == G
        self.lib = lib
        # Q4_0 on the maddubs fallback saturates int16 pair sums (ops/utils.hpp:229-231)
        self.exact_int_dot = bool(lib.ref_uses_vnni()) or qtype == Q4_1

    def threads(self) -> int:
        return int(self.lib.ref_max_threads())

    def set_threads(self, n: int) -> int:
        """Size of the OpenMP team of later calls; returns what is in force (older builds of the checker
        library have no setter: then the inherited OMP_NUM_THREADS stands)."""
        if hasattr(self.lib, "ref_set_threads"):
            return int(self.lib.ref_set_threads(int(n)))
        return self.threads()

    def pack(self, w) -> np.ndarray:
        w = _f32(w)
        N, K = w.shape
        G = self.G
        if K % G:
            raise ValueError("the reference reads past the row end when K % G != 0")
        Ng, Kg = (N + 31) // 32, K // G
        out = np.zeros((Ng, Kg, block_bytes(self.qtype, G)), dtype=np.int8)
        if self.lib.ref_pack(_p(w, C.c_float), N, K, _p(out, C.c_int8)):
            raise RuntimeError("ref_pack failed")
        return out

    def dequant(self, wq) -> np.ndarray:
        wq = np.ascontiguousarray(wq, dtype=np.int8)
        Ng, Kg, _ = wq.shape
        out = np.empty((Ng * 32, Kg * self.G), dtype=np.float32)
        if self.lib.ref_dequant(_p(wq, C.c_int8), Ng, Kg, _p(out, C.c_float)):
            raise RuntimeError("ref_dequant failed")
        return out

    def quant_x(self, x):
        x = _f32(x)
        if x.ndim == 2:
            x = x[None]
        B, M, K = x.shape
        Kg = (K + self.G - 1) // self.G
        codes = np.empty((B, M, Kg * self.G), dtype=np.int8)
        scales = np.empty((B, M, Kg), dtype=np.float32)
        gsums = np.empty((B, M, Kg), dtype=np.float32)
        if self.lib.ref_quant_x(_p(x, C.c_float), B, M, K, _p(codes, C.c_int8), _p(scales, C.c_float),
                                _p(gsums, C.c_float)):
            raise RuntimeError("ref_quant_x failed")
        return codes, scales, gsums

    def fc(self, x, wq, N: int) -> np.ndarray:
        x = _f32(x)
        if x.ndim == 2:
            x = x[None]
        B, M, K = x.shape
        wq = np.ascontiguousarray(wq, dtype=np.int8)
        Ng, Kg, _ = wq.shape
        if N % 32 or N > Ng * 32:
            raise ValueError("the reference writes 32 outputs per block: N must be a multiple of 32")
        y = np.empty((B, M, N), dtype=np.float32)
        if self.lib.ref_fc(_p(x, C.c_float), B, M, K, _p(wq, C.c_int8), Ng, Kg, N, _p(y, C.c_float)):
            raise RuntimeError("ref_fc failed")
        return y


_ref_cache: dict = {}


def compiled_reference(qtype: int, G: int, isa: str | None = None) -> CompiledReference:
    key = (qtype, G, isa)
    if key not in _ref_cache:
        _ref_cache[key] = CompiledReference(qtype, G, isa)
    return _ref_cache[key]


def have_compiled_reference(qtype: int = Q4_1, G: int = 32) -> bool:
    try:
        compiled_reference(qtype, G)
        return True
    except (OSError, FileNotFoundError, AssertionError):
        return False
