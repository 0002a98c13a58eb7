"""ctypes binding of ``lib/libq4fc_b200.so`` (C-ABI in ``include/q4fc_b200.h``).

There is no fallback: if the library is missing or a call fails, a
``RuntimeError`` is raised.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "lib", "libq4fc_b200.so")

Q4_0, Q4_1 = 0, 1
FLAG_NIBBLE_SIGNED = 1
FLAG_PDL = 2
FLAG_STREAMK = 4
FLAG_PREQUANT = 8

# every symbol declared in include/q4fc_b200.h
SYMBOLS = (
    "q4fc_version", "q4fc_strerror", "q4fc_last_error", "q4fc_block_bytes", "q4fc_infer_variant",
    "q4fc_pack", "q4fc_dequant", "q4fc_quant_x", "q4fc_fc_workspace_bytes", "q4fc_fc_workspace_init",
    "q4fc_fc_decode", "q4fc_fc_prefill", "q4fc_fc", "q4fc_fc_check_status", "q4fc_fc_decode_noalloc",
    "q4fc_fc_decode_add", "q4fc_fc_decode_multi", "q4fc_fc_decode_batch",
    "q4fc_tp_arena_create", "q4fc_tp_arena_open", "q4fc_tp_arena_close", "q4fc_tp_arena_destroy",
    "q4fc_tp_step_begin", "q4fc_tp_collect", "q4fc_fc_decode_tp", "q4fc_tp_site_bytes",
    "q4fc_fc_decode_tp_batch", "q4fc_tp_collect_multi",
    "q4fc_xq_bytes", "q4fc_quant_x_q8", "q4fc_rmsnorm_quant", "q4fc_add_rmsnorm_quant", "q4fc_fc_decode_q8",
    "q4fc_silu_mul_quant", "q4fc_quant_x_q8_batch",
    "q4fc_fc_chain_create", "q4fc_fc_chain_run", "q4fc_fc_chain_check", "q4fc_fc_chain_destroy",
    "q4fc_q8c_pack", "q4fc_q8c_workspace_bytes", "q4fc_q8c_fc", "q4fc_emb_q8c_quant", "q4fc_emb_q8c",
)


class TpSite(C.Structure):
    """``q4fc_tp_site`` of include/q4fc_b200.h."""
    _fields_ = [
        ("world", C.c_int),
        ("x_stamped", C.c_int),
        ("col_off", C.c_int64),
        ("y_peer", C.c_void_p * 8),
        ("epoch", C.c_void_p),
        ("status", C.c_void_p),
        ("xq_scratch", C.c_void_p),
    ]



class FcJob(C.Structure):
    """``q4fc_fc_job`` of include/q4fc_b200.h."""
    _fields_ = [
        ("wq", C.c_void_p),
        ("Ng", C.c_int64),
        ("N", C.c_int64),
        ("y", C.c_void_p),
        ("ldy", C.c_int64),
        ("addend", C.c_void_p),
        ("ld_addend", C.c_int64),
    ]


class ChainStep(C.Structure):
    """``q4fc_chain_step`` of include/q4fc_b200.h."""
    _fields_ = [
        ("x", C.c_void_p),
        ("ldx", C.c_int64),
        ("K", C.c_int64),
        ("transform", C.c_int),
        ("eps", C.c_float),
        ("aux", C.c_void_p),
        ("njobs", C.c_int),
    ]


CHAIN_PLAIN, CHAIN_RMSNORM, CHAIN_SILU_MUL = 0, 1, 2


class XqCall(C.Structure):
    """``q4fc_xq_call`` of include/q4fc_b200.h."""
    _fields_ = [("x", C.c_void_p), ("rows", C.c_int64), ("K", C.c_int64), ("ldx", C.c_int64), ("xq", C.c_void_p)]


class TpCall(C.Structure):
    """``q4fc_tp_call`` of include/q4fc_b200.h."""
    _fields_ = [
        ("x", C.c_void_p),
        ("xq", C.c_void_p),
        ("rows", C.c_int64),
        ("K", C.c_int64),
        ("ldx", C.c_int64),
        ("wq", C.c_void_p),
        ("Ng", C.c_int64),
        ("Kg", C.c_int64),
        ("N", C.c_int64),
        ("ldy", C.c_int64),
    ]


class FcCall(C.Structure):
    """``q4fc_fc_call`` of include/q4fc_b200.h."""
    _fields_ = [
        ("xq", C.c_void_p),
        ("rows", C.c_int64),
        ("K", C.c_int64),
        ("wq", C.c_void_p),
        ("Ng", C.c_int64),
        ("Kg", C.c_int64),
        ("N", C.c_int64),
        ("y", C.c_void_p),
        ("ldy", C.c_int64),
        ("addend", C.c_void_p),
        ("ld_addend", C.c_int64),
    ]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python llama.cl_b200/build.py` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback.")
    L = C.CDLL(LIB_PATH)
    i64, i32, u32, vp, sz, f32 = C.c_int64, C.c_int, C.c_uint, C.c_void_p, C.c_size_t, C.c_float
    L.q4fc_version.restype = i32
    L.q4fc_strerror.restype = C.c_char_p
    L.q4fc_strerror.argtypes = [i32]
    L.q4fc_last_error.restype = C.c_char_p
    L.q4fc_block_bytes.argtypes = [i32, i32]
    L.q4fc_infer_variant.argtypes = [i32, C.POINTER(i32), C.POINTER(i32)]
    L.q4fc_pack.argtypes = [vp, i64, i64, i32, i32, vp, vp]
    L.q4fc_dequant.argtypes = [vp, i64, i64, i32, i32, i32, vp, vp]
    L.q4fc_quant_x.argtypes = [vp, i64, i64, i64, i32, f32, vp, vp, vp, vp]
    L.q4fc_fc_workspace_bytes.restype = sz
    L.q4fc_fc_workspace_bytes.argtypes = [i64, i64, i64, i32, i32]
    L.q4fc_fc_workspace_init.argtypes = [vp, sz, vp]
    fc_args = [vp, i64, i64, i64, vp, i64, i64, i32, i32, i64, vp, i64, vp, sz, u32, vp]
    for name in ("q4fc_fc_decode", "q4fc_fc_prefill", "q4fc_fc"):
        getattr(L, name).argtypes = fc_args
    L.q4fc_fc_decode_add.argtypes = [vp, i64, i64, i64, vp, i64, i64, i32, i32, i64, vp, i64, vp, i64, vp, sz, u32, vp]
    L.q4fc_fc_decode_multi.argtypes = [vp, vp, i64, i64, i64, i64, i32, i32, C.POINTER(FcJob), i32, vp, sz, u32, vp]
    L.q4fc_fc_decode_batch.argtypes = [C.POINTER(FcCall), i32, i32, i32, u32, vp]
    L.q4fc_fc_check_status.argtypes = [vp, vp]
    L.q4fc_fc_decode_noalloc.argtypes = [vp, i64, i64, i64, vp, i64, i64, i32, i32, i64, vp, i64, u32, vp]
    L.q4fc_xq_bytes.restype = sz
    L.q4fc_xq_bytes.argtypes = [i64, i64, i32]
    L.q4fc_quant_x_q8.argtypes = [vp, i64, i64, i64, i32, i32, vp, u32, vp]
    L.q4fc_quant_x_q8_batch.argtypes = [C.POINTER(XqCall), i32, i32, i32, u32, vp]
    L.q4fc_rmsnorm_quant.argtypes = [vp, i64, i64, i64, vp, f32, vp, i64, i32, i32, vp, u32, vp]
    L.q4fc_add_rmsnorm_quant.argtypes = [vp, vp, vp, i64, i64, i64, vp, f32, vp, i64, i32, i32, vp, u32, vp]
    L.q4fc_silu_mul_quant.argtypes = [vp, vp, i64, i64, i64, vp, i64, i32, i32, vp, u32, vp]
    L.q4fc_fc_decode_q8.argtypes = [vp, i64, i64, vp, i64, i64, i32, i32, i64, vp, i64, u32, vp]
    L.q4fc_fc_chain_create.argtypes = [C.POINTER(ChainStep), i32, C.POINTER(FcJob), i32, i64, i32, i32, C.POINTER(vp)]
    L.q4fc_fc_chain_run.argtypes = [vp, vp]
    L.q4fc_fc_chain_check.argtypes = [vp, vp]
    L.q4fc_fc_chain_destroy.argtypes = [vp]
    L.q4fc_q8c_pack.argtypes = [vp, i64, i64, vp, vp, vp]
    L.q4fc_q8c_workspace_bytes.restype = sz
    L.q4fc_q8c_workspace_bytes.argtypes = [i64, i64]
    L.q4fc_q8c_fc.argtypes = [vp, i64, i64, i64, vp, vp, i64, i64, i64, vp, i64, vp, sz, vp]
    L.q4fc_emb_q8c_quant.argtypes = [vp, i64, i64, vp, vp, vp]
    L.q4fc_emb_q8c.argtypes = [vp, i32, i64, vp, vp, i64, i64, vp, i64, vp]
    L.q4fc_tp_site_bytes.restype = sz
    if L.q4fc_tp_site_bytes() != C.sizeof(TpSite):
        raise RuntimeError(f"q4fc_tp_site is {L.q4fc_tp_site_bytes()} bytes in the library, {C.sizeof(TpSite)} here")
    L.q4fc_tp_arena_create.argtypes = [sz, C.POINTER(vp), C.c_char_p]
    L.q4fc_tp_arena_open.argtypes = [C.c_char_p, C.POINTER(vp)]
    L.q4fc_tp_arena_close.argtypes = [vp]
    L.q4fc_tp_arena_destroy.argtypes = [vp]
    L.q4fc_tp_step_begin.argtypes = [vp, C.POINTER(vp), vp, i32, vp, vp]
    L.q4fc_tp_collect.argtypes = [vp, i64, i64, i64, vp, i64, vp, vp, vp]
    L.q4fc_fc_decode_tp.argtypes = [vp, i64, i64, i64, vp, i64, i64, i32, i32, i64, i64, C.POINTER(TpSite), u32, vp]
    L.q4fc_fc_decode_tp_batch.argtypes = [C.POINTER(TpCall), C.POINTER(C.POINTER(TpSite)), i32, i32, i32, u32, vp]
    L.q4fc_tp_collect_multi.argtypes = [C.POINTER(vp), C.POINTER(i64), C.POINTER(i64), C.POINTER(i64), C.POINTER(vp),
                                        C.POINTER(i64), i32, vp, vp, vp]
    _lib = L
    return L


def check(rc: int, what: str) -> None:
    if rc != 0:
        L = lib()
        raise RuntimeError(
            f"{what}: {L.q4fc_strerror(rc).decode()} ({rc}): {L.q4fc_last_error().decode()}")


_VARIANTS = {576: (Q4_0, 32), 2112: (Q4_0, 128), 640: (Q4_1, 32), 2176: (Q4_1, 128)}


def infer_variant(block_bytes: int) -> tuple[int, int]:
    """(qtype, group_k) from the last dimension of a packed tensor."""
    try:
        return _VARIANTS[int(block_bytes)]
    except KeyError:
        raise RuntimeError(
            f"assert weiq.size(2) == sizeof(q4_block) failed: block size {block_bytes} "
            "is none of 576 / 640 / 2112 / 2176") from None


def block_bytes(qtype: int, group_k: int) -> int:
    return 16 * group_k + (128 if qtype == Q4_1 else 64)


def parse_qtype(qtype) -> int:
    if qtype in (Q4_0, "q4_0", "Q4_0"):
        return Q4_0
    if qtype in (Q4_1, "q4_1", "Q4_1"):
        return Q4_1
    raise RuntimeError(f"unknown qtype {qtype!r}: expected 'q4_0' or 'q4_1'")
