"""Build recipe for the two CPU checkers (TEST INFRASTRUCTURE ONLY).

1. ``oracle/libq4fc_oracle.so`` -- gcc build of ``q4fc_oracle.c``, the plain-C
   restatement of the reference's quantized-FC arithmetic.  Always built.
2. ``oracle/_ref/libref_<variant>_<isa>.so`` -- the reference's own
   ``ops/op_fc.hpp`` (with ``tensor.hpp`` / ``utils.hpp``) compiled where it
   lies in the reference checkout.  Only built when that checkout is present.
   The block type is a compile-time alias in the reference
   (``ops/op_fc.hpp:109``), so the header is streamed through a one-line
   rewrite of that alias into the compiler's stdin; nothing is copied into
   this tree.  ``isa`` is ``vnni`` (``-mavxvnni``: ``vnni()`` in
   ``ops/utils.hpp:222`` uses ``dpbusd``) or ``avx2`` (``maddubs``+``madd``
   fallback, which saturates only on the Q4_0 operands).  Two flavours are
   kept because the machine that runs the checker may lack AVX-VNNI.

Only tests, the smoke check and the benchmark's CPU-baseline leg may load
these libraries; the shipped CUDA path never does.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
ORACLE_SO = os.path.join(HERE, "libq4fc_oracle.so")

# variant name -> right-hand side of the alias on ops/op_fc.hpp:109
VARIANTS = {
    "q4_1_g32": "q4_1_block<32>",
    "q4_1_g128": "q4_1_block<128>",
    "q4_0_g32": "q4_0_block<32>",
    "q4_0_g128": "q4_0_block<128>",
}
ISAS = {
    "vnni": ["-mavx2", "-mfma", "-mf16c", "-mavxvnni"],
    "avx2": ["-mavx2", "-mfma", "-mf16c"],
}
STOCK_ALIAS = "using q4_block = q4_1_block<32>;"


def _cxx() -> str:
    # a toolchain under /opt/gcc may lack libgomp.spec; prefer the system one
    for c in ("/usr/bin/g++", shutil.which("g++")):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("no g++ found")


def _cc() -> str:
    for c in ("/usr/bin/gcc", shutil.which("gcc")):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("no gcc found")


def _newer(target: str, *deps: str) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps if os.path.exists(d))


def build_restatement(force: bool = False) -> str:
    src = os.path.join(HERE, "q4fc_oracle.c")
    if not force and _newer(ORACLE_SO, src):
        return ORACLE_SO
    # -ffp-contract=off: every fp32 product is rounded before it is used,
    # fused multiply-adds appear only where the source calls fmaf().
    cmd = [_cc(), "-O2", "-std=c11", "-shared", "-fPIC", "-fopenmp", "-ffp-contract=off",
           "-mf16c", "-mfma", src, "-o", ORACLE_SO, "-lm"]
    subprocess.run(cmd, check=True)
    return ORACLE_SO


def ref_lib_path(variant: str, isa: str) -> str:
    return os.path.join(REF_DIR, f"libref_{variant}_{isa}.so")


def reference_root() -> str | None:
    """Where the reference checkout lies: the environment variable Q4FC_REFERENCE, or --reference on the command line."""
    return os.environ.get("Q4FC_REFERENCE") or None


def build_reference(reference_root: str | None = None, force: bool = False) -> list[str]:
    """Compile the reference's FC for the four block variants x two ISAs.

    ``reference_root``: the reference checkout (default: the environment variable Q4FC_REFERENCE).  Returns the
    list of libraries built (empty when no checkout is given or it is absent)."""
    if reference_root is None:
        reference_root = os.environ.get("Q4FC_REFERENCE")
    if not reference_root:
        return []
    ops = os.path.join(reference_root, "ops")
    hdr = os.path.join(ops, "op_fc.hpp")
    if not os.path.exists(hdr):
        return []
    os.makedirs(REF_DIR, exist_ok=True)
    head = open(os.path.join(HERE, "ref_shim_head.inc")).read()
    tail = open(os.path.join(HERE, "ref_shim_tail.inc")).read()
    body = open(hdr).read()
    if STOCK_ALIAS not in body:
        raise RuntimeError("reference alias line not found in ops/op_fc.hpp")
    built = []
    for variant, rhs in VARIANTS.items():
        unit = head + body.replace("#pragma once", "").replace(
            STOCK_ALIAS, f"using q4_block = {rhs};") + tail
        for isa, flags in ISAS.items():
            out = ref_lib_path(variant, isa)
            if not force and _newer(out, hdr, os.path.join(HERE, "ref_shim_tail.inc"),
                                    os.path.join(HERE, "ref_shim_head.inc")):
                built.append(out)
                continue
            cmd = [_cxx(), "-O2", "-std=c++17", "-shared", "-fPIC", "-fopenmp", "-w",
                   *flags, "-I", ops, "-x", "c++", "-", "-o", out]
            subprocess.run(cmd, input=unit.encode(), check=True)
            built.append(out)
    return built


def main() -> None:
    force = "--force" in sys.argv
    ref = None
    if "--reference" in sys.argv:
        ref = sys.argv[sys.argv.index("--reference") + 1]
    print(build_restatement(force))
    for p in build_reference(ref, force=force):
        print(p)


if __name__ == "__main__":
    main()
