"""TEST INFRASTRUCTURE ONLY.  Compiles the reference's own pybind11 module ``llmops`` (ops/main.cpp,
ops/profiler.cpp, with every header they include) from the sources where they lie, into
``oracle/_ref/llmops<ext-suffix>.so``.  No source is copied or changed; the pybind11 headers are the
ones of the installed ``pybind11`` package (the reference's own copy is an empty submodule).

Used to generate the checkpoint fixture of ``tests/golden/`` (``make_checkpoint_fixture.py``) and, where
it is present, to check the checkpoint reader against genuine pickles.  Nothing in the product imports it.

    python oracle/build_ref_module.py [--reference /path/to/llama.cl]
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def module_path() -> str:
    return os.path.join(OUT, "llmops" + sysconfig.get_config_var("EXT_SUFFIX"))


def build(reference: str, force: bool = False) -> str | None:
    """Returns the module's path, or None when the reference tree or pybind11 is not available."""
    ops = os.path.join(reference, "ops")
    srcs = [os.path.join(ops, "main.cpp"), os.path.join(ops, "profiler.cpp")]
    if not all(os.path.exists(s) for s in srcs):
        return None
    try:
        import pybind11
    except ImportError:
        return None
    out = module_path()
    if os.path.exists(out) and not force and all(os.path.getmtime(out) >= os.path.getmtime(s) for s in srcs):
        return out
    os.makedirs(OUT, exist_ok=True)
    cmd = ["g++", "-O2", "-shared", "-fPIC", "-std=c++17", "-mavx2", "-mfma", "-mf16c", "-fopenmp", "-w",
           "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], "-I", ops, *srcs, "-o", out]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("g++ failed on the reference's module:\n" + res.stderr[-4000:])
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("Q4FC_REFERENCE"), required="Q4FC_REFERENCE" not in os.environ)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    p = build(a.reference, a.force)
    print(p if p else "reference tree or pybind11 not available: nothing built")
    sys.exit(0)
