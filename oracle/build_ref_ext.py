"""Builds the reference's OLDER torch extension (ext/llama_ext.cpp: FC_quant_Q8C / FC_evaluate_Q8C and the Q4A
functions on torch tensors) as a checker module in ``oracle/_ref``.  TEST INFRASTRUCTURE ONLY.

The sources are compiled where they lie after two edits made on the fly in a temporary copy (nothing of the
reference is stored in this tree):
  * ``ext/ktensor.hpp``: the friend declaration's parameter ``T`` shadows the class template parameter, which
    g++ 13 rejects -- renamed;
  * ``ext/llama_ext.cpp``: ``.device(torch::kCPU, 1)`` aborts under current torch -- the device index is dropped.
Needs the reference checkout, torch's C++ headers and /usr/bin/g++ (the OpenMP spec file of other compilers on
the image is missing).

    python oracle/build_ref_ext.py --reference /path/to/llama.cl
"""
from __future__ import annotations

import argparse
import glob
import os
import shutil
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")


def module_path() -> str | None:
    hits = glob.glob(os.path.join(REF_DIR, "ref_c_ext*.so"))
    return hits[0] if hits else None


def build(reference: str, force: bool = False) -> str | None:
    src_dir = os.path.join(reference, "ext")
    if not os.path.exists(os.path.join(src_dir, "llama_ext.cpp")):
        return None
    if module_path() and not force:
        return module_path()
    os.makedirs(REF_DIR, exist_ok=True)
    from torch.utils.cpp_extension import load

    with tempfile.TemporaryDirectory() as tmp:
        for name in ("llama_ext.cpp", "ktensor.hpp", "intrinsic_helpers.hpp"):
            text = open(os.path.join(src_dir, name)).read()
            if name == "llama_ext.cpp":
                text = text.replace(".device(torch::kCPU, 1)", ".device(torch::kCPU)")
            if name == "ktensor.hpp":
                text = text.replace("friend std::ostream &operator<<(std::ostream &os, const Ktensor<U> &T);",
                                    "friend std::ostream &operator<<(std::ostream &os, const Ktensor<U> &t_);")
            open(os.path.join(tmp, name), "w").write(text)
        os.environ["CXX"] = "/usr/bin/g++"  # the only compiler on the image whose OpenMP links
        load(name="ref_c_ext", sources=[os.path.join(tmp, "llama_ext.cpp")],
             extra_cflags=["-O2", "-mavx2", "-mfma", "-mf16c", "-fopenmp", "-w"], extra_ldflags=["-fopenmp"],
             build_directory=tmp, verbose=False)
        for so in glob.glob(os.path.join(tmp, "ref_c_ext*.so")):
            shutil.copy(so, REF_DIR)
    return module_path()


def load_module():
    """The built checker module, or None."""
    p = module_path()
    if not p:
        return None
    import importlib.util

    import torch  # noqa: F401  (the extension links against libtorch)

    spec = importlib.util.spec_from_file_location("ref_c_ext", p)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("Q4FC_REFERENCE"), required="Q4FC_REFERENCE" not in os.environ)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build(a.reference, a.force))
