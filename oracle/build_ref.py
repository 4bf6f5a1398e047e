"""Build `oracle/_ref/_apr_ref*.so`: the reference's CPU operators compiled unmodified.

Sources are read from the reference checkout where they lie (never copied into this repository);
only the compiled module is written, into oracle/_ref/ (git-ignored).  Run:

    python oracle/build_ref.py [--reference /path/to/APR-CNN]

Needs g++, OpenMP and the CPU libtorch that ships with the installed torch wheel.
"""
import argparse
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))


def reference_root():
    """Checkout of the reference project: the environment variable APRNET_REFERENCE, else a sibling `reference`
    directory of this repository."""
    return os.environ.get("APRNET_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(reference=None, force=False, verbose=True):
    reference = reference or reference_root()
    src_dir = os.path.join(reference, "pyapr", "aprnet", "src")
    if not os.path.isfile(os.path.join(src_dir, "conv.hpp")):
        raise FileNotFoundError("reference aprnet sources not found under " + src_dir)
    import torch
    from torch.utils import cpp_extension
    import pybind11

    out_dir = os.path.join(HERE, "_ref")
    os.makedirs(out_dir, exist_ok=True)
    ext = sysconfig.get_config_var("EXT_SUFFIX")
    out = os.path.join(out_dir, "_apr_ref" + ext)
    deps = [os.path.join(HERE, "ref_bind.cpp"),
            os.path.join(HERE, "ref_shim", "data_structures", "APR", "APR.hpp"),
            os.path.join(HERE, "ref_shim", "data_structures", "APR", "particles", "ParticleData.hpp")]
    if not force and os.path.isfile(out) and all(os.path.getmtime(out) >= os.path.getmtime(d) for d in deps):
        return out
    inc = ["-I" + os.path.join(HERE, "ref_shim"), "-I" + src_dir, "-I" + pybind11.get_include(),
           "-I" + sysconfig.get_paths()["include"]]
    inc += ["-I" + p for p in cpp_extension.include_paths()]
    lib_dir = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fopenmp", "-DPYAPR_HAVE_OPENMP",
           "-DTORCH_EXTENSION_NAME=_apr_ref", "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch.compiled_with_cxx11_abi()),
           "-w"] + inc + [deps[0], "-o", out, "-L" + lib_dir, "-Wl,-rpath," + lib_dir,
                          "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_python"]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=reference_root())
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build(a.reference, a.force))
