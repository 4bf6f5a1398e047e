"""Build the two native artefacts of this package, in-tree:

  libaprnet_b200.so   CUDA kernels + C ABI (include/aprnet_b200.h), nvcc, sm_100a only
  _pyaprwrapper*.so   pybind11/torch host layer exporting the reference's module interface

Run `python apr-cnn_b200/build.py` (add --force to rebuild).  nvcc cross-compiles without a GPU.
"""
import argparse
import concurrent.futures
import os
import subprocess
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-diag-suppress", "177"]


def _newer(target, deps):
    if not os.path.isfile(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def cuda_sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def build_library(force=False, verbose=False):
    out = os.path.join(HERE, "libaprnet_b200.so")
    srcs = cuda_sources()
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(ROOT, "include", "aprnet_b200.h"))
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    objs, jobs = [], []
    for s in srcs:
        o = os.path.join(objdir, os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or _newer(o, [s] + headers):
            jobs.append([NVCC] + NVCC_FLAGS + ["-c", s, "-o", o])
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for cmd, res in zip(jobs, ex.map(lambda c: subprocess.run(c, capture_output=True, text=True), jobs)):
                if verbose or res.returncode:
                    print(" ".join(cmd)); print(res.stdout, res.stderr)
                if res.returncode:
                    raise RuntimeError("nvcc failed for " + cmd[-3])
    if jobs or force or _newer(out, objs):
        subprocess.check_call([NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", out] + objs + ["-lcudart"])
    return out


def build_binding(force=False, verbose=False):
    import torch
    from torch.utils import cpp_extension
    import pybind11
    ext = sysconfig.get_config_var("EXT_SUFFIX")
    out = os.path.join(HERE, "_pyaprwrapper" + ext)
    src = os.path.join(HERE, "bind", "pyaprwrapper.cpp")
    deps = [src, os.path.join(ROOT, "include", "aprnet_b200.h")]
    if not force and not _newer(out, deps):
        return out
    lib_dir = os.path.join(os.path.dirname(torch.__file__), "lib")
    inc = ["-I" + p for p in cpp_extension.include_paths()] + ["-I" + pybind11.get_include(),
           "-I" + sysconfig.get_paths()["include"], "-I/usr/local/cuda/include"]
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-w", "-DTORCH_EXTENSION_NAME=_pyaprwrapper",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch.compiled_with_cxx11_abi())] + inc + [src, "-o", out,
           "-L" + HERE, "-laprnet_b200", "-Wl,-rpath,$ORIGIN", "-L" + lib_dir, "-Wl,-rpath," + lib_dir,
           "-ltorch", "-ltorch_cpu", "-lc10", "-lc10_cuda", "-ltorch_cuda", "-ltorch_python"]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return out


def build_all(force=False, verbose=False):
    return build_library(force, verbose), build_binding(force, verbose)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("-v", "--verbose", action="store_true")
    a = ap.parse_args()
    print(build_all(a.force, a.verbose))
