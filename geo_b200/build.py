"""In-tree build of the native code: ``libgeo_sc.so`` (CUDA kernels + C ABI, sm_100a) and the
thin torch extension modules that expose it under the reference's module names.

    python -m geo_b200.build [--force] [--verbose]

nvcc cross-compiles for sm_100a without a GPU.  Nothing is installed outside the tree.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libgeo_sc.so")
EXT_DIR = os.path.join(PKG, "ext")  # holds sc_extension_cuda*.so and sc_extension*.so

CUDA_SOURCES = ["sc_api.cu", "sc_streams.cu", "sc_accumulate.cu", "sc_accumulate_sorted.cu", "sc_accumulate_rows.cu", "sc_accumulate_taps.cu", "sc_accumulate_short.cu", "sc_accumulate_fullbin.cu", "sc_peak.cu", "sc_guide.cu", "sc_guide_mma.cu", "sc_guide_tc.cu", "sc_bn.cu", "sc_static.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def _nvcc():
    home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    return os.path.join(home, "bin", "nvcc")


def _run(cmd, verbose):
    if verbose:
        print("+", " ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("build step failed: " + " ".join(cmd))
    if verbose and (r.stdout or r.stderr):
        print(r.stdout + r.stderr)


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_lib(force=False, verbose=False, ptxas_info=False):
    """nvcc -> geo_b200/lib/libgeo_sc.so"""
    srcs = [os.path.join(CSRC, s) for s in CUDA_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    deps = srcs + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    deps.append(os.path.join(ROOT, "include", "geo_sc.h"))
    if not force and not _stale(LIB_PATH, deps):
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    flags = list(NVCC_FLAGS)
    if ptxas_info:
        flags += ["-Xptxas", "-v"]
    objs = []
    procs = []
    for s in srcs:
        o = os.path.join(LIB_DIR, os.path.basename(s) + ".o")
        objs.append(o)
        cmd = [_nvcc(), *flags, "-c", s, "-o", o]
        if verbose:
            print("+", " ".join(cmd), flush=True)
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            sys.stderr.write(out)
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
        if (verbose or ptxas_info) and out:
            print(out)
    _run([_nvcc(), "-shared", "-o", LIB_PATH, *objs, "-Xcompiler", "-fPIC", "-cudart", "shared"], verbose)
    for o in objs:
        os.remove(o)
    return LIB_PATH


def build_torch_ext(force=False, verbose=False):
    """g++ -> geo_b200/ext/sc_extension_cuda.so and geo_b200/ext/sc_extension.so (pybind11 shims
    over the C ABI; no CUDA code of their own)."""
    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(EXT_DIR, exist_ok=True)
    inc = []
    for p in ce.include_paths():
        inc += ["-isystem", p]
    inc += ["-isystem", sysconfig.get_paths()["include"], "-I", os.path.join(ROOT, "include")]
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc += ["-isystem", os.path.join(cuda_home, "include")]
    libdir = ce.library_paths()[0]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    common = ["-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-std=c++17", "-O2", "-fPIC",
              "-shared"]
    link = [f"-L{libdir}", f"-Wl,-rpath,{libdir}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch", "-ltorch_cuda",
            "-ltorch_python", f"-L{LIB_DIR}", "-lgeo_sc", "-Wl,-rpath,$ORIGIN/../lib"]
    out = []
    for name in ("sc_extension_cuda", "sc_extension"):
        src = os.path.join(CSRC, name + ".cpp")
        target = os.path.join(EXT_DIR, name + ".so")
        out.append(target)
        if not force and not _stale(target, [src, os.path.join(ROOT, "include", "geo_sc.h")]):
            continue
        _run(["g++", *common, f"-DTORCH_EXTENSION_NAME={name}", *inc, src, "-o", target, *link], verbose)
    return out


def build_all(force=False, verbose=False):
    build_lib(force, verbose)
    build_torch_ext(force, verbose)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true", help="print registers / spills / shared memory per kernel")
    ap.add_argument("--lib-only", action="store_true")
    a = ap.parse_args(argv)
    build_lib(a.force or a.ptxas_info, a.verbose, a.ptxas_info)
    if not a.lib_only:
        build_torch_ext(a.force, a.verbose)
    return 0


if __name__ == "__main__":
    sys.exit(main())
