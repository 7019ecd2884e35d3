"""Build the reference's own SC extension sources, unmodified, into ``oracle/_ref/``.

TEST INFRASTRUCTURE ONLY.  Nothing here is part of the product path; the built
modules are used as the checker in ``tests/`` and as the timed CPU baseline in
``bench.py``.

The sources are compiled where they lie in the mounted reference tree
(``torch_c/sc-extension/{sc.cpp,sc_cuda.cpp,sc_cuda_kernel.cu}``); only compiled
objects are written, and only into ``oracle/_ref/``:

* ``oracle/_ref/avx512/sc_extension.so`` and ``oracle/_ref/avx2/sc_extension.so``
  -- the CPU extension (``sc.cpp``) built twice, because ``-march=native`` of the
  machine that builds is not necessarily the machine that runs; the loader in
  ``oracle/ref_loader.py`` picks the variant the running CPU supports.
* ``oracle/_ref/cuda/ref_sc_extension_cuda.so`` -- the CUDA extension built for
  sm_100a under another module name so that it can sit beside this repository's
  own ``sc_extension_cuda``.

Usage:  python oracle/build_ref.py [--reference /path/to/reference] [--no-cuda]
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
# GEO_REFERENCE_ROOT, else a checkout named "reference" beside this repository
REFERENCE_ROOT = os.environ.get("GEO_REFERENCE_ROOT",
                                os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))


def _torch_flags():
    import sysconfig

    import torch
    from torch.utils import cpp_extension as ce

    inc = []
    for p in ce.include_paths():
        inc += ["-isystem", p]
    inc += ["-isystem", sysconfig.get_paths()["include"]]
    libdir = ce.library_paths()[0]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    common = ["-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-std=c++17", "-O3", "-fPIC"]
    link = [f"-L{libdir}", f"-Wl,-rpath,{libdir}", "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python"]
    return inc, common, link, libdir


def _run(cmd):
    print("+", " ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_cpu(ref_root, variant):
    """sc.cpp -> oracle/_ref/<variant>/sc_extension.so (module name sc_extension)."""
    src = os.path.join(ref_root, "torch_c", "sc-extension", "sc.cpp")
    outdir = os.path.join(OUT, variant)
    os.makedirs(outdir, exist_ok=True)
    target = os.path.join(outdir, "sc_extension.so")
    if _newer(target, [src]):
        return target
    inc, common, link, _ = _torch_flags()
    march = {"avx512": ["-march=x86-64-v4"], "avx2": ["-march=x86-64-v3"]}[variant]
    # libgomp is linked by name: the compiler wrapper in this image cannot find
    # libgomp.spec when -fopenmp is given at link time.
    gomp_dir = "/usr/lib/gcc/x86_64-linux-gnu/13"
    # compile and link separately so that -fopenmp is only seen by the compile step
    obj = os.path.join(outdir, "sc.o")
    _run(["g++", "-c", *common, *march, "-fopenmp", "-DTORCH_EXTENSION_NAME=sc_extension", *inc, src, "-o", obj])
    _run(["g++", "-shared", obj, "-o", target, *link, f"-L{gomp_dir}", "-lgomp"])
    os.remove(obj)
    return target


def build_cuda(ref_root):
    """sc_cuda.cpp + sc_cuda_kernel.cu -> oracle/_ref/cuda/ref_sc_extension_cuda.so (sm_100a)."""
    d = os.path.join(ref_root, "torch_c", "sc-extension")
    srcs = [os.path.join(d, "sc_cuda.cpp"), os.path.join(d, "sc_cuda_kernel.cu")]
    outdir = os.path.join(OUT, "cuda")
    os.makedirs(outdir, exist_ok=True)
    target = os.path.join(outdir, "ref_sc_extension_cuda.so")
    if _newer(target, srcs):
        return target
    inc, common, link, libdir = _torch_flags()
    name = "-DTORCH_EXTENSION_NAME=ref_sc_extension_cuda"
    o1 = os.path.join(outdir, "sc_cuda.o")
    o2 = os.path.join(outdir, "sc_cuda_kernel.o")
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    nvcc = os.path.join(cuda_home, "bin", "nvcc")
    nv_common = [c for c in common if c != "-fPIC"]
    with ThreadPoolExecutor(2) as ex:
        f1 = ex.submit(_run, ["g++", "-c", *common, name, *inc, "-isystem", os.path.join(cuda_home, "include"),
                              srcs[0], "-o", o1])
        f2 = ex.submit(_run, [nvcc, "-c", *nv_common, name, *inc, "-Xcompiler", "-fPIC",
                              "-gencode", "arch=compute_100a,code=sm_100a", "--expt-relaxed-constexpr",
                              srcs[1], "-o", o2])
        f1.result()
        f2.result()
    _run(["g++", "-shared", o1, o2, "-o", target, *link, "-lc10_cuda", "-ltorch_cuda",
          f"-L{cuda_home}/lib64", "-lcudart"])
    os.remove(o1)
    os.remove(o2)
    return target


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=REFERENCE_ROOT)
    ap.add_argument("--no-cuda", action="store_true")
    args = ap.parse_args(argv)
    if not os.path.isdir(args.reference):
        print(f"reference tree {args.reference} not present; keeping prebuilt files in {OUT}")
        return 0
    build_cpu(args.reference, "avx512")
    build_cpu(args.reference, "avx2")
    if not args.no_cuda:
        build_cuda(args.reference)
    return 0


if __name__ == "__main__":
    sys.exit(main())
