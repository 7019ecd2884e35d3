"""Load the reference's own extension modules built by ``oracle/build_ref.py``.

TEST INFRASTRUCTURE ONLY (checker and timed CPU baseline).
"""
from __future__ import annotations

import importlib.util
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")


def _cpu_flags():
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def _load(path, name):
    import torch  # noqa: F401  (libtorch must be loaded before the extension)

    # Creating an extension module also files it in sys.modules under its own name, where it would shadow
    # this repository's modules of the same names (the torch shims sc_extension / sc_extension_cuda): put back
    # whatever was there.
    saved = sys.modules.get(name)
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    if saved is not None:
        sys.modules[name] = saved
    elif sys.modules.get(name) is mod:
        del sys.modules[name]
    return mod


def cpu_variant():
    """Name of the sc.cpp build the running CPU can execute, or None."""
    flags = _cpu_flags()
    need512 = {"avx512f", "avx512bw", "avx512cd", "avx512dq", "avx512vl"}
    if need512 <= flags and os.path.exists(os.path.join(REF_DIR, "avx512", "sc_extension.so")):
        return "avx512"
    if {"avx2", "fma", "bmi2"} <= flags and os.path.exists(os.path.join(REF_DIR, "avx2", "sc_extension.so")):
        return "avx2"
    return None


_cpu_mod = None
_cuda_mod = None


def ref_sc_extension():
    """The reference CPU module ``sc_extension`` (sc.cpp:474-476) or None if not built."""
    global _cpu_mod
    if _cpu_mod is None:
        v = cpu_variant()
        if v is None:
            return None
        _cpu_mod = _load(os.path.join(REF_DIR, v, "sc_extension.so"), "sc_extension")
    return _cpu_mod


def ref_sc_extension_cuda():
    """The reference CUDA module (sc_cuda.cpp:78-83) built for sm_100a, or None."""
    global _cuda_mod
    if _cuda_mod is None:
        p = os.path.join(REF_DIR, "cuda", "ref_sc_extension_cuda.so")
        if not os.path.exists(p):
            return None
        _cuda_mod = _load(p, "ref_sc_extension_cuda")
    return _cuda_mod


def reference_python(ref_root=None):
    """Import the reference's ``utils_functional`` from its own tree (fixture generation
    only; the tree does not exist where the GPU tests run).  ``sc_extension`` resolves to
    the reference CPU build; ``sc_extension_cuda`` to an empty stand-in, because no GPU
    code can run where fixtures are generated."""
    if ref_root is None:
        from . import REFERENCE_ROOT as ref_root
    if "utils_functional" in sys.modules and getattr(sys.modules["utils_functional"], "__geo_ref__", False):
        return sys.modules["utils_functional"]
    cpu = ref_sc_extension()
    if cpu is None:
        raise RuntimeError("reference sc_extension not built (run oracle/build_ref.py)")
    saved = {k: sys.modules.get(k) for k in ("sc_extension", "sc_extension_cuda", "utils_functional")}
    sys.modules["sc_extension"] = cpu
    sys.modules["sc_extension_cuda"] = types.ModuleType("sc_extension_cuda")
    sys.path.insert(0, ref_root)
    try:
        sys.modules.pop("utils_functional", None)
        import utils_functional as uf

        uf.__geo_ref__ = True
    finally:
        sys.path.remove(ref_root)
        for k in ("sc_extension", "sc_extension_cuda"):
            if saved[k] is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = saved[k]
        sys.modules.pop("utils_functional", None)
    return uf
