"""geo_b200: the stochastic-computing (SC) conv2d / linear hot path of nanocad-lab/geo as
hand-written CUDA for NVIDIA B200 (sm_100a), behind the reference's own operator interface.

    geo_b200.functional   conv2d_generic / linear_generic / quantize   (utils_functional.py)
    geo_b200.layers       Conv2d_Add_Partial, BatchNorm2d_fixed, ...   (utils_class.py)
    geo_b200.network      CONV_tiny_add_partial, VGG11_add_partial     (network.py)
    geo_b200.ops          torch front end of the C ABI (include/geo_sc.h)
    geo_b200.ext          sc_extension_cuda / sc_extension pybind11 modules (reference names)

The native library is built in-tree by ``python -m geo_b200.build``; nothing here falls back to
PyTorch or the CPU when it is missing.
"""
import os
import sys

__all__ = ["install_reference_module_names", "EXT_DIR"]

EXT_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ext")


def install_reference_module_names():
    """Make ``import sc_extension`` and ``import sc_extension_cuda`` (what the reference's
    utils_functional.py:11-12 does at import time) resolve to this package's modules."""
    if EXT_DIR not in sys.path:
        sys.path.insert(0, EXT_DIR)
    import torch  # noqa: F401  (libtorch before the extension modules)
    import sc_extension  # noqa: F401
    import sc_extension_cuda  # noqa: F401
    return sys.modules["sc_extension"], sys.modules["sc_extension_cuda"]
