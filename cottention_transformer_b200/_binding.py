"""Loader of the compiled torch binding (``cott_torch_binding.so``, built from ``csrc_torch/torch_binding.cpp`` by
``python -m cottention_transformer_b200.build``).

The binding is a thin C++ layer over the same C ABI that ``_lib`` reaches through ctypes: the reference's four
``FastAttention2.kernel`` functions with their pybind signature, and the fused operators as ``torch.ops.cottention_b200.*``.
When the file is there the package uses it (fewer Python-level calls per step); when it is not, the ctypes route does
the same work -- both end in the same CUDA kernels, neither is a fallback off the GPU.
"""
from __future__ import annotations

import importlib.util
import os

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cott_torch_binding.so")
_mod = None
_tried = False


def module():
    """The compiled module, or None when it has not been built."""
    global _mod, _tried
    if not _tried:
        _tried = True
        if os.path.exists(_PATH) and os.environ.get("COTT_NO_TORCH_BINDING", "") != "1":
            import torch  # noqa: F401  (libtorch must be loaded first)
            spec = importlib.util.spec_from_file_location("cott_torch_binding", _PATH)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)  # also registers torch.ops.cottention_b200.*
            _mod = mod
    return _mod


def ops():
    """``torch.ops.cottention_b200`` when the binding is loaded, else None."""
    if module() is None:
        return None
    import torch
    return torch.ops.cottention_b200
