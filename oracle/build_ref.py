"""Test infrastructure: compile the reference's own CUDA extension for sm_100a.

The sources are compiled where they lie (``<reference>/Cuda_Kernel/combined_kernel_general.cu``,
the only file ``Cuda_Kernel/setup.py:13-15`` builds) and nothing but build products is
written, all of it under ``oracle/_ref/``.  The result is a package directory
``oracle/_ref/FastAttention2/`` holding ``kernel.so`` (module name ``kernel``, the
``TORCH_EXTENSION_NAME`` the reference's pybind block registers, ``combined_kernel_general.cu:444``)
and a generated one-line ``__init__.py``.

Only tests and the parity section of the benchmark import the product of this
script; it is the checker, never the thing measured or shipped.

Usage:  python oracle/build_ref.py [--reference /path/to/Cottention_Transformer]
"""
import argparse
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def build(reference_root: str, verbose: bool = False) -> str:
    src = os.path.join(reference_root, "Cuda_Kernel", "combined_kernel_general.cu")
    if not os.path.isfile(src):
        raise FileNotFoundError(src)
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0a"
    os.environ.setdefault("MAX_JOBS", "4")
    from torch.utils.cpp_extension import load

    pkg = os.path.join(OUT, "FastAttention2")
    bld = os.path.join(OUT, "build")
    os.makedirs(pkg, exist_ok=True)
    os.makedirs(bld, exist_ok=True)
    load(
        name="kernel",
        sources=[src],
        build_directory=bld,
        extra_cuda_cflags=["-O3", "-lineinfo"],
        is_python_module=False,
        verbose=verbose,
    )
    so = os.path.join(bld, "kernel.so")
    shutil.copy2(so, os.path.join(pkg, "kernel.so"))
    with open(os.path.join(pkg, "__init__.py"), "w") as f:
        f.write("import torch  # noqa: F401  (loads libtorch before the extension)\nfrom . import kernel  # noqa: F401\n")
    copy_modules(reference_root)
    return pkg


def copy_modules(reference_root: str) -> str:
    """The reference's GPT attention module, byte for byte, for the drop-in test (it is imported there with this
    library's Custom_Kernel / FastAttention2 shims first on sys.path).  Git-ignored like everything under _ref/."""
    mods = os.path.join(OUT, "reference_modules")
    os.makedirs(mods, exist_ok=True)
    shutil.copy2(os.path.join(reference_root, "GPT_Trainer", "GPTCosAttention.py"), os.path.join(mods, "GPTCosAttention.py"))
    return mods


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("COTT_REFERENCE_ROOT"), required="COTT_REFERENCE_ROOT" not in os.environ,
                    help="path of the reference checkout (or set COTT_REFERENCE_ROOT)")
    ap.add_argument("-v", "--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.reference, a.verbose))
    sys.exit(0)
