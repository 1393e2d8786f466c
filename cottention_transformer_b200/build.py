"""Build recipe for the native library: one nvcc invocation per translation unit, sm_100a only.

    python -m cottention_transformer_b200.build [--force] [-v]

produces ``cottention_transformer_b200/libcottention_b200.so`` next to this file.  The library has
a plain C ABI (``include/cottention_b200.h``) and links the CUDA runtime statically, so it can be
loaded from any host language.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libcottention_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _newest_dep() -> float:
    t = os.path.getmtime(os.path.join(PKG, "..", "include", "cottention_b200.h"))
    for f in os.listdir(CSRC):
        t = max(t, os.path.getmtime(os.path.join(CSRC, f)))
    return t


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest_dep():
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    srcs = sources()

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        log = os.path.join(OBJ, os.path.basename(src)[:-3] + ".ptxas.log")
        with open(log, "w") as f:
            f.write(r.stderr)
        if verbose or r.returncode != 0:
            sys.stderr.write(r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(compile_one, srcs))
    cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *objs]
    subprocess.check_call(cmd)
    return LIB


BINDING = os.path.join(PKG, "cott_torch_binding.so")


def build_torch_binding(force: bool = False, verbose: bool = False) -> str:
    """Compile ``csrc_torch/torch_binding.cpp`` (host C++ only: the compiled torch binding over the C ABI) next to the
    library it links, ``cott_torch_binding.so``.  Needs the library itself to exist."""
    src = os.path.join(PKG, "csrc_torch", "torch_binding.cpp")
    hdr = os.path.join(PKG, "..", "include", "cottention_b200.h")
    if not force and os.path.exists(BINDING) and os.path.getmtime(BINDING) >= max(os.path.getmtime(src), os.path.getmtime(hdr)):
        return BINDING
    build(force=False)
    from torch.utils.cpp_extension import load
    bld = os.path.join(OBJ, "torch_binding")
    os.makedirs(bld, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")  # no device code here; silences the arch probe on CPU-only hosts
    # Link the C++ runtime the process already runs on, by name.  (Some toolchain layouts resolve -lstdc++ to the static
    # archive; a second, uninitialised copy of the iostream machinery inside the binding crashes on first use.)
    import torch  # noqa: F401
    stdcpp = []
    with open("/proc/self/maps") as f:
        for line in f:
            if "libstdc++.so" in line:
                stdcpp = [f"-L{os.path.dirname(line.split()[-1])}", "-l:libstdc++.so.6"]
                break
    load(name="cott_torch_binding", sources=[src], build_directory=bld, with_cuda=True, is_python_module=False, verbose=verbose,
         extra_cflags=["-O2"], extra_ldflags=[*stdcpp, f"-L{PKG}", "-l:libcottention_b200.so", "-Wl,-rpath,'$$ORIGIN'", "-Wl,-rpath,'$$ORIGIN/../..'"])  # ($$: ninja's escape for a literal $)
    shutil.copy2(os.path.join(bld, "cott_torch_binding.so"), BINDING)
    return BINDING


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("-v", "--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
    print(build_torch_binding(a.force, a.verbose))
