"""CPU tests of the C-ABI library: it loads and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = []
    for f in sorted(os.listdir(os.path.join(REPO, "include"))):
        if not f.endswith(".h"):
            continue
        src = open(os.path.join(REPO, "include", f)).read()
        src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
        names += re.findall(r"\b(cott_[a-z0-9_]+)\s*\(", src)
    return sorted(set(names))


@pytest.fixture(scope="module")
def lib():
    from cottention_transformer_b200 import build
    return ctypes.CDLL(build.build())


def test_header_declares_entry_points():
    d = _declared()
    assert "cott_scan" in d and "cott_scan_bwd" in d and "cott_version" in d


def test_library_exports_every_declared_symbol(lib):
    for name in _declared():
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"


def test_python_binding_covers_every_declared_symbol():
    from cottention_transformer_b200 import _lib
    assert sorted(_lib.exported_symbols()) == _declared()


def test_version_and_status_strings(lib):
    lib.cott_version.restype = ctypes.c_char_p
    assert b"sm_100a" in lib.cott_version()
    lib.cott_status_string.restype = ctypes.c_char_p
    assert lib.cott_status_string(0) == b"ok"
    assert lib.cott_status_string(2) == b"unsupported shape"


def test_argument_validation_needs_no_gpu(lib):
    """Bad arguments are rejected before any CUDA call."""
    lib.cott_last_error.restype = ctypes.c_char_p
    P = ctypes.c_void_p
    lib.cott_scan.argtypes = [P, P, P, P] + [ctypes.c_int] * 7 + [P]
    assert lib.cott_scan(None, None, None, None, 1, 1, 8, 24, 16, 0, 0, None) == 2  # Dk % 16
    assert b"divisible by 16" in lib.cott_last_error()
    assert lib.cott_scan(None, None, None, None, 1, 1, 8, 32, 16, 9, 0, None) == 3  # dtype
    assert lib.cott_scan(None, None, None, None, 1, 1, 8, 32, 16, 0, 0, None) == 1  # null
    assert lib.cott_scan(None, None, None, None, 0, 1, 8, 32, 16, 0, 0, None) == 0  # empty: nothing to do


def test_rotary_arguments_are_checked_without_a_gpu():
    """``cott_cos_attn_fwd_rotary``: the rotary descriptor is validated before any pointer is touched."""
    from cottention_transformer_b200 import _lib
    L = _lib.lib()
    buf = (ctypes.c_float * 64)()
    addr = ctypes.addressof(buf)
    addr += (-addr) % 16  # 16-byte aligned inside the buffer

    def call(rot):
        return L.cott_cos_attn_fwd_rotary(None, None, None, None, None, None, None, None, None if rot is None else ctypes.byref(rot),
                                          1, 2, 128, 64, 64, 3, None)

    assert call(None) == 1                                                     # no descriptor
    assert call(_lib.CottRotaryTables(None, None, 64, 0)) == 1                 # null tables
    assert call(_lib.CottRotaryTables(addr, addr, 24, 0)) == 2                 # rotary dim not a multiple of 16
    assert b"multiple of 16" in L.cott_last_error()
    assert call(_lib.CottRotaryTables(addr, addr, 128, 0)) == 2                # wider than the head
    assert call(_lib.CottRotaryTables(addr + 4, addr, 64, 0)) == 5             # misaligned table
    assert call(_lib.CottRotaryTables(addr, addr, 64, 6)) == 5                 # batch stride not a multiple of 4
    assert L.cott_cos_attn_fwd_rotary(None, None, None, None, None, None, None, None, None, 1, 2, 128, 128, 128, 3, None) == 7  # head dim 128


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from cottention_transformer_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.lib()


def test_dropin_names_import():
    import sys
    sys.path.insert(0, os.path.join(REPO, "cottention_transformer_b200", "dropin"))
    try:
        import FastAttention   # the extension's older name
        import FastAttention2
        from FastAttention2 import kernel
        from Custom_Kernel import CustomAttention
        assert all(hasattr(kernel, n) for n in ("float32", "float64", "float16", "bfloat16"))
        assert hasattr(FastAttention2, "kernel") and hasattr(CustomAttention, "apply")
        assert FastAttention.kernel is FastAttention2.kernel
    finally:
        sys.path.pop(0)


def test_kernel_rejects_cpu_tensors_like_the_reference():
    import torch
    from cottention_transformer_b200 import kernel
    x = torch.zeros(1, 1, 4, 32)
    with pytest.raises(RuntimeError, match="Q must be a CUDA tensor"):
        kernel.float32(x, x, x, 1, False, False)


def test_segment_plan_is_host_arithmetic(lib):
    """cott_cos_attn_seg_count / _seg_workspace_bytes need no GPU: few sequences and a long N get segments
    (148 SMs assumed when no device answers), many sequences or short ones do not."""
    L = lib
    L.cott_cos_attn_seg_workspace_bytes.restype = ctypes.c_size_t
    assert L.cott_cos_attn_seg_count(8, 16, 4096) == 1          # 128 sequences: one per SM already
    assert L.cott_cos_attn_seg_count(1, 16, 262144) == 9        # 16 heads -> 9 segments each (144 CTAs)
    assert L.cott_cos_attn_seg_count(1, 1, 256) == 1            # two chunks: nothing to cut
    assert L.cott_cos_attn_seg_count(1, 1, 1024) == 4           # at least two chunks per segment
    n = L.cott_cos_attn_seg_workspace_bytes(1, 16, 262144, 9)
    assert n == 5 * 16 * 9 * 64 * 64 * 4 + 262144 * 4
    # a segment count the sequence cannot use is clamped (1000 tokens = 8 chunks -> at most 8 segments)
    assert L.cott_cos_attn_seg_workspace_bytes(1, 1, 1000, 50) == 5 * 8 * 64 * 64 * 4 + 1000 * 4


def test_package_input_recipe_equals_the_oracles():
    """The benchmark's product arm takes its seeded inputs from the package; the tests take theirs from oracle/.
    Both must be the same tensors for the same seed."""
    import torch
    from cottention_transformer_b200.synthetic import make_inputs
    from oracle import cott_oracle as O
    for kw in (dict(seed=7), dict(seed=1234, normalize=False, dtype=torch.bfloat16)):
        a, b = make_inputs(2, 3, 50, 32, 16, **kw), O.make_inputs(2, 3, 50, 32, 16, **kw)
        assert all(torch.equal(x, y) for x, y in zip(a, b))


def test_compiled_torch_binding_exports_the_reference_signature():
    """The compiled binding (csrc_torch/torch_binding.cpp) registers the reference's four pybind functions
    (combined_kernel_general.cu:444-454) with six arguments in the reference's order, and the fused operators as
    torch.library ops.  No compute: loading and introspection only."""
    import torch
    from cottention_transformer_b200 import _binding, build
    build.build_torch_binding()
    m = _binding.module()
    assert m is not None
    for name in ("float32", "float64", "float16", "bfloat16"):
        doc = getattr(m, name).__doc__
        assert "Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, block_size" in doc and "inplace: bool = False, reversed: bool = False" in doc
    for op in ("causal_fwd", "causal_bwd", "bidir_fwd", "bidir_bwd"):
        assert hasattr(torch.ops.cottention_b200, op)
    with __import__("pytest").raises(RuntimeError, match="Q must be a CUDA tensor"):
        z = torch.zeros(1, 1, 8, 32)
        m.float32(z, z, z, 1, False, False)
    # a failing C call becomes a RuntimeError with the status text (this also runs the binding's string formatting,
    # which a statically linked second copy of the C++ runtime once crashed)
    m._raise_for_status(0)
    with __import__("pytest").raises(RuntimeError, match=r"cottention_b200: unsupported shape \(2\)"):
        m._raise_for_status(2)
