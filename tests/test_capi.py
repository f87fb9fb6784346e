"""The C-ABI library loads without a GPU and exports every symbol the header declares."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "vkgrad_b200.h")


def header_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vkg_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_loads():
    import __graft_entry__ as entry
    path = entry.build()
    assert os.path.exists(path)
    lib = ctypes.CDLL(path)
    lib.vkg_version.restype = ctypes.c_char_p
    assert b"sm_100a" in lib.vkg_version()


def test_every_declared_symbol_is_exported_and_bound():
    from vkgrad_b200 import _lib
    lib = _lib.load()
    declared = header_functions()
    assert len(declared) > 50
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    bound = set(_lib.exported_names())
    assert set(declared) == bound, (set(declared) ^ bound)


def test_gemm_args_layout_matches_header():
    """ctypes mirror of struct vkg_gemm_args: same field order as the header."""
    from vkgrad_b200._lib import GemmArgs
    text = open(HEADER).read()
    body = text[text.index("typedef struct vkg_gemm_args {"):text.index("} vkg_gemm_args;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    names = []
    for decl in body.split(";"):
        decl = decl.replace("typedef struct vkg_gemm_args {", "").strip()
        if not decl:
            continue
        for part in decl.split(","):
            names.append(re.findall(r"([A-Za-z_0-9]+)\s*$", part.strip())[0])
    assert names == [f[0] for f in GemmArgs._fields_]


def test_no_gpu_is_a_clean_error_not_a_fallback():
    """Without a CUDA device the runtime refuses to create a Device."""
    from vkgrad_b200 import _lib, vk
    lib = _lib.load()
    n = ctypes.c_int(-1)
    assert lib.vkg_device_count(ctypes.byref(n)) == 0
    if n.value > 0:
        pytest.skip("a GPU is present")
    with pytest.raises(vk.VkError, match="no CUDA device|no CPU fallback"):
        vk.Device()


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "vkgrad_b200")
    for fn in os.listdir(pkg):
        if fn.endswith(".py"):
            src = open(os.path.join(pkg, fn)).read()
            assert "oracle" not in src, f"{fn} mentions the oracle"
