"""The shared library loads without a GPU and exports every function that
include/fhert_b200.h declares; the Python binding knows each of them."""
import ctypes
import os
import re

import ace_compiler_b200 as rt

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "fhert_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"typedef\s+(struct|enum)\s*\{.*?\}\s*\w+\s*;", "", text, flags=re.S)
    text = re.sub(r"enum\s*\{.*?\}\s*;", "", text, flags=re.S)
    text = re.sub(r"^#define[^\n]*(\\\n[^\n]*)*", "", text, flags=re.M)  # macros are not symbols
    names = re.findall(r"\b([A-Z][A-Za-z0-9_]*)\s*\([^;{}]*\)\s*;", text)
    return sorted(set(names))


def test_header_functions_are_exported_and_bound():
    names = declared_functions()
    assert len(names) > 60
    lib = ctypes.CDLL(rt.LIB_PATH)
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared but not exported: {missing}"
    unbound = [n for n in names if n not in rt.SIGNATURES]
    assert not unbound, f"declared but missing from the Python binding: {unbound}"


def test_struct_layout_matches_abi():
    assert ctypes.sizeof(rt.MODULUS) == 48
    assert ctypes.sizeof(rt.POLYNOMIAL) == 48
    assert rt.POLYNOMIAL._data.offset == 40
    assert ctypes.sizeof(rt.CIPHERTEXT) == 2 * 48 + 24
