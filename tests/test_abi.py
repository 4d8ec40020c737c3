"""CPU: the C-ABI library builds, loads, and exports every symbol include/rotor_b200.h declares.
No compute call is made here (there is no GPU)."""
import ctypes
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "rotor_b200.h")
LIB = os.path.join(ROOT, "rotor-rag_b200", "rotor_b200", "librotor_b200.so")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"^\s*#.*$", "", text, flags=re.M)          # preprocessor lines are not declarations
    return sorted(set(re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{]*\)\s*;", text)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(LIB):
        subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "rotor-rag_b200", "csrc")])
    return ctypes.CDLL(LIB)


def test_header_declares_functions():
    names = declared_functions()
    assert "rotor_b200_bitlinear_acc" in names and "bitnet_to_rotor" in names
    assert len(names) >= 20


def test_every_declared_symbol_is_exported(lib):
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_python_binding_matches_header():
    from rotor_b200 import abi
    bound = set(abi._SIGNATURES)
    declared = set(declared_functions())
    assert declared <= bound, f"header functions without a ctypes signature: {sorted(declared - bound)}"
    assert bound <= declared, f"ctypes signatures without a header declaration: {sorted(bound - declared)}"


def test_pure_host_queries(lib):
    lib.rotor_b200_tiles_bytes.restype = ctypes.c_size_t
    lib.rotor_b200_tiles_bytes.argtypes = [ctypes.c_size_t, ctypes.c_size_t]
    assert lib.rotor_b200_tiles_bytes(6912, 2560) == 6912 * 2560 // 4
    assert lib.rotor_b200_tiles_bytes(20, 72) == 32 * 128 // 4      # padded to 32 x 128
    lib.rotor_b200_status_string.restype = ctypes.c_char_p
    assert lib.rotor_b200_status_string(0) == b"ok"
    assert lib.rotor_b200_version() >= 100


def test_argument_errors_do_not_need_a_gpu(lib):
    # null pointers and zero sizes are rejected before any CUDA call
    lib.rotor_b200_bitlinear_acc.restype = ctypes.c_int
    lib.rotor_b200_bitlinear_acc.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_void_p,
                                             ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_int,
                                             ctypes.c_void_p]
    assert lib.rotor_b200_bitlinear_acc(None, 16, 128, None, None, 1, None, 0, None) == 1
    lib.rotor_b200_pack.restype = ctypes.c_int
    lib.rotor_b200_pack.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p]
    assert lib.rotor_b200_pack(None, None, 6, None, None) == 1      # length must be a multiple of 4
