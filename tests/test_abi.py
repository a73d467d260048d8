"""The C-ABI library loads without a GPU and exports every symbol the public header declares."""
import ctypes
import os
import re

from cuda_mace_b200 import _abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "cuda_mace_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cmace_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(built_library):
    lib = ctypes.CDLL(built_library)
    names = declared_symbols()
    assert len(names) >= 35
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in include/cuda_mace_b200.h but not exported: {missing}"


def test_binding_covers_header(built_library):
    names = set(declared_symbols()) - {"cmace_last_error"}
    assert names == set(_abi.SIGNATURES), names ^ set(_abi.SIGNATURES)


def test_version_and_queries_need_no_gpu(built_library):
    assert _abi.call("cmace_abi_version") == 1
    # pure host arithmetic: chunking rule of the backward scratch
    assert _abi.call("cmace_imp_bwd_scratch_elems", 1000, 128, 0) == 0       # f32, one 128-channel chunk
    assert _abi.call("cmace_imp_bwd_scratch_elems", 1000, 128, 1) == 2 * 16 * 1000  # f64, two chunks
    assert _abi.call("cmace_imp_bwd_scratch_elems", 1000, 96, 0) == 3 * 16 * 1000   # f32, three 32-channel chunks


def test_argument_errors_are_reported_not_raised(built_library):
    lib = _abi.load()
    rc = lib.cmace_imp_fwd_f32(None, None, None, None, None, 4, 4, 33, None, None)
    assert rc == 3  # CMACE_ERR_UNSUPPORTED: channels not a multiple of 32
    assert b"multiple of 32" in lib.cmace_last_error()
    rc = lib.cmace_linear_f32(None, None, None, None, 1, 5, 32, 32, 1.0, None, None)
    assert rc == 1 and b"null" in lib.cmace_last_error()
