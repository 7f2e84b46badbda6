"""The C-ABI library loads and exports every symbol include/nb_b200.h declares (no GPU needed)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    hdr = open(os.path.join(ROOT, "include", "nb_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    return sorted(set(re.findall(r"\b(nb_[a-z0-9_]+)\s*\(", hdr)))


def test_library_exports_every_declared_symbol():
    """libnb_b200.so exports the compute entry points, libnb_b200_comm.so the NCCL layer at the end of the header."""
    from neutronbench_b200 import _lib
    lib, comm = _lib.load(), _lib.load_comm()
    names = _declared()
    assert len(names) >= 20
    for n in names:
        where = comm if n in _lib.COMM_SIGNATURES else lib
        assert hasattr(where, n), f"{n} is declared in include/nb_b200.h but not exported"


def test_binding_table_matches_header():
    from neutronbench_b200 import _lib
    assert sorted(list(_lib.SIGNATURES) + list(_lib.COMM_SIGNATURES)) == _declared()


def test_argument_counts_match_header():
    from neutronbench_b200 import _lib
    hdr = open(os.path.join(ROOT, "include", "nb_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    for name, args in re.findall(r"\b(nb_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", hdr, flags=re.S):
        n = 0 if args.strip() in ("", "void") else args.count(",") + 1
        table = _lib.COMM_SIGNATURES if name in _lib.COMM_SIGNATURES else _lib.SIGNATURES
        assert len(table[name][1]) == n, name


def test_missing_library_fails_loudly(monkeypatch):
    from neutronbench_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libnb_b200.so")
    with pytest.raises(ImportError, match="no CPU fallback"):
        _lib.load()


def test_no_device_is_an_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    from neutronbench_b200 import _lib
    lib = _lib.load()
    h = C.c_void_p()
    st = lib.nb_ws_create(C.byref(h), None, 1 << 20)
    assert st == -2  # NB_ERR_CUDA
    assert b"cuda" in lib.nb_last_error().lower()


def test_argument_validation_needs_no_device():
    from neutronbench_b200 import _lib
    lib = _lib.load()
    assert lib.nb_spmm_csc_fwd(None, None, None, None, None, 4, 8, None) == -1
    assert lib.nb_gemm(None, 1, 1, 1, 4, 4, 4, 1, 1, None) == -1   # TT unsupported
    assert lib.nb_spmm_csc_fwd(None, None, None, None, None, 0, 8, None) == 0   # empty block is a no-op
    assert lib.nb_version() >= 100
