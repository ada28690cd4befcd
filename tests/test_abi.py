"""The C-ABI library loads and exports every symbol include/axiom_b200.h declares.
No compute call is made: this runs without a GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from axiom_b200 import build
    return ctypes.CDLL(build.build())


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "axiom_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(axb_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    names = declared_symbols()
    assert len(names) >= 25
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_python_binding_lists_the_same_symbols():
    from axiom_b200.engine import EXPORTS
    assert sorted(EXPORTS) == declared_symbols()


def test_no_gpu_means_loud_failure(lib):
    """Without a device the engine reports AX_ERR_BACKEND; it never computes on the host."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib.axb_last_error.restype = ctypes.c_char_p
    assert lib.axb_init(0) == 9
    assert b"CUDA" in lib.axb_last_error() or b"device" in lib.axb_last_error()
    buf = (ctypes.c_float * 4)()
    st = lib.axb_gemm(buf, buf, buf, ctypes.c_int64(2), ctypes.c_int64(2), ctypes.c_int64(2))
    assert st == 9


def test_missing_library_raises(tmp_path):
    from axiom_b200.engine import Engine
    with pytest.raises(FileNotFoundError):
        Engine(so_path=str(tmp_path / "nope.so"))
