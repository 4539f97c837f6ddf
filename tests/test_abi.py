"""The C-ABI library builds for sm_100a, loads, and exports every symbol the header declares.
No compute call is made here (there is no GPU on the machines that run this file)."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from switchyard_b200 import build, _lib
    build.build()
    return _lib.load()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "switchyard_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sy_\w+)\s*\(", text)))


def test_header_and_binding_agree(lib):
    from switchyard_b200 import _lib
    assert declared_symbols() == sorted(_lib.SYMBOLS)


def test_every_declared_symbol_is_exported(lib):
    for name in declared_symbols():
        assert getattr(lib, name) is not None, name


def test_version_and_argument_errors(lib):
    assert b"sm_100a" in lib.sy_version()
    # argument checks run before anything touches a device
    rc = lib.sy_route(None, 4, 200, 8, 0, 0, None, None, None)
    assert rc == -1 and b"128 experts" in lib.sy_last_error()
    rc = lib.sy_combine(None, None, None, 4, 9, 64, None, 0, None)
    assert rc == -1 and b"top_k" in lib.sy_last_error()
    rc = lib.sy_grouped_gemv(None, None, None, None, 64, 8, 100, 64, 0, None, None, 0, None)
    assert rc == -1 and b"multiple of 8" in lib.sy_last_error()
    rc = lib.sy_grouped_gemm(None, None, None, None, 64, 8, 64, 60, 0, None, None, 0, None)
    assert rc == -1 and b"multiple of 8" in lib.sy_last_error()
    assert lib.sy_sort_scratch_bytes(512, 64) == 0
    assert lib.sy_sort_scratch_bytes(65536, 64) > 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from switchyard_b200 import _lib
    monkeypatch.setattr(_lib, "_LIB", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()


def test_no_cpu_fallback_in_expert_parallel():
    from switchyard_b200.ep import ExpertParallel
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        ExpertParallel(["cpu", "cpu"], 4, 2, False)
