"""The C-ABI library without a GPU: it loads, exports every symbol the header declares, the ctypes binding covers
exactly those symbols, and argument validation answers with status codes before anything touches a device."""
import ctypes
import re
from pathlib import Path

import pytest

from conftest import ROOT, pkg

HEADER = ROOT / "include" / "ptj_b200.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(ptj_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    build = pkg("build")
    build.build()
    return pkg("_lib").lib()


def test_header_symbols_are_exported(lib):
    names = declared_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/ptj_b200.h but not exported"


def test_binding_matches_header(lib):
    assert pkg("_lib").exported_symbols() == declared_symbols()


def test_status_strings_and_version(lib):
    assert lib.ptj_version() >= 100
    assert lib.ptj_status_string(0) == b"ok"
    for code in range(-8, 0):
        assert lib.ptj_status_string(code) != b"unknown status"
    assert lib.ptj_status_string(-99) == b"unknown status"


def test_validation_needs_no_device(lib):
    """Bad sizes / null pointers / unknown dtypes are refused up front (negative status, no launch)."""
    before = lib.ptj_launch_count()
    assert lib.ptj_layernorm_fwd(None, None, None, None, 4, 8, 0, None) == -1
    assert lib.ptj_layernorm_fwd(None, None, None, None, -1, 8, 0, None) == -1
    assert lib.ptj_gelu_fwd(None, None, -5, 0, None) == -1
    assert lib.ptj_gelu_fwd(None, None, 0, 0, None) == 0  # empty input is fine
    assert lib.ptj_log_softmax_fwd(None, None, 1, 8, 4, 8, 0, None) == -1  # leading dimension < cols
    assert lib.ptj_dropout(None, None, None, 8, ctypes.c_float(1.5), 1, 0, 0, 0, None) == -1
    assert lib.ptj_adamw(None, None, None, None, None, 6, None, None, 0, 0, 0, 0, 0, 0, 1, 1, None, 0, None) == -1
    assert lib.ptj_gemm(None, None, None, None, None, None, 8, 8, 8, 8, 8, 8, 1, 1, 1, 1, 0, None, 1, None, 0, None) == -1
    assert lib.ptj_layernorm_bwd_scratch_floats(1024, 768) == 128 * 3 * 768  # dgamma, dbeta, optional column sums
    assert lib.ptj_colsum_scratch_floats(0, 10) == 0
    assert lib.ptj_launch_count() == before


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    m = pkg("_lib")
    monkeypatch.setattr(m, "_lib", None)
    monkeypatch.setattr(m, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        m.lib()


def test_cpu_tensors_are_refused():
    import torch
    ops = pkg("operators")
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        ops.t_gelu_fwd_t(torch.zeros(4))
