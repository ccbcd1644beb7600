"""Every function declared in include/*.h is exported by the library that header describes, and the ABI versions are the
reference's.  Loads the libraries only; no device call is made."""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
LIBS = {"flagrot_kernels.h": ("libflagrot_kernels.so", "fr_abi_version", 9),
        "flagrot_kivi.h": ("libflagrot_kivi.so", "kv_abi_version", 9),
        "flagrot_mq.h": ("libflagrot_mq.so", "frmq_abi_version", 7)}


def declared(header: Path):
    text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    return sorted(set(re.findall(r"\b((?:fr|kv|frmq)_[a-z0-9_]+)\s*\(", text)))


@pytest.mark.parametrize("header", sorted(LIBS))
def test_header_symbols_exported(header):
    so, abi_fn, abi = LIBS[header]
    path = ROOT / "flagrot_releaser_b200" / "lib" / so
    assert path.exists(), f"{path} missing: run python -m flagrot_releaser_b200._build"
    lib = ctypes.CDLL(str(path))
    names = declared(ROOT / "include" / header)
    assert len(names) >= 7, names
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    fn = getattr(lib, abi_fn)
    fn.restype = ctypes.c_int
    assert fn() == abi
