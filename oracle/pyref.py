"""TEST / BENCH INFRASTRUCTURE ONLY: loads the byte code of the reference's own ctypes front ends
(integrations/vllm_flagrot/vllm_flagrot/kernels.py, kivi.py, prefill_mq.py), compiled by oracle/build_ref.sh from the
sources where they lie into oracle/_ref/pyref/*.bytecode (git-ignored build output; plain files, so that they travel with
the rest of oracle/_ref).  The modules are executed unmodified; they read FLAGROT_LIB / FLAGROT_KIVI_LIB / FLAGROT_MQ_LIB /
FLAGROT_NO_REBUILD from the environment like the originals.  Nothing in the product imports this module."""
from __future__ import annotations

import marshal
import os
import sys
import types
from pathlib import Path

DIR = Path(__file__).resolve().parent / "_ref" / "pyref"
NAMES = ("kernels", "kivi", "prefill_mq")


def available() -> bool:
    return all((DIR / f"{n}.bytecode").exists() for n in NAMES)


def load(name: str, libs: dict | None = None):
    """the reference module `name` (a fresh instance is cached in sys.modules as vllm_flagrot_ref.<name>).  libs: environment
    variables (FLAGROT_LIB ...) set before the module body runs."""
    assert name in NAMES, name
    full = f"vllm_flagrot_ref.{name}"
    if full in sys.modules:
        return sys.modules[full]
    for k, v in (libs or {}).items():
        os.environ[k] = str(v)
    os.environ.setdefault("FLAGROT_NO_REBUILD", "1")
    data = (DIR / f"{name}.bytecode").read_bytes()
    code = marshal.loads(data[16:])                      # a .pyc body: 16 header bytes, then the marshalled code object
    mod = types.ModuleType(full)
    mod.__file__ = str(DIR / "vllm_flagrot" / f"{name}.py")
    sys.modules[full] = mod
    try:
        exec(code, mod.__dict__)
    except BaseException:
        del sys.modules[full]
        raise
    return mod
