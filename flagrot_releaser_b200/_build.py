"""In-tree build of the CUDA libraries for sm_100a (nvcc cross-compiles without a GPU).

    python -m flagrot_releaser_b200._build [--force]

Outputs flagrot_releaser_b200/lib/libflagrot_kernels.so (and the other libraries as they are added), linked against
the static CUDA runtime like the reference's libraries (integrations/vllm_flagrot/csrc/build.sh:29).
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "lib"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-O3", "-std=c++17", *ARCH, "--expt-relaxed-constexpr", "-lineinfo", "-Xcompiler", "-fPIC", f"-I{CSRC}"]

LIBS = {
    "libflagrot_kernels.so": ["fr_capi.cu", "fr_writer.cu", "fr_decode.cu", "fr_dequant.cu", "fr_xchg.cu"],
    "libflagrot_kivi.so": ["kv_capi.cu"],
    "libflagrot_mq.so": ["mq_capi.cu"],
    # test-only: known-answer kernels for the tcgen05 primitives of csrc/fr_tc5.cuh (not part of any C ABI)
    "libflagrot_tc5test.so": ["fr_tc5_selftest.cu"],
}


def _deps(src: Path):
    return [src, *CSRC.glob("*.cuh"), *CSRC.glob("*.h"), *(PKG.parent / "include").glob("*.h")]


def _stale(out: Path, deps) -> bool:
    return not out.exists() or any(d.stat().st_mtime > out.stat().st_mtime for d in deps if d.exists())


def _compile(src: Path, obj: Path, verbose: bool):
    cmd = [NVCC, *FLAGS, "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    return r.stderr


def build(force: bool = False, verbose: bool = False) -> dict:
    LIBDIR.mkdir(exist_ok=True)
    objdir = LIBDIR / "obj"
    objdir.mkdir(exist_ok=True)
    jobs, logs = [], {}
    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        for lib, srcs in LIBS.items():
            for s in srcs:
                src, obj = CSRC / s, objdir / (s + ".o")
                if not src.exists():
                    continue
                if force or _stale(obj, _deps(src)):
                    jobs.append((s, ex.submit(_compile, src, obj, verbose)))
        for s, j in jobs:
            logs[s] = j.result()
    built = {}
    for lib, srcs in LIBS.items():
        objs = [objdir / (s + ".o") for s in srcs if (CSRC / s).exists()]
        if not objs:
            continue
        out = LIBDIR / lib
        if force or _stale(out, objs):
            r = subprocess.run([NVCC, "-shared", *ARCH, "-cudart", "static", "-o", str(out), *map(str, objs)],
                               capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"link failed for {lib}:\n{r.stdout}\n{r.stderr}")
        built[lib] = out
    if verbose:
        for s, lg in logs.items():
            print(f"== {s}\n{lg}")
    return built


if __name__ == "__main__":
    b = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    for k, v in b.items():
        print(k, v.stat().st_size)
