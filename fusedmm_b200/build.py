"""Builds ``fusedmm_b200/lib/libfusedmm_b200.so`` from ``fusedmm_b200/csrc/*.cu`` with nvcc for sm_100a.

The translation units (one per message pattern and value type, plus the C ABI) are compiled in parallel
and linked into one shared library that sits in the source tree.  ``python -m fusedmm_b200.build`` runs it.
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
OBJDIR = PKG.parent / "build" / "obj"
LIB = LIBDIR / "libfusedmm_b200.so"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (cand == "nvcc" or Path(cand).exists()):
            return cand
    raise RuntimeError("nvcc not found")


def _newer(target: Path, deps) -> bool:
    return target.exists() and all(target.stat().st_mtime >= d.stat().st_mtime for d in deps)


def _embed_kernel_source() -> Path:
    """Writes the text of csrc/fusedmm_kernels.cuh as a C++ string constant (build/obj/fusedmm_kernels_src.h):
    fusedmm_jit.cu hands that text to NVRTC at run time to build kernels for messages that have no built-in one."""
    src = (CSRC / "fusedmm_kernels.cuh").read_text()
    delim = "FMMKSRC"
    assert f"){delim}\"" not in src
    # string literals have a length limit in some front ends: emit pieces of at most 8 KB, concatenated by the compiler
    pieces, pos = [], 0
    while pos < len(src):
        end = min(len(src), pos + 8000)
        if end < len(src):
            end = src.rfind("\n", pos, end) + 1 or end
        pieces.append(f'R"{delim}({src[pos:end]}){delim}"')
        pos = end
    text = ("// generated from csrc/fusedmm_kernels.cuh by fusedmm_b200/build.py; do not edit\n"
            "static const char kKernelsSource[] =\n" + "\n".join(pieces) + ";\n")
    out = OBJDIR / "fusedmm_kernels_src.h"
    if not out.exists() or out.read_text() != text:
        out.write_text(text)
    return out


def build(force: bool = False, verbose: bool = False, extra_flags=()) -> Path:
    """Compile what is out of date and link.  Returns the path of the shared library."""
    extra_flags = tuple(extra_flags) + tuple(os.environ.get("FUSEDMM_B200_NVCC_FLAGS", "").split())
    OBJDIR.mkdir(parents=True, exist_ok=True)
    LIBDIR.mkdir(parents=True, exist_ok=True)
    embedded = _embed_kernel_source()
    extra_flags = extra_flags + ("-I", str(OBJDIR))
    headers = sorted(CSRC.glob("*.cuh")) + sorted((PKG.parent / "include").glob("*.h")) + [embedded]
    sources = sorted(CSRC.glob("*.cu"))
    nvcc = _nvcc()
    jobs = []
    for src in sources:
        obj = OBJDIR / (src.stem + ".o")
        if force or not _newer(obj, [src] + headers):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [nvcc, *NVCC_FLAGS, *extra_flags, "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        if verbose and (r.stdout or r.stderr):
            print(r.stdout, r.stderr, file=sys.stderr)
        return obj

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            list(ex.map(compile_one, jobs))
    objs = [OBJDIR / (s.stem + ".o") for s in sources]
    if force or jobs or not _newer(LIB, objs):
        tmp = LIB.with_suffix(f".{os.getpid()}.tmp")
        cmd = [nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
