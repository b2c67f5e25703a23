"""Build libatrex_fa_sm100.so in-tree with nvcc for sm_100a.

    python build.py            # rebuild only when a source changed
    python build.py --force

The explicit ``-gencode arch=compute_100a,code=sm_100a`` form is required:
``tcgen05`` and the other architecture-specific instructions only assemble for
the ``a`` target.  The reference builds its native code the same way, with an
explicit gencode pair and a content hash as the build identity
(python/atrex/core/compile_cu.py:121-170,267-271); here the library is built
ahead of time so nothing compiles at call time.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
# sources of the sibling operator that ships in the same library (src/nvidia/qsa/sm100)
QSA_CSRC = HERE.parents[1] / "qsa" / "sm100" / "csrc"
REPO_INCLUDE = HERE.parents[4] / "include"
LIB = HERE / "libatrex_fa_sm100.so"
STAMP = HERE / "build" / "stamp.txt"

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo", "--use_fast_math",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def include_dir() -> Path:
    """The C-ABI header lives in the repository's include/ (a wheel ships a copy next to csrc)."""
    for cand in (REPO_INCLUDE, CSRC):
        if (cand / "atrex_fa_sm100.h").is_file():
            return cand
    raise FileNotFoundError("atrex_fa_sm100.h")


def source_hash() -> str:
    h = hashlib.sha256()
    files = (sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + sorted(QSA_CSRC.glob("*.cu"))
             + sorted(include_dir().glob("atrex_*_sm100.h")) + [Path(__file__)])
    for f in files:
        h.update(f.name.encode())
        h.update(f.read_bytes())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    digest = source_hash()
    if not force and LIB.is_file() and STAMP.is_file() and STAMP.read_text().strip() == digest:
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        raise RuntimeError("nvcc not found: cannot build libatrex_fa_sm100.so")
    obj_dir = HERE / "build"
    obj_dir.mkdir(exist_ok=True)
    flags = NVCC_FLAGS + ["-I", str(include_dir()), "-I", str(CSRC)] + (["-Xptxas", "-v"] if verbose else [])
    objs, procs = [], []
    for src in sorted(CSRC.glob("*.cu")) + sorted(QSA_CSRC.glob("*.cu")):
        obj = obj_dir / (src.stem + ".o")
        objs.append(obj)
        procs.append((src, subprocess.Popen([nvcc, *flags, "-c", str(src), "-o", str(obj)],
                                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0 or verbose:
            sys.stderr.write(f"--- {src.name}\n{out}\n")
        failed |= proc.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.check_call([nvcc, "-shared", "-o", str(LIB), *map(str, objs), "-Xcompiler", "-fvisibility=hidden"])
    STAMP.write_text(digest + "\n")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
