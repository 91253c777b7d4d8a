"""Builds ``libmono_b200.so`` (the C-ABI kernel library) in-tree with nvcc for sm_100a.

``python -m sgl_amd_mono_b200.build`` or ``build_library()``.  nvcc cross-compiles
without a GPU.  The reference has no build step (its kernels are JIT-compiled by
FlyDSL at server start, ``common/plan.py:175-201``); here the library is compiled
once, ahead of time, and the spec refuses to attach when it is missing.
"""

from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libmono_b200.so"
STAMP = PKG / "csrc" / ".build_stamp"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _flags() -> list[str]:
    # MONO_TIMELINE=1: kernels record global-timer stamps at numbered points (csrc/mono_common.cuh)
    # (MONO_TIMELINE_DEFS: further -D switches of a stamped build, space separated)
    if os.environ.get("MONO_TIMELINE") != "1":
        return NVCC_FLAGS
    return NVCC_FLAGS + ["-DMONO_TIMELINE"] + [f"-D{d}" for d in os.environ.get("MONO_TIMELINE_DEFS", "").split()]


def _digest() -> str:
    h = hashlib.sha256()
    for p in sources() + sorted(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "mono_b200.h"]:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(_flags()).encode())
    return h.hexdigest()


def build_library(force: bool = False, verbose: bool = False) -> Path:
    digest = _digest()
    if not force and LIB.exists() and STAMP.exists() and STAMP.read_text().strip() == digest:
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objs = []
    build_dir = PKG / "csrc" / "build"
    build_dir.mkdir(exist_ok=True)
    procs = []
    for src in sources():
        obj = build_dir / (src.stem + ".o")
        cmd = [nvcc, *_flags(), "-c", str(src), "-o", str(obj)]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    log = []
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        log.append(f"== {src.name}\n{out}")
        failed |= p.returncode != 0
    (build_dir / "ptxas.log").write_text("\n".join(log))
    if failed or verbose:
        print("\n".join(log), file=sys.stderr)
    if failed:
        raise RuntimeError("nvcc failed; see the log above")
    cmd = [nvcc, "-shared", "-o", str(LIB), *map(str, objs)]
    subprocess.run(cmd, check=True)
    STAMP.write_text(digest)
    return LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
