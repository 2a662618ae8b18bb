"""Build the sm_100a kernel library in-tree with nvcc.

``python -m cppmega_b200.ops.cuda.build`` compiles every ``csrc/*.cu`` for
``compute_100a/sm_100a`` and links ``libcppmega_b200_kernels.so`` next to this file.  No GPU
is needed to build.  Objects are rebuilt only when their source (or a header) is newer.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path
from typing import List

HERE = Path(__file__).resolve().parent
CSRC = HERE.parent / "csrc"
BUILD = HERE / "_build"
LIB = HERE / "libcppmega_b200_kernels.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def sources() -> List[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale(obj: Path, src: Path, headers: List[Path]) -> bool:
    if not obj.exists():
        return True
    t = obj.stat().st_mtime
    return any(p.stat().st_mtime > t for p in [src, *headers])


def _compile(nvcc: str, src: Path, obj: Path, verbose: bool) -> str:
    cmd = [nvcc, *NVCC_FLAGS, "-Xptxas", "-v", "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    (obj.with_suffix(".ptxas.txt")).write_text(r.stderr)
    return r.stderr if verbose else ""


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = nvcc_path()
    BUILD.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    srcs = sources()
    objs = [BUILD / (s.stem + ".o") for s in srcs]
    todo = [(s, o) for s, o in zip(srcs, objs) if force or _stale(o, s, headers)]
    if todo:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
            for out in ex.map(lambda so: _compile(nvcc, so[0], so[1], verbose), todo):
                if out:
                    print(out)
    if todo or not LIB.exists():
        cmd = [nvcc, "-shared", "-o", str(LIB), *map(str, objs), "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    lib = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(lib)
