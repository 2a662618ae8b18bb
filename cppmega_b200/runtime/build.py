"""Build the host-side C++ runtime (``libcppmega_b200_runtime.so``) in-tree with g++."""
from __future__ import annotations

import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libcppmega_b200_runtime.so"


def build(force: bool = False) -> Path:
    srcs = sorted(CSRC.glob("*.cpp"))
    if not srcs:
        return LIB
    newest = max(p.stat().st_mtime for p in [*srcs, *CSRC.glob("*.h")])
    if LIB.exists() and LIB.stat().st_mtime >= newest and not force:
        return LIB
    cxx = shutil.which("g++") or "g++"
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-pthread", "-o", str(LIB), *map(str, srcs)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"runtime build failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
