"""Launch preflight: check, before any training step, that the kernel library fits the device it will run on.

The reference scans its generated kernels for a shared-memory merge flag and probes the device's opt-in shared
memory, failing hard on parts where the big kernels cannot launch (cppmega/megatron/preflight_smem_check.py:100-350
static scan, :352-474 runtime probe).  The equivalents here:

* static: parse the ``ptxas -v`` reports written by the in-tree build (registers, spills, static shared memory per
  kernel) and the dynamic shared-memory requests declared by the sources, and compare them with the sm_100 limits
  (227 KB dynamic shared memory per CTA, 255 registers per thread, 512 TMEM columns per SM);
* runtime: query the device (compute capability 10.x, opt-in shared memory per block, SM count) and refuse to start
  on anything that is not a Blackwell data-centre part, where ``tcgen05`` does not exist.

``python -m cppmega_b200.utils.preflight`` prints the report and exits non-zero on a violation.
"""
from __future__ import annotations

import re
import sys
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional

SM100_MAX_DYNAMIC_SMEM = 227 * 1024
SM100_MAX_REGS = 255
SM100_TMEM_COLS = 512

_BUILD = Path(__file__).resolve().parent.parent / "ops" / "cuda" / "_build"
_CSRC = Path(__file__).resolve().parent.parent / "ops" / "csrc"


@dataclass
class KernelResources:
    name: str
    registers: int = 0
    static_smem: int = 0
    spill_stores: int = 0
    spill_loads: int = 0
    stack: int = 0


@dataclass
class PreflightReport:
    kernels: List[KernelResources] = field(default_factory=list)
    problems: List[str] = field(default_factory=list)
    warnings: List[str] = field(default_factory=list)
    device: Dict[str, object] = field(default_factory=dict)

    @property
    def ok(self) -> bool:
        return not self.problems

    def render(self) -> str:
        lines = [f"{len(self.kernels)} kernels checked"]
        if self.device:
            lines.append("device: " + ", ".join(f"{k}={v}" for k, v in self.device.items()))
        lines += [f"WARNING: {w}" for w in self.warnings]
        lines += [f"ERROR: {p}" for p in self.problems]
        lines.append("preflight " + ("passed" if self.ok else "FAILED"))
        return "\n".join(lines)


_FUNC = re.compile(r"Compiling entry function '([^']+)'")
_USED = re.compile(r"Used (\d+) registers(?:, used \d+ barriers)?(?:, (\d+) bytes smem)?")
_SPILL = re.compile(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads")


def parse_ptxas(text: str) -> List[KernelResources]:
    out: List[KernelResources] = []
    cur: Optional[KernelResources] = None
    for line in text.splitlines():
        m = _FUNC.search(line)
        if m:
            cur = KernelResources(m.group(1))
            out.append(cur)
            continue
        if cur is None:
            continue
        m = _SPILL.search(line)
        if m:
            cur.stack, cur.spill_stores, cur.spill_loads = int(m.group(1)), int(m.group(2)), int(m.group(3))
        m = _USED.search(line)
        if m:
            cur.registers = int(m.group(1))
            cur.static_smem = int(m.group(2) or 0)
    return out


def static_check(build_dir: Path = _BUILD, spill_limit: int = 64) -> PreflightReport:
    rep = PreflightReport()
    files = sorted(build_dir.glob("*.ptxas.txt")) if build_dir.exists() else []
    if not files:
        rep.warnings.append(f"no ptxas reports under {build_dir}: build the kernel library first")
        return rep
    for f in files:
        for k in parse_ptxas(f.read_text()):
            rep.kernels.append(k)
            if k.registers > SM100_MAX_REGS:
                rep.problems.append(f"{k.name}: {k.registers} registers per thread exceeds {SM100_MAX_REGS}")
            if k.static_smem > 48 * 1024:
                rep.problems.append(f"{k.name}: {k.static_smem} bytes of static shared memory exceeds 48 KB")
            if k.spill_stores > spill_limit:
                rep.warnings.append(f"{k.name}: spills {k.spill_stores} bytes per thread to local memory")
    return rep


_SMEM_FN = re.compile(r"constexpr int (\w*smem\w*)\(\)\s*\{[^}]*\}", re.S)
_TMEM_ALLOC = re.compile(r"tmem_alloc\([^,]+,\s*(\d+)\)")


def source_check(csrc: Path = _CSRC) -> PreflightReport:
    """TMEM budget: a kernel may not allocate more than the SM has."""
    rep = PreflightReport()
    for f in sorted(csrc.glob("*.cu")):
        for m in _TMEM_ALLOC.finditer(f.read_text()):
            cols = int(m.group(1))
            if cols > SM100_TMEM_COLS or cols & (cols - 1) or cols < 32:
                rep.problems.append(f"{f.name}: TMEM allocation of {cols} columns is not a power of two in [32, 512]")
    return rep


def runtime_check(device_index: int = 0) -> PreflightReport:
    rep = PreflightReport()
    try:
        import torch
    except Exception as e:                                       # pragma: no cover
        rep.problems.append(f"torch import failed: {e}")
        return rep
    if not torch.cuda.is_available():
        rep.warnings.append("no CUDA device visible: runtime checks skipped")
        return rep
    p = torch.cuda.get_device_properties(device_index)
    optin = getattr(p, "shared_memory_per_block_optin", 0)
    rep.device = {"name": p.name, "cc": f"{p.major}.{p.minor}", "sms": p.multi_processor_count,
                  "smem_optin": optin, "mem_gb": round(p.total_memory / 2 ** 30, 1)}
    if p.major != 10:
        rep.problems.append(f"{p.name} has compute capability {p.major}.{p.minor}; the kernels are built for sm_100a "
                            "(tcgen05 / TMEM) and cannot run elsewhere")
    if optin and optin < SM100_MAX_DYNAMIC_SMEM:
        rep.problems.append(f"device offers {optin} bytes of opt-in shared memory per block; kernels request up to "
                            f"{SM100_MAX_DYNAMIC_SMEM}")
    return rep


def run_all(device_index: int = 0) -> PreflightReport:
    total = PreflightReport()
    for part in (static_check(), source_check(), runtime_check(device_index)):
        total.kernels += part.kernels
        total.problems += part.problems
        total.warnings += part.warnings
        total.device.update(part.device)
    return total


def main() -> int:
    rep = run_all()
    print(rep.render())
    return 0 if rep.ok else 1


if __name__ == "__main__":
    sys.exit(main())
