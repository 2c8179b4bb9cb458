"""Discovery and the isolated-subprocess runner of the parity gates (the reference's
parity/_modelfree.py:95-111 in small): a gate is a file ``parity/*_test.py``; it passes when it exits 0,
printed ``PARITY-CHECKS: n`` with n > 0, and printed no traceback that it did not account for.  A gate
whose source carries the line ``# parity-gate: gpu`` needs a CUDA device."""

from __future__ import annotations

import re
import subprocess
import sys
from dataclasses import dataclass
from pathlib import Path

PARITY_DIR = Path(__file__).resolve().parent
ROOT = PARITY_DIR.parent
GPU_SENTINEL = "# parity-gate: gpu"


@dataclass
class GateResult:
    name: str
    ok: bool
    checks: int
    why: str
    output: str


def discover() -> dict[str, bool]:
    """gate name -> needs a GPU"""
    return {p.stem: GPU_SENTINEL in p.read_text() for p in sorted(PARITY_DIR.glob("*_test.py"))}


def run_gate(name: str, timeout: int = 600) -> GateResult:
    r = subprocess.run([sys.executable, "-m", f"parity.{name}"], cwd=ROOT, capture_output=True, text=True, timeout=timeout)
    out = r.stdout + r.stderr
    m = re.findall(r"^PARITY-CHECKS: (\d+)\s*$", r.stdout, flags=re.M)
    checks = int(m[-1]) if m else 0
    if r.returncode != 0:
        return GateResult(name, False, checks, f"exit code {r.returncode}", out)
    if checks <= 0:
        return GateResult(name, False, checks, "no positive PARITY-CHECKS line: the gate proved no work", out)
    return GateResult(name, True, checks, "", out)


class Checks:
    """Counts a gate's assertions; ``done()`` prints the proof-of-work line."""

    def __init__(self, gate: str):
        self.gate, self.n = gate, 0

    def ok(self, cond: bool, what: str) -> None:
        if not cond:
            raise AssertionError(f"{self.gate}: {what}")
        self.n += 1

    def done(self) -> None:
        print(f"{self.gate}: all {self.n} checks passed")
        print(f"PARITY-CHECKS: {self.n}")
