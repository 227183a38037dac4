"""Builds the CPU oracle (TEST INFRASTRUCTURE ONLY; never imported by the package).

  oracle/liboracle.so        the C restatement in oracle/oracle.c
  oracle/_ref/libmslref.so   the reference's own emitted RK4 kernel
                             (tests/golden/rk4_lotka_volterra.metal, compiled as
                             C++ where it lies in the reference checkout), built
                             only when that checkout is present

Both use -O2 -ffp-contract=off (no fused multiply-add unless written as fmaf,
no fast-math) so that each float operation rounds exactly once, in source order.
"""

from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ORACLE_LIB = HERE / "liboracle.so"
REF_DIR = HERE / "_ref"
REF_LIB = REF_DIR / "libmslref.so"
# The reference checkout: PALLADIUM_REFERENCE, else a directory named "reference" beside this repository.
REFERENCE_ROOT = Path(os.environ.get("PALLADIUM_REFERENCE", str(HERE.parent.parent / "reference")))
GOLDEN_RK4 = REFERENCE_ROOT / "tests" / "golden" / "rk4_lotka_volterra.metal"

CFLAGS = ["-O2", "-ffp-contract=off", "-fno-fast-math", "-mfma", "-fopenmp", "-fPIC", "-shared",
          "-fvisibility=hidden"]


def _stale(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return True
    built = target.stat().st_mtime
    return any(s.exists() and s.stat().st_mtime > built for s in sources)


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"oracle build failed: {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")


def build_oracle(force: bool = False) -> Path:
    src = HERE / "oracle.c"
    header = HERE.parent / "palladium_b200" / "csrc" / "pd_math.h"
    if force or _stale(ORACLE_LIB, [src, header]):
        _run(["gcc", "-std=c11", *CFLAGS, str(src), "-o", str(ORACLE_LIB), "-lm"])
    return ORACLE_LIB


def build_reference(force: bool = False) -> Path | None:
    """Compile the reference's golden RK4 kernel, if the checkout is here."""
    if not GOLDEN_RK4.exists():
        return REF_LIB if REF_LIB.exists() else None
    src = HERE / "msl_ref.cpp"
    if force or _stale(REF_LIB, [src, GOLDEN_RK4, HERE / "msl_shim" / "metal_stdlib"]):
        REF_DIR.mkdir(exist_ok=True)
        _run(["g++", "-std=c++17", *CFLAGS, "-Wno-attributes", f"-I{HERE / 'msl_shim'}",
              f'-DPD_GOLDEN_RK4="{GOLDEN_RK4}"', str(src), "-o", str(REF_LIB)])
    return REF_LIB


if __name__ == "__main__":
    print(build_oracle(force="-f" in sys.argv))
    print(build_reference(force="-f" in sys.argv))
