"""Build recipe for libpalladium_cuda.so (sm_100a only).

The kernel translation unit is compiled three times, once per math mode, each
with the nvcc flag set that *is* that mode's definition (the reference selects
the mode when it compiles MSL: `mr.Kernel(msl, name, math_mode=...)`,
src/palladium/dispatch.py:290; here the three variants are built ahead of time):

  SAFE     -fmad=false -prec-div=true -prec-sqrt=true -ftz=false
  RELAXED  -fmad=true  -prec-div=true -prec-sqrt=true -ftz=false
  FAST     -use_fast_math

Run `python -m palladium_b200.build` (add `-v` for ptxas register / shared
memory statistics).  The library is written next to this file so that it
travels with the source tree.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
BUILD_DIR = PKG_DIR / "build"
LIBRARY = PKG_DIR / "libpalladium_cuda.so"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
MODE_FLAGS = {
    "safe": ["-DPD_MODE=0", "-fmad=false", "-prec-div=true", "-prec-sqrt=true", "-ftz=false"],
    "relaxed": ["-DPD_MODE=1", "-fmad=true", "-prec-div=true", "-prec-sqrt=true", "-ftz=false"],
    "fast": ["-DPD_MODE=2", "-use_fast_math"],
}


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found: libpalladium_cuda.so cannot be built")
    return found


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.h")) + [PKG_DIR.parent / "include" / "palladium_cuda.h"]


def is_stale() -> bool:
    if not LIBRARY.exists():
        return True
    built = LIBRARY.stat().st_mtime
    return any(src.stat().st_mtime > built for src in _sources())


def _run(cmd: list[str], verbose: bool) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    if verbose and (proc.stdout or proc.stderr):
        print(proc.stdout + proc.stderr, file=sys.stderr)


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile and link the library; a no-op when it is newer than its sources."""
    if not force and not is_stale():
        return LIBRARY
    nvcc = _nvcc()
    BUILD_DIR.mkdir(exist_ok=True)
    # pd_math.h as a string literal: the run-time compiled kernels include it from memory.
    # Split into pieces below the 64 KiB a single literal may hold.
    text = (CSRC / "pd_math.h").read_text()
    pieces = [text[i:i + 8000] for i in range(0, len(text), 8000)]
    (BUILD_DIR / "pd_math_embedded.inc").write_text("".join(f'R"PDMATH({piece})PDMATH"\n' for piece in pieces))
    extra = ["-Xptxas", "-v"] if verbose else []
    jobs: list[tuple[list[str], Path]] = []
    for mode, flags in MODE_FLAGS.items():
        obj = BUILD_DIR / f"pd_kernels_{mode}.o"
        jobs.append(([nvcc, *ARCH, *COMMON, *flags, *extra, "-c", str(CSRC / "pd_kernels.cu"), "-o", str(obj)], obj))
    api_obj = BUILD_DIR / "pd_api.o"
    jobs.append(([nvcc, *ARCH, *COMMON, "-c", str(CSRC / "pd_api.cu"), "-o", str(api_obj)], api_obj))
    noalloc_obj = BUILD_DIR / "pd_noalloc.o"
    jobs.append(([nvcc, *ARCH, *COMMON, "-c", str(CSRC / "pd_noalloc.cu"), "-o", str(noalloc_obj)], noalloc_obj))
    rtc_obj = BUILD_DIR / "pd_rtc.o"
    jobs.append(([nvcc, *ARCH, *COMMON, f"-I{BUILD_DIR}", "-c", str(CSRC / "pd_rtc.cu"), "-o", str(rtc_obj)], rtc_obj))
    with ThreadPoolExecutor(max_workers=len(jobs)) as pool:
        list(pool.map(lambda job: _run(job[0], verbose), jobs))
    link = [nvcc, *ARCH, "-shared", "-o", str(LIBRARY), *[str(obj) for _, obj in jobs], "-ldl"]
    _run(link, verbose)
    return LIBRARY


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force=True)
    print(path)
