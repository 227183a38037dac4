"""Builds the CPU oracle (TEST INFRASTRUCTURE ONLY; never imported by the package).

  oracle/liboracle.so        the C restatement in oracle/oracle.c
  oracle/_ref/libmslref.so   the reference's own emitted RK4 kernel
                             (tests/golden/rk4_lotka_volterra.metal, compiled as
                             C++ where it lies in the reference checkout), built
                             only when that checkout is present
  oracle/_ref/libgbmref.so   the reference's hand-written Monte Carlo kernel (the
                             GBM_MSL string of examples/03_sde_montecarlo.py:34-70,
                             taken out of the example where it lies), compiled as
                             C++ through the same shim
  oracle/_ref/libdf32ref.so  the reference's hand-written df32 kernel (DF32_KERNEL of
                             examples/05_df32_precision.py:27-80) on this oracle's
                             restatement of the external df32 prelude
  oracle/_ref/libthreefryref.so   the Threefry-2x32-20 block as the reference's
                             emitter writes it: the text-emitting helper
                             `_emit_threefry2x32` (src/palladium/emit/rules.py:
                             121-165) is run where it lies and the statements it
                             emits are compiled as C; built only when the
                             checkout is present

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
REF_THREEFRY_LIB = REF_DIR / "libthreefryref.so"
REF_GBM_LIB = REF_DIR / "libgbmref.so"
REF_DF32_LIB = REF_DIR / "libdf32ref.so"
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


def _module_string(example: Path, name: str) -> str:
    """The string constant `name` of a reference example, without importing it."""
    import ast

    for node in ast.parse(example.read_text()).body:
        if isinstance(node, ast.Assign) and any(isinstance(t, ast.Name) and t.id == name for t in node.targets):
            return ast.literal_eval(node.value)
    raise RuntimeError(f"{name} was not found in {example.name}")


def _build_msl_string(example: Path, name: str, msl_name: str, wrapper: str, define: str, lib: Path,
                      force: bool) -> Path | None:
    if not example.exists():
        return lib if lib.exists() else None
    text = _module_string(example, name)
    REF_DIR.mkdir(exist_ok=True)
    msl = REF_DIR / msl_name   # generated from the reference; this directory is not committed
    src = HERE / wrapper
    if force or not msl.exists() or msl.read_text() != text or _stale(
            lib, [src, HERE / "msl_shim" / "metal_stdlib", HERE / "df32_ops.h"]):
        msl.write_text(text)
        _run(["g++", "-std=c++17", *CFLAGS, "-Wno-attributes", f"-I{HERE / 'msl_shim'}", f"-I{HERE}",
              f'-D{define}="{msl}"', str(src), "-o", str(lib)])
    return lib


def build_reference_gbm(force: bool = False) -> Path | None:
    """Compile the reference's hand-written `gbm_paths` MSL kernel for the CPU."""
    return _build_msl_string(REFERENCE_ROOT / "examples" / "03_sde_montecarlo.py", "GBM_MSL", "gbm_paths.metal",
                             "msl_gbm_ref.cpp", "PD_GBM_MSL", REF_GBM_LIB, force)


def build_reference_df32(force: bool = False) -> Path | None:
    """Compile the reference's hand-written `lv_rk4_df32` MSL kernel for the CPU
    (on this oracle's restatement of the df32 prelude it expects)."""
    return _build_msl_string(REFERENCE_ROOT / "examples" / "05_df32_precision.py", "DF32_KERNEL",
                             "lv_rk4_df32.metal", "msl_df32_ref.cpp", "PD_DF32_MSL", REF_DF32_LIB, force)


class _TextCursor:
    """The two methods of the emitter's Cursor that `_emit_threefry2x32` uses
    (it is documented as pure text emission: src/palladium/emit/rules.py:129-133)."""

    def __init__(self) -> None:
        self.lines: list[str] = []
        self._count = 0

    def fresh(self, prefix: str = "_t") -> str:
        self._count += 1
        return f"{prefix}{self._count}"

    def emit(self, line: str) -> None:
        self.lines.append(line)


def reference_threefry_statements() -> tuple[list[str], str, str] | None:
    """Runs the reference's `_emit_threefry2x32` on operands named k1, k2, c0, c1
    and returns (emitted statements, name of output word 0, name of output word 1).
    The function and its two rotation tables are taken out of rules.py by name:
    the module itself imports JAX, which is not installed."""
    import ast

    rules = REFERENCE_ROOT / "src" / "palladium" / "emit" / "rules.py"
    if not rules.exists():
        return None
    tree = ast.parse(rules.read_text())
    wanted = []
    for node in tree.body:
        if isinstance(node, ast.Assign) and any(
                isinstance(t, ast.Name) and t.id in ("_THREEFRY_ROT0", "_THREEFRY_ROT1") for t in node.targets):
            wanted.append(node)
        if isinstance(node, ast.FunctionDef) and node.name == "_emit_threefry2x32":
            wanted.append(node)
    if len(wanted) != 3:
        raise RuntimeError("the reference's Threefry emitter was not found where expected in rules.py")
    namespace: dict = {"Cursor": _TextCursor}
    exec(compile(ast.Module(body=wanted, type_ignores=[]), str(rules), "exec"), namespace)
    cursor = _TextCursor()
    out0, out1 = namespace["_emit_threefry2x32"](cursor, "k1", "k2", "c0", "c1")
    return cursor.lines, out0, out1


def build_reference_threefry(force: bool = False) -> Path | None:
    """Compile the Threefry block the reference's emitter writes, plus the two
    compositions its rules make of it: random_bits = block(key, (0, flat index))
    with the output words xor-ed (rules.py:168-185) and fold_in = block(key,
    (0, data)) with both words as the new key (rules.py:188-201)."""
    emitted = reference_threefry_statements()
    if emitted is None:
        return REF_THREEFRY_LIB if REF_THREEFRY_LIB.exists() else None
    lines, out0, out1 = emitted
    REF_DIR.mkdir(exist_ok=True)
    src = REF_DIR / "threefry_ref.c"
    body = "\n".join("    " + line for line in lines)
    text = f"""/* generated by oracle/build.py from the reference's emitter; not source of this repository */
typedef unsigned int uint;
#define EXPORT __attribute__((visibility("default")))
static void block(uint k1, uint k2, uint c0, uint c1, uint* o0, uint* o1) {{
{body}
    *o0 = {out0};
    *o1 = {out1};
}}
EXPORT void ref_threefry2x32(const uint* key, const uint* ctr, uint* out) {{
    block(key[0], key[1], ctr[0], ctr[1], &out[0], &out[1]);
}}
EXPORT void ref_random_bits(const uint* key, long long n, uint* out) {{
    for (long long i = 0; i < n; ++i) {{ uint a, b; block(key[0], key[1], 0u, (uint)i, &a, &b); out[i] = a ^ b; }}
}}
EXPORT void ref_fold_in(const uint* key, const uint* data, long long n, uint* out) {{
    for (long long i = 0; i < n; ++i) block(key[0], key[1], 0u, data[i], &out[2 * i], &out[2 * i + 1]);
}}
"""
    if force or not src.exists() or src.read_text() != text or not REF_THREEFRY_LIB.exists():
        src.write_text(text)
        _run(["gcc", "-std=c11", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", str(src), "-o",
              str(REF_THREEFRY_LIB)])
    return REF_THREEFRY_LIB


if __name__ == "__main__":
    print(build_oracle(force="-f" in sys.argv))
    print(build_reference(force="-f" in sys.argv))
    print(build_reference_threefry(force="-f" in sys.argv))
    print(build_reference_gbm(force="-f" in sys.argv))
    print(build_reference_df32(force="-f" in sys.argv))
