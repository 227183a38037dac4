"""The C-ABI library: loads, exports every symbol the header declares, and
answers the calls that need no GPU (explain, tuning, argument validation)."""

import ctypes
import re
from pathlib import Path

import pytest

from palladium_b200 import _native

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    names = set()
    for header in (ROOT / "include").glob("*.h"):
        text = header.read_text()
        names |= set(re.findall(r"PD_API\s+[\w\s\*]+?\b(pd_\w+)\s*\(", text))
    return names


def test_header_and_binding_agree_on_the_symbol_list():
    assert declared_symbols() == set(_native.EXPORTED_SYMBOLS)


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(str(_native.library_path()))
    for name in declared_symbols():
        assert hasattr(lib, name), name
    assert lib.pd_version() == 1


def test_struct_layouts_match_the_header():
    text = (ROOT / "include" / "palladium_cuda.h").read_text()

    def fields(struct):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (struct, struct), text, re.S).group(1)
        out = []
        for decl in re.findall(r"(double|int64_t|int32_t|char)\s+([^;]+);", body):
            for name in decl[1].split(","):
                out.append(re.sub(r"\[.*\]", "", name).strip())
        return out

    pairs = [("pd_lv_rk4_params", _native.LvRk4Params), ("pd_vdp_bs32_params", _native.VdpBs32Params),
             ("pd_gbm_params", _native.GbmParams), ("pd_gray_scott_params", _native.GrayScottParams),
             ("pd_lv_rk4_df32_params", _native.LvRk4Df32Params), ("pd_kepler_rk4_df32_params", _native.KeplerRk4Df32Params),
             ("pd_threefry_params", _native.ThreefryParams), ("pd_launch_info", _native.LaunchInfo)]
    for cname, cls in pairs:
        assert fields(cname) == [f[0] for f in cls._fields_], cname


def test_explain_without_gpu_reports_geometry():
    info = _native.explain(0, _native.LvRk4Params(0.01, 1000), 2, (100_000,), None)
    assert info.kernel_name.decode() == "pd_lv_rk4_kernel<2>"     # two trajectories per thread from 512 per SM up
    assert info.cuda_grid[0] * info.cuda_block[0] * 2 >= 100_000
    small = _native.explain(0, _native.LvRk4Params(0.01, 1000), 2, (10_000,), None)
    assert small.kernel_name.decode() == "pd_lv_rk4_kernel<1>"
    assert info.launches == 1 and info.scratch_bytes == 0
    if _native.device_count() == 0:
        assert info.regs_per_thread == -1 and info.blocks_per_sm == -1


def test_invalid_math_mode_is_invalid_argument():
    from palladium_b200.errors import DispatchError

    with pytest.raises(DispatchError, match="math_mode out of range"):  # native/ffi/palladium_ffi.cpp:118-121
        _native.explain(0, _native.LvRk4Params(0.01, 10), 7, (16,), None)


def test_params_size_is_checked():
    lib = _native.library()
    err = ctypes.create_string_buffer(256)
    grid = (ctypes.c_int64 * 3)(16, 1, 1)
    info = _native.LaunchInfo()
    p = _native.LvRk4Params(0.01, 10)
    rc = lib.pd_explain(0, ctypes.addressof(p), 4, 2, grid, None, ctypes.byref(info), err, 256)
    assert rc == 1 and b"params block must be 16 bytes" in err.value
    rc = lib.pd_explain(99, ctypes.addressof(p), 16, 2, grid, None, ctypes.byref(info), err, 256)
    assert rc == 1 and b"unknown kernel family" in err.value


def test_tuning_knobs_round_trip():
    assert _native.get_tuning("vdp_variant") == 2
    _native.set_tuning("vdp_variant", 0)
    try:
        assert _native.get_tuning("vdp_variant") == 0
    finally:
        _native.set_tuning("vdp_variant", 2)
    with pytest.raises(KeyError):
        _native.set_tuning("no_such_knob", 1)


def test_thread_tuning_overrides_only_the_calling_thread():
    import threading

    seen = {}
    with _native.thread_tuning(gs_variant=1, vdp_variant=0):
        assert _native.get_tuning("gs_variant") == 1 and _native.get_tuning("vdp_variant") == 0
        worker = threading.Thread(target=lambda: seen.update(other=_native.get_tuning("gs_variant")))
        worker.start()
        worker.join()
    assert seen["other"] == -1                      # another thread kept the process-wide value
    assert _native.get_tuning("gs_variant") == -1   # and the override ended with the block
    with pytest.raises(KeyError):
        with _native.thread_tuning(no_such_knob=1):
            pass


def test_launch_without_device_fails_loudly():
    if _native.device_count() > 0:
        pytest.skip("a GPU is present")
    from palladium_b200.errors import DispatchError

    with pytest.raises(DispatchError, match="no CUDA device is available"):
        _native.dispatch_host(0, _native.LvRk4Params(0.01, 1), 2, (4,), None, [(0, 16)] * 6, [(0, 16)] * 2)


def test_missing_library_is_an_emit_error(monkeypatch, tmp_path):
    from palladium_b200.errors import EmitError

    monkeypatch.setenv("PALLADIUM_FFI_LIBRARY", str(tmp_path / "nope.so"))
    monkeypatch.setattr(_native, "_lib", None)
    with pytest.raises(EmitError, match="isn't built"):
        _native.library()


def test_pointer_carrying_structs_match_the_compilers_layout(tmp_path):
    """The parameter blocks with pointers in them are checked against the C
    compiler itself: size and the offset of every field."""
    import subprocess

    structs = {
        "pd_custom_ode_params": _native.CustomOdeParams,
        "pd_source_kernel_params": _native.SourceKernelParams,
        "pd_gs_neighbours": _native.GsNeighbours,
    }
    lines = ['#include <stddef.h>', '#include <stdio.h>', f'#include "{ROOT / "include" / "palladium_cuda.h"}"',
             "int main(void) {"]
    for cname, cls in structs.items():
        lines.append(f'  printf("{cname} size %zu\\n", sizeof({cname}));')
        for field, _ in cls._fields_:
            lines.append(f'  printf("{cname} {field} %zu\\n", offsetof({cname}, {field}));')
    lines += ["  return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c11", str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    seen = {}
    for line in out.splitlines():
        cname, field, value = line.split()
        seen[(cname, field)] = int(value)
    for cname, cls in structs.items():
        assert seen[(cname, "size")] == ctypes.sizeof(cls), cname
        for field, _ in cls._fields_:
            assert seen[(cname, field)] == getattr(cls, field).offset, (cname, field)


def test_wait_on_an_unknown_ticket_is_invalid_argument():
    from palladium_b200.errors import DispatchError

    with pytest.raises(DispatchError, match="unknown or already retired ticket"):
        _native.wait_host(123456789, [])
