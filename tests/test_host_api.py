"""Host-side contract of cuda_call / cuda_call_jit without a GPU: signature
validation, the error taxonomy, explain(), the per-shape cache and its locking,
environment hooks.  Modelled on the reference's tests/test_16_diagnostics.py and
tests/test_17_robustness.py."""

import threading

import numpy as np
import pytest

import palladium_b200 as pd
from palladium_b200 import DispatchError, EmitError, PalladiumError, TraceError, UnsupportedPrimitiveError
from palladium_b200 import families, pl
from tests import helpers as H

F32 = np.float32


# ------------------------------------------------------------------ error taxonomy
def test_error_hierarchy_matches_reference():
    # src/palladium/errors.py:19-44
    assert issubclass(TraceError, PalladiumError) and issubclass(TraceError, ValueError)
    assert issubclass(EmitError, PalladiumError)
    assert issubclass(UnsupportedPrimitiveError, EmitError) and issubclass(UnsupportedPrimitiveError, NotImplementedError)
    assert issubclass(DispatchError, PalladiumError) and issubclass(DispatchError, TypeError)


def test_math_mode_values_and_ordinals():
    from palladium_b200.math_mode import math_mode_ordinal

    assert [m.value for m in pd.MathMode] == ["safe", "relaxed", "fast"]
    assert [math_mode_ordinal(m) for m in pd.MathMode] == [0, 1, 2]  # src/palladium/ffi.py:38
    assert math_mode_ordinal("relaxed") == 1 and math_mode_ordinal(2) == 2
    with pytest.raises(ValueError):
        math_mode_ordinal("fastest")


# ------------------------------------------------------------------ explain()
def test_explain_reports_geometry():
    diag = H.lv_solver(1000).explain(*[H.shaped(1000)] * 6)
    assert diag.grid == (1000,)
    assert diag.threadgroup is None
    assert diag.msl_lines > 0
    assert f"palladium kernel {diag.name}" in str(diag)
    assert diag.cuda_kernel.startswith("pd_lv_rk4_kernel")
    assert diag.cuda_grid[0] * diag.cuda_block[0] * diag.items_per_thread >= 1000


def test_explain_explicit_threadgroup():
    call = H.lv_solver(64, threadgroup=64)
    diag = call.explain(*[H.shaped(64)] * 6)
    assert diag.threadgroup == (64,)
    assert "threadgroup=(64,)" in str(diag)
    assert diag.cuda_block[0] == 64


def test_explain_accepts_arrays_and_reads_no_data():
    n = 100
    args = [np.zeros(n, F32)] * 6
    assert H.lv_solver(n).explain(*args).grid == (n,)


def test_explain_large_ensemble_uses_vector_items():
    n = 1 << 22
    diag = H.lv_solver(n).explain(*[H.shaped(n)] * 6)
    assert diag.items_per_thread == 4 and diag.cuda_kernel == "pd_lv_rk4_kernel<4>"


def test_explain_other_families():
    d = H.vdp_solver(5000, outputs=6).explain(*[H.shaped(5000)] * 3)
    assert d.cuda_kernel == "pd_vdp_compact_kernel" and d.scratch_bytes > 0
    d = H.gs_solver(256, 256, steps=10).explain(H.shaped(256, 256), H.shaped(256, 256))
    assert d.cuda_kernel == "pd_gs_tb_kernel<4>" and d.launches == 3 and d.scratch_bytes == 2 * 256 * 256 * 4
    d = H.gs_solver(256, 256, steps=1).explain(H.shaped(256, 256), H.shaped(256, 256))
    assert d.cuda_kernel == "pd_gs_vec4_kernel" and d.launches == 1 and d.scratch_bytes == 0
    d = H.gs_solver(30, 50).explain(H.shaped(30, 50), H.shaped(30, 50))
    assert d.cuda_kernel == "pd_gs_cell_kernel"
    d = H.gbm_solver(1 << 16, with_sums=True).explain(H.shaped(2, dtype=np.uint32))
    assert d.cuda_kernel == "pd_gbm_kernel<threefry>" and d.launches == 2
    d = H.gbm_pcg_solver(1 << 16).explain()
    assert d.cuda_kernel == "pd_gbm_kernel<pcg>"


def test_explain_logging_once_per_shape(monkeypatch, capsys):
    # tests/test_16_diagnostics.py:72-80 in the reference: one line per compile, cached shapes stay silent
    monkeypatch.setenv("PALLADIUM_EXPLAIN", "1")
    call = H.lv_solver(128)
    arrays = [np.ones(128, F32)] * 6
    call._bound(arrays)
    call._bound(arrays)
    err = capsys.readouterr().err
    assert err.count("palladium kernel palladium_lv_rk4") == 1


def test_dump_hook_writes_a_launch_record(monkeypatch, tmp_path):
    monkeypatch.setenv("PALLADIUM_DUMP_MSL", str(tmp_path))
    H.lv_solver(32)._bound([np.ones(32, F32)] * 6)
    files = list(tmp_path.iterdir())
    assert len(files) == 1 and "palladium_lv_rk4" in files[0].read_text()


# ------------------------------------------------------------------ call-boundary validation
def test_float64_rejected_with_hint():
    call = H.lv_solver(16)
    with pytest.raises(DispatchError, match="jax_enable_x64"):
        call(*[np.zeros(16, np.float64)] * 6)


def test_wrong_count_shape_dtype():
    call = H.lv_solver(16)
    with pytest.raises((DispatchError, TraceError), match="takes 6 arrays, got 5"):
        call(*[np.zeros(16, F32)] * 5)
    with pytest.raises(TraceError, match="shape"):
        call(*[np.zeros(17, F32)] * 6)
    with pytest.raises(DispatchError, match="does not match the traced float32; cast explicitly"):
        call(*[np.zeros(16, np.int32)] * 6)


def test_bound_kernel_checks_like_reference():
    # src/palladium/dispatch.py:150-176
    call = H.lv_solver(16)
    bound = call._bound([np.zeros(16, F32)] * 6)
    with pytest.raises(DispatchError, match="kernel takes 6 arrays, got 2"):
        bound.launch(np.zeros(16, F32), np.zeros(16, F32))
    with pytest.raises(DispatchError, match=r"argument 0: expected shape \(16,\), got \(8,\)"):
        bound.launch(np.zeros(8, F32), *[np.zeros(16, F32)] * 5)
    with pytest.raises(DispatchError, match="argument 3: dtype float64 does not match the traced float32"):
        bound.launch(*[np.zeros(16, F32)] * 3, np.zeros(16, np.float64), *[np.zeros(16, F32)] * 2)


def test_no_gpu_is_a_loud_error(has_gpu):
    if has_gpu:
        pytest.skip("a GPU is present")
    with pytest.raises(DispatchError, match="no CUDA device"):
        H.lv_solver(16)(*[np.zeros(16, F32)] * 6)
    with pytest.raises(DispatchError, match="no CUDA device"):
        H.lv_solver(16, call=pd.cuda_call_jit)(*[np.zeros(16, F32)] * 6)


def test_trace_rejects_malformed_requests():
    fam = families.lv_rk4()
    spec = H.SPEC_1
    with pytest.raises(TraceError, match="grid must be"):
        pd.cuda_call(fam, grid=(4, 4), out_shape=(H.shaped(4), H.shaped(4)))
    with pytest.raises(TraceError, match="out_shape"):
        pd.cuda_call(fam, grid=(4,), out_shape=(H.shaped(5), H.shaped(4)))
    with pytest.raises(TraceError, match=r"out_shape\[0\] is \(4,\)"):
        pd.cuda_call(fam, grid=(4,), out_shape=H.shaped(4))
    with pytest.raises(TraceError, match="in_specs has 5 entries"):
        pd.cuda_call(fam, grid=(4,), in_specs=[spec] * 5, out_shape=(H.shaped(4), H.shaped(4)))
    with pytest.raises(TraceError, match="block shape"):
        pd.cuda_call(fam, grid=(4,), in_specs=[pl.BlockSpec((2,), lambda i: (i,))] * 6, out_shape=(H.shaped(4),) * 2)
    with pytest.raises(TraceError, match="index_map"):
        pd.cuda_call(fam, grid=(4,), in_specs=[pl.BlockSpec((1,), lambda i: (0,))] * 6, out_shape=(H.shaped(4),) * 2)
    with pytest.raises(TraceError, match="out_shape is required"):
        pd.cuda_call(fam, grid=(4,))
    with pytest.raises(TraceError, match="unsupported pallas_call keywords"):
        pd.cuda_call(fam, grid=(4,), out_shape=(H.shaped(4),) * 2, scratch_shapes=[])
    with pytest.raises(TraceError, match="grid_spec"):
        pd.cuda_call(fam, grid=(4,), out_shape=(H.shaped(4),) * 2, grid_spec=object())


def test_arbitrary_pallas_function_is_unsupported():
    def kernel(x_ref, o_ref):
        o_ref[...] = x_ref[...] * 2.0

    with pytest.raises(UnsupportedPrimitiveError, match="kernel family"):
        pd.cuda_call(kernel, out_shape=H.shaped(8))
    with pytest.raises(NotImplementedError):
        pd.cuda_call_jit(kernel, out_shape=H.shaped(8))
    with pytest.raises(UnsupportedPrimitiveError):
        families.lv_rk4()(1, 2)


def test_gray_scott_and_vdp_signatures():
    with pytest.raises(TraceError, match="6, 5 or 3 outputs"):
        pd.cuda_call(families.vdp_bs32(), grid=(8,), out_shape=(H.shaped(8),) * 4)
    with pytest.raises(TraceError, match="grid must be \\(rows, cols\\)"):
        pd.cuda_call(families.gray_scott(), grid=(8,), out_shape=(H.shaped(8, 8),) * 2)
    call = H.gs_solver(16, 32, steps=3, halo=4)
    assert call.explain(H.shaped(24, 32), H.shaped(24, 32)).grid == (16, 32)
    with pytest.raises((DispatchError, PalladiumError), match="at most 2 steps"):
        H.gs_solver(16, 32, steps=3, halo=2).explain(H.shaped(20, 32), H.shaped(20, 32))
    with pytest.raises(TraceError):
        families.gbm_threefry(output="both")


def test_vmap_method_validation():
    # src/palladium/ffi.py:118-125
    for ok in (None, "sequential", "sequential_unrolled"):
        H.lv_solver(8, call=pd.cuda_call_jit, vmap_method=ok)
    with pytest.raises(ValueError, match="vmap_method 'expand_dims' is not supported"):
        H.lv_solver(8, call=pd.cuda_call_jit, vmap_method="expand_dims")
    with pytest.raises(ValueError):
        H.lv_solver(8, call=pd.cuda_call_jit, vmap_method="broadcast_all")


def test_threadgroup_is_validated_by_the_native_library():
    call = H.lv_solver(64, threadgroup=48)
    with pytest.raises(DispatchError, match="multiple of 32"):
        call.explain(*[H.shaped(64)] * 6)


# ------------------------------------------------------------------ cache and threads
def test_cache_is_per_shape_signature():
    call = H.lv_solver(32)
    arrays = [np.zeros(32, F32)] * 6
    b1 = call._bound(arrays)
    b2 = call._bound([a.copy() for a in arrays])
    assert b1 is b2 and len(call.cache) == 1
    key = next(iter(call.cache))
    assert key == tuple(((32,), "<f4") for _ in range(6))
    assert call.cache[key].msl_source.endswith("pd_kernels.cu")


def test_concurrent_first_calls_bind_once(monkeypatch):
    # tests/test_17_robustness.py:22-50: 16 threads, exactly one compile per shape
    from palladium_b200 import call as package

    binds = []
    real_bind = package.bind

    def counting_bind(*a, **k):
        binds.append(1)
        return real_bind(*a, **k)

    monkeypatch.setattr(package, "bind", counting_bind)
    call = H.lv_solver(64)
    arrays = [np.zeros(64, F32)] * 6
    barrier = threading.Barrier(16)
    results = []

    def worker():
        barrier.wait()
        results.append(call._bound(arrays))

    threads = [threading.Thread(target=worker) for _ in range(16)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    assert len(binds) == 1
    assert all(r is results[0] for r in results)


def test_interpret_resolution(interpret_provider):
    import oracle
    from palladium_b200 import workloads as W

    call = H.lv_solver(33, steps=50)
    args = W.lotka_volterra_ensemble(33)
    got = call.interpret(*args)
    want = oracle.lv_rk4(*args, dt=0.01, steps=50)
    np.testing.assert_array_equal(got[0], want[0])
    # the jit-flavoured callable carries the same oracle attribute
    got2 = H.lv_solver(33, steps=50, call=pd.cuda_call_jit).interpret(*args)
    np.testing.assert_array_equal(got2[1], want[1])


def test_interpret_without_provider_explains_itself():
    previous = pd.register_interpret_provider(None)
    try:
        with pytest.raises(PalladiumError, match="register_interpret_provider"):
            H.lv_solver(4).interpret(*[np.zeros(4, F32)] * 6)
    finally:
        pd.register_interpret_provider(previous)


def test_debug_msl_returns_a_launch_record():
    text = pd.debug_msl(families.lv_rk4(), *[H.shaped(256)] * 6, grid=(256,), out_shape=(H.shaped(256),) * 2)
    assert "palladium kernel palladium_lv_rk4" in text and "pd_kernels.cu" in text


def test_public_names():
    for name in ("cuda_call", "cuda_call_jit", "CudaCallable", "FfiCallable", "BoundKernel", "PendingResult",
                 "KernelDiagnostics", "KernelSpec", "BlockInfo", "MathMode", "bind", "trace", "debug_msl",
                 "PalladiumError", "TraceError", "EmitError", "UnsupportedPrimitiveError", "DispatchError"):
        assert hasattr(pd, name), name


def test_device_tensors_are_checked_before_any_launch():
    """Outputs handed to the device path are validated like inputs: a host tensor, a
    strided view, a short tensor or one on another GPU is refused before the native
    call, which would write the traced byte count from the pointer regardless."""
    import torch

    from palladium_b200.dispatch import check_device_tensors

    class OnGpu:   # what the check reads of a tensor, for shapes a CPU-only box cannot allocate on a device
        is_cuda = True

        def __init__(self, numel, contiguous=True, index=0):
            self._numel, self._contiguous = numel, contiguous
            self.device = torch.device("cuda", index)

        def is_contiguous(self):
            return self._contiguous

        def numel(self):
            return self._numel

        def element_size(self):
            return 4

    check_device_tensors("output", [OnGpu(100)], [400], 0)
    with pytest.raises(pd.DispatchError, match="output 0: expected a CUDA tensor"):
        check_device_tensors("output", [torch.empty(100)], [400], 0)
    with pytest.raises(pd.DispatchError, match="output 1: expected 400 bytes, got 396"):
        check_device_tensors("output", [OnGpu(100), OnGpu(99)], [400, 400], 0)
    with pytest.raises(pd.DispatchError, match="output 0: expected a contiguous tensor"):
        check_device_tensors("output", [OnGpu(100, contiguous=False)], [400], 0)
    with pytest.raises(pd.DispatchError, match="is on cuda:1 but the launch runs on cuda:0"):
        check_device_tensors("output", [OnGpu(100, index=1)], [400], 0)
