"""The call objects on a real device: launch/wait, pin, concurrent use, the
host-buffer C-ABI path and the device-tensor path.  Modelled on the reference's
tests/test_dispatch_launch.py, tests/test_17_robustness.py and the parts of
tests/test_11_ffi.py that do not need JAX."""

import threading

import numpy as np
import pytest

import oracle
import palladium_b200 as pd
from palladium_b200 import workloads as W
from tests import helpers as H

pytestmark = pytest.mark.gpu
SAFE = pd.MathMode.SAFE


def test_launch_then_wait_equals_call():
    # tests/test_dispatch_launch.py:42-51
    n = 1000
    args = W.lotka_volterra_ensemble(n)
    call = H.lv_solver(n, steps=100, math_mode=SAFE)
    direct = call(*args)
    pending = call.launch(*args)
    assert isinstance(pending, pd.PendingResult)
    waited = pending.wait()
    np.testing.assert_array_equal(direct[0], waited[0])
    np.testing.assert_array_equal(direct[1], waited[1])


def test_second_launch_before_wait_does_not_corrupt_the_first():
    # tests/test_dispatch_launch.py:74-87
    n = 4096
    a = W.lotka_volterra_ensemble(n, seed=1)
    b = W.lotka_volterra_ensemble(n, seed=2)
    call = H.lv_solver(n, steps=200, math_mode=SAFE)
    first = call.launch(*a)
    second = call.launch(*b)
    got_b = second.wait()
    got_a = first.wait()
    np.testing.assert_array_equal(got_a[0], oracle.lv_rk4(*a, dt=0.01, steps=200)[0])
    np.testing.assert_array_equal(got_b[0], oracle.lv_rk4(*b, dt=0.01, steps=200)[0])


@pytest.mark.parametrize("n", [1000, 100_000])      # results collected at the wait / downloaded into page-locked arrays
def test_launch_copies_its_inputs_and_many_calls_stay_in_flight(n):
    """`launch` has read its arrays when it returns (the caller may overwrite them at once), thirty-two
    calls in flight keep their results apart, and a second `wait` hands back the same arrays."""
    call = H.lv_solver(n, steps=20, math_mode=SAFE)
    ensembles = [W.lotka_volterra_ensemble(n, seed=s) for s in range(4)]
    scratch = [a.copy() for a in ensembles[0]]
    pending = []
    for i in range(32):
        for dst, src in zip(scratch, ensembles[i % 4]):
            dst[...] = src
        pending.append(call.launch(*scratch))
        for dst in scratch:
            dst[...] = np.nan            # overwritten while the call is still in flight
    want = [oracle.lv_rk4(*e, dt=0.01, steps=20) for e in ensembles]
    results = [h.wait() for h in reversed(pending)][::-1]
    for i, got in enumerate(results):
        np.testing.assert_array_equal(got[0], want[i % 4][0])
        np.testing.assert_array_equal(got[1], want[i % 4][1])
    assert pending[0].wait()[0] is results[0][0]
    assert results[0][0].ctypes.data != results[4][0].ctypes.data     # equal values, separate arrays


def test_too_many_launches_in_flight_is_an_error_and_dropped_results_free_their_slots():
    import gc

    n = 256
    args = W.lotka_volterra_ensemble(n)
    call = H.lv_solver(n, steps=2, math_mode=SAFE)
    pending = [call.launch(*args) for _ in range(64)]
    with pytest.raises(pd.DispatchError, match="in flight"):
        call.launch(*args)
    del pending[32:]                     # never waited for: the slots come back when the handles go
    gc.collect()
    more = [call.launch(*args) for _ in range(32)]
    want = oracle.lv_rk4(*args, dt=0.01, steps=2)
    for h in pending + more:
        np.testing.assert_array_equal(h.wait()[0], want[0])


def test_native_submit_and_wait_argument_errors_keep_the_ticket():
    from palladium_b200 import _native

    n = 512
    args = W.lotka_volterra_ensemble(n)
    params = _native.LvRk4Params(0.01, 10)
    ticket = _native.submit_host(0, params, 0, (n,), None, [(a.ctypes.data, a.nbytes) for a in args], [4 * n, 4 * n])
    x, y = np.empty(n, np.float32), np.empty(n, np.float32)
    with pytest.raises(pd.DispatchError, match="produced 2 arrays, 1 were offered"):
        _native.wait_host(ticket, [(x.ctypes.data, x.nbytes)])
    with pytest.raises(pd.DispatchError, match="bytes offered"):
        _native.wait_host(ticket, [(x.ctypes.data, x.nbytes), (y.ctypes.data, 8)])
    _native.wait_host(ticket, [(x.ctypes.data, x.nbytes), (y.ctypes.data, y.nbytes)])
    want = oracle.lv_rk4(*args, dt=0.01, steps=10)
    np.testing.assert_array_equal(x, want[0])
    np.testing.assert_array_equal(y, want[1])
    with pytest.raises(pd.DispatchError, match="unknown or already retired"):
        _native.wait_host(ticket, [])


def test_stepping_loop_feeds_outputs_back():
    # tests/test_dispatch_launch.py:54-72: outputs of one dispatch are the next one's inputs
    size = 64
    u, v = W.gray_scott_initial_state(size, patches=2, patch=8)
    call = H.gs_solver(size, size, math_mode=SAFE)
    cu, cv = u, v
    for _ in range(5):
        cu, cv = call.launch(cu, cv).wait()
    want = oracle.gray_scott(u, v, steps=5)
    np.testing.assert_array_equal(cu, want[0])
    np.testing.assert_array_equal(cv, want[1])


def test_pin_redispatches_on_resident_inputs():
    n = 2000
    args = [a.copy() for a in W.lotka_volterra_ensemble(n)]
    call = H.lv_solver(n, steps=50, math_mode=SAFE)
    pinned = call.pin(*args)
    want = oracle.lv_rk4(*args, dt=0.01, steps=50)
    args[0][:] = 0.0  # later mutation of the passed arrays is not observed
    for _ in range(3):
        got = pinned()
        np.testing.assert_array_equal(got[0], want[0])
        np.testing.assert_array_equal(got[1], want[1])


def test_single_output_is_a_bare_array_and_outputs_are_fresh():
    key = W.gbm_key(1)
    call = H.gbm_solver(512, math_mode=SAFE, steps=16)
    first = call(key)
    second = call(key)
    assert isinstance(first, np.ndarray) and first.shape == (512,)
    assert first is not second and not np.shares_memory(first, second)
    np.testing.assert_array_equal(first, second)


def test_many_threads_share_one_bound_kernel():
    # tests/test_17_robustness.py:52-78
    n = 3000
    call = H.lv_solver(n, steps=40, math_mode=SAFE)
    inputs = [W.lotka_volterra_ensemble(n, seed=s) for s in range(8)]
    wants = [oracle.lv_rk4(*a, dt=0.01, steps=40) for a in inputs]
    results = [None] * 8
    errors = []

    def worker(i):
        try:
            results[i] = call(*inputs[i])
        except Exception as exc:  # surfaced below
            errors.append(exc)

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(8)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    assert not errors
    assert len(call.cache) == 1
    for got, want in zip(results, wants):
        np.testing.assert_array_equal(got[0], want[0])
        np.testing.assert_array_equal(got[1], want[1])


def test_host_buffer_path_matches_eager_and_oracle():
    """cuda_call_jit on NumPy arrays goes through pd_dispatch_host, the call an
    XLA:CPU FFI handler would make (tests/test_11_ffi.py:35-60: eager == interpret)."""
    n = 5001
    args = W.lotka_volterra_ensemble(n)
    jit = H.lv_solver(n, steps=120, call=pd.cuda_call_jit, math_mode=SAFE)
    got = jit(*args)
    want = oracle.lv_rk4(*args, dt=0.01, steps=120)
    np.testing.assert_array_equal(got[0], want[0])
    np.testing.assert_array_equal(got[1], want[1])


def test_host_buffer_path_from_many_threads():
    n = 1024
    jit = H.lv_solver(n, steps=30, call=pd.cuda_call_jit, math_mode=SAFE)
    inputs = [W.lotka_volterra_ensemble(n, seed=s) for s in range(6)]
    results = [None] * 6

    def worker(i):
        results[i] = jit(*inputs[i])

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(6)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    for a, got in zip(inputs, results):
        np.testing.assert_array_equal(got[0], oracle.lv_rk4(*a, dt=0.01, steps=30)[0])


def test_device_tensor_path_is_stream_ordered_and_composes_with_torch_ops():
    import torch

    n = 4096
    args = W.lotka_volterra_ensemble(n)
    jit = H.lv_solver(n, steps=60, call=pd.cuda_call_jit, math_mode=SAFE)
    dev = [torch.from_numpy(a).cuda() for a in args]
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        scaled = dev[0] * 1.0                       # a torch op before ...
        x, y = jit(scaled, *dev[1:])
        total = (x * x + y * y).sum()               # ... and after, on the same stream, no sync in between
    stream.synchronize()
    want = oracle.lv_rk4(*args, dt=0.01, steps=60)
    np.testing.assert_array_equal(x.cpu().numpy(), want[0])
    np.testing.assert_allclose(float(total), float((want[0].astype(np.float64) ** 2 + want[1].astype(np.float64) ** 2).sum()), rtol=1e-5)


def test_multi_output_and_math_mode_reach_the_kernel():
    """Different math modes must select different compiled kernels
    (tests/test_11_ffi.py:123-145 checks the same by a NaN probe): SAFE equals
    the oracle bit for bit, FAST does not."""
    n = 20_000
    args = W.lotka_volterra_ensemble(n)
    safe = H.lv_solver(n, steps=500, call=pd.cuda_call_jit, math_mode=SAFE)(*args)
    fast = H.lv_solver(n, steps=500, call=pd.cuda_call_jit, math_mode=pd.MathMode.FAST)(*args)
    want = oracle.lv_rk4(*args, dt=0.01, steps=500)
    assert np.array_equal(safe[0], want[0])
    assert not np.array_equal(fast[0], want[0])
    np.testing.assert_allclose(fast[0], want[0], rtol=1e-4)


def test_unaligned_host_and_device_buffers_take_the_scalar_path():
    import torch

    n = 1003
    args = W.lotka_volterra_ensemble(n)
    backing = [torch.empty(n + 1, dtype=torch.float32, device="cuda") for _ in range(6)]
    views = [b[1:] for b in backing]  # 4-byte aligned only
    for v, a in zip(views, args):
        v.copy_(torch.from_numpy(a))
    jit = H.lv_solver(n, steps=25, call=pd.cuda_call_jit, math_mode=SAFE)
    x, y = jit(*[v.contiguous() if False else v for v in views])
    want = oracle.lv_rk4(*args, dt=0.01, steps=25)
    np.testing.assert_array_equal(x.cpu().numpy(), want[0])


def test_explain_on_device_reports_registers_and_occupancy():
    diag = H.lv_solver(1 << 20).explain(*[H.shaped(1 << 20)] * 6)
    assert diag.regs > 0 and diag.blocks_per_sm > 0 and diag.smem_bytes >= 0


def test_empty_ensemble():
    call = H.lv_solver(0, steps=10, math_mode=SAFE)
    x, y = call(*[np.zeros(0, np.float32)] * 6)
    assert x.shape == (0,) and y.shape == (0,)


def test_peak_measurements_are_plausible():
    from palladium_b200 import _native

    fma = _native.measure_fp32_fma_peak()
    alu = _native.measure_int32_alu_peak()
    assert 30e12 < fma < 90e12
    assert 5e12 < alu < 60e12


# ------------------------------------------------------------------ chunked host pipeline
def test_large_host_call_is_chunked_and_still_exact():
    """Above 2^18 trajectories pd_dispatch_host pipelines upload / compute /
    download in chunks; results must not depend on the chunking."""
    n = (1 << 18) + 12_345
    args = W.lotka_volterra_ensemble(n)
    got = H.lv_solver(n, steps=20, call=pd.cuda_call_jit, math_mode=SAFE)(*args)
    want = oracle.lv_rk4(*args, dt=0.01, steps=20)
    np.testing.assert_array_equal(got[0], want[0])
    np.testing.assert_array_equal(got[1], want[1])


@pytest.mark.parametrize("threads", [4, 1, 0])
def test_pageable_inputs_of_a_large_call_go_through_the_copy_threads(threads):
    """From 16 MB of input on, ordinary NumPy arrays are staged into page-locked buffers by the
    library's copy threads, chunk by chunk; page-locked arrays are uploaded where they are.  Both
    must give the oracle's result, with any number of threads (0: the driver's own pageable copy),
    as must an eager call of that size, which fills its slot the same way."""
    import torch

    from palladium_b200 import _native

    n = (1 << 20) + 4097              # 25 MB of input in 8 chunks, an odd tail
    args = W.lotka_volterra_ensemble(n)
    want = oracle.lv_rk4(*args, dt=0.01, steps=8)
    locked = [torch.from_numpy(a).pin_memory().numpy() for a in args]
    _native.set_tuning("host_copy_threads", threads)
    try:
        for arrays in (args, locked, args):
            got = H.lv_solver(n, steps=8, call=pd.cuda_call_jit, math_mode=SAFE)(*arrays)
            np.testing.assert_array_equal(got[0], want[0])
            np.testing.assert_array_equal(got[1], want[1])
        got = H.lv_solver(n, steps=8, math_mode=SAFE)(*args)       # eager: pd_submit_host
        np.testing.assert_array_equal(got[0], want[0])
        np.testing.assert_array_equal(got[1], want[1])
    finally:
        _native.set_tuning("host_copy_threads", 4)


def test_chunked_gbm_keeps_global_path_indices():
    import torch

    n = (1 << 18) + 77
    key = W.gbm_key(4)
    host = H.gbm_solver(n, call=pd.cuda_call_jit, math_mode=SAFE, output="terminal", steps=8)(key)
    dev = H.gbm_solver(n, call=pd.cuda_call_jit, math_mode=SAFE, output="terminal", steps=8)(torch.from_numpy(key).cuda())
    np.testing.assert_array_equal(host, dev.cpu().numpy())
    np.testing.assert_allclose(host[:4096], oracle.gbm(key, 4096, s0=100.0, strike=105.0, r=0.03, sigma=0.2, t=1.0, steps=8)[0], rtol=1e-5)


def test_chunked_adaptive_counts_are_exact():
    n = 1 << 18
    x0, v0, mu = W.van_der_pol_ensemble(n)
    cfg = dict(t1=0.5, rtol=1e-5, atol=1e-7, dt0=1e-2, max_steps=400)
    state, accepted, rejected = H.vdp_solver(n, outputs=3, call=pd.cuda_call_jit, math_mode=SAFE, **cfg)(x0, v0, mu)
    pick = np.r_[0:300, n // 2:n // 2 + 300, n - 300:n]
    want = oracle.vdp_bs32(x0[pick], v0[pick], mu[pick], pow="pd", **cfg)
    np.testing.assert_array_equal(state[pick, 0], want[1])
    np.testing.assert_array_equal(accepted[pick], want[5].astype(np.int32))
    np.testing.assert_array_equal(rejected[pick], want[4].astype(np.int32))


# ------------------------------------------------------------------ device-resident stepping
def test_stepper_keeps_the_grid_on_the_device():
    # examples/04_reaction_diffusion.py:92-109: ping-pong buffers, one wait, device-side time
    size = 128
    u, v = W.gray_scott_initial_state(size, patches=4, patch=16)
    call = H.gs_solver(size, size, math_mode=SAFE, steps=4)
    stepper = pd.Stepper(call, u, v)
    stepper.advance(5).advance(2)
    got_u, got_v = stepper.read()
    want = oracle.gray_scott(u, v, steps=28)
    np.testing.assert_array_equal(got_u, want[0])
    np.testing.assert_array_equal(got_v, want[1])
    assert stepper.launches == 7 and stepper.gpu_time > 0.0


def test_stepper_graph_replay_equals_eager_stepping():
    size = 128
    u, v = W.gray_scott_initial_state(size, patches=4, patch=16)
    call = H.gs_solver(size, size, math_mode=SAFE, steps=2)
    eager = pd.Stepper(call, u, v).advance(25).read()
    graphed = pd.Stepper(call, u, v)
    graphed.advance(11, graph=True).advance(14, graph=True)   # odd and even counts, graph reused
    got = graphed.read()
    assert graphed.launches == 25
    np.testing.assert_array_equal(got[0], eager[0])
    np.testing.assert_array_equal(got[1], eager[1])
    want = oracle.gray_scott(u, v, steps=50)
    np.testing.assert_array_equal(got[0], want[0])


def test_stepper_feeds_state_and_keeps_parameters():
    n = 3000
    args = W.lotka_volterra_ensemble(n)
    stepper = pd.Stepper(H.lv_solver(n, steps=100, math_mode=SAFE), *args)
    got = stepper.advance(3).read()
    want = oracle.lv_rk4(*args, dt=0.01, steps=300)
    np.testing.assert_array_equal(got[0], want[0])
    np.testing.assert_array_equal(got[1], want[1])


def test_stepper_rejects_mismatched_feedback():
    n = 64
    args = W.lotka_volterra_ensemble(n)
    with pytest.raises(pd.DispatchError, match="one input slot per output"):
        pd.Stepper(H.lv_solver(n, steps=1), *args, feedback=[0])
    key = W.gbm_key(0)
    with pytest.raises(pd.DispatchError, match="cannot feed"):
        pd.Stepper(H.gbm_solver(32, steps=4), key)


def test_sequential_vmap_over_a_batch_axis():
    """tests/test_11_ffi.py in the reference: vmap with 'sequential' dispatches once
    per batch element; a call built without vmap_method refuses."""
    import torch

    n, batch = 257, 3
    ins = W.lotka_volterra_ensemble(n * batch)
    batched = [a.reshape(batch, n) for a in ins]
    call = H.lv_solver(n, steps=40, call=pd.cuda_call_jit, vmap_method="sequential", math_mode=pd.MathMode.SAFE)
    x, y = call.vmap(*batched)
    wx, wy = oracle.lv_rk4(*ins, dt=0.01, steps=40)
    np.testing.assert_array_equal(x.reshape(-1), wx)
    np.testing.assert_array_equal(y.reshape(-1), wy)
    # shared parameters, mapped initial states, device tensors
    dev = [torch.from_numpy(a).cuda() for a in batched[:2]] + [torch.from_numpy(a[0].copy()).cuda() for a in batched[2:]]
    x2, _ = call.vmap(*dev, in_axes=[0, 0, None, None, None, None])
    assert x2.is_cuda and x2.shape == (batch, n)
    np.testing.assert_array_equal(x2[0].cpu().numpy(), wx[:n])
    plain = H.lv_solver(n, steps=40, call=pd.cuda_call_jit)
    with pytest.raises(NotImplementedError, match="vmap_method"):
        plain.vmap(*batched)
    with pytest.raises(ValueError, match="batch size"):
        call.vmap(batched[0], batched[1][:2], *batched[2:])


# ------------------------------------------------------------------ the example scripts run
@pytest.mark.parametrize("script", ["01_ode_ensembles", "02_adaptive_lockstep", "03_sde_montecarlo",
                                    "04_reaction_diffusion", "05_df32_precision", "06_custom_rhs",
                                    "07_multi_gpu_stencil"])
def test_example_scripts_run(script):
    import runpy
    from pathlib import Path

    path = Path(__file__).resolve().parent.parent / "examples" / f"{script}.py"
    runpy.run_path(str(path), run_name="__main__")
