"""Out-of-bounds canaries.  Every output (and input) buffer is carved out of a
larger device allocation whose surroundings are filled with a sentinel; after
the launch the sentinels must be untouched, the inputs unchanged, and the
results equal to a launch on ordinary buffers.  Sizes are chosen to exercise
vector tails, partial tiles and grid-stride remainders."""

import numpy as np
import pytest

import palladium_b200 as pd
from palladium_b200 import _native
from palladium_b200 import workloads as W
from tests import helpers as H

pytestmark = pytest.mark.gpu
SENTINEL = 0x5A
PAD = 4096  # bytes of sentinel on each side (a multiple of 256 keeps the payload's alignment)


def _guarded(nbytes):
    import torch

    buf = torch.full((nbytes + 2 * PAD,), SENTINEL, dtype=torch.uint8, device="cuda")
    return buf, buf[PAD:PAD + nbytes]


def _run_guarded(call, arrays):
    """Launch `call` (an FfiCallable) with every operand inside a guarded allocation."""
    import torch

    shapes = tuple((a.shape, a.dtype.name) for a in arrays)
    spec, bound = call._entry(shapes)
    ins, in_bufs = [], []
    for a in arrays:
        buf, view = _guarded(a.nbytes)
        view.copy_(torch.from_numpy(a.reshape(-1).view(np.uint8).copy()).cuda())
        ins.append(view)
        in_bufs.append((buf, a))
    outs, out_bufs = [], []
    for info in spec.outputs:
        nbytes = int(np.prod(info.array_shape)) * info.dtype.itemsize
        buf, view = _guarded(nbytes)
        outs.append(view)
        out_bufs.append((buf, info, nbytes))
    bound.launch_device(ins, outs)
    torch.cuda.synchronize()
    for buf, a in in_bufs:
        host = buf.cpu().numpy()
        assert (host[:PAD] == SENTINEL).all() and (host[PAD + a.nbytes:] == SENTINEL).all()
        np.testing.assert_array_equal(host[PAD:PAD + a.nbytes], a.reshape(-1).view(np.uint8))
    results = []
    for buf, info, nbytes in out_bufs:
        host = buf.cpu().numpy()
        assert (host[:PAD] == SENTINEL).all(), "write before the output buffer"
        assert (host[PAD + nbytes:] == SENTINEL).all(), "write past the output buffer"
        results.append(host[PAD:PAD + nbytes].view(info.dtype).reshape(info.array_shape).copy())
    return results


def _plain(call, arrays):
    out = call(*arrays)
    return list(out) if isinstance(out, tuple) else [out]


@pytest.mark.parametrize("n", [1, 3, 127, 4097, 600_001])
@pytest.mark.parametrize("mode", [pd.MathMode.SAFE, pd.MathMode.FAST])
def test_lv_rk4_stays_in_bounds(n, mode):
    args = list(W.lotka_volterra_ensemble(n))
    call = H.lv_solver(n, steps=3, call=pd.cuda_call_jit, math_mode=mode)
    for g, w in zip(_run_guarded(call, args), _plain(call, args)):
        np.testing.assert_array_equal(g, w)


@pytest.mark.parametrize("n,outputs", [(1, 6), (33, 5), (1000, 3), (70_001, 3)])
def test_adaptive_stays_in_bounds(n, outputs):
    args = list(W.van_der_pol_ensemble(n))
    call = H.vdp_solver(n, outputs=outputs, call=pd.cuda_call_jit, math_mode=pd.MathMode.SAFE, t1=0.2, max_steps=200)
    for g, w in zip(_run_guarded(call, args), _plain(call, args)):
        np.testing.assert_array_equal(g, w)


@pytest.mark.parametrize("n", [1, 255, 257, 100_003])
def test_gbm_stays_in_bounds(n):
    key = W.gbm_key(2)
    call = H.gbm_solver(n, with_sums=True, call=pd.cuda_call_jit, math_mode=pd.MathMode.SAFE, steps=5)
    got = _run_guarded(call, [key])
    want = _plain(call, [key])
    np.testing.assert_array_equal(got[0], want[0])
    np.testing.assert_allclose(got[1], want[1], rtol=1e-12)


@pytest.mark.parametrize("shape,steps,halo", [((7, 9), 3, 0), ((33, 132), 5, 0), ((17, 128), 4, 0), ((40, 244), 9, 0),
                                              ((48, 256), 4, 4), ((20, 128), 2, 3)])
@pytest.mark.parametrize("variant", [-1, 1, "register tiles"])
def test_gray_scott_stays_in_bounds(shape, steps, halo, variant):
    rows, cols = shape
    form = -1
    if variant == "register tiles":   # the copy-engine fed kernel, forced also on grids the planner gives to the block kernel
        variant, form = -1, 2
    rng = np.random.default_rng(3)
    full = (rows + 2 * halo, cols)
    u = (1 - 0.5 * rng.random(full)).astype(np.float32)
    v = (0.25 * rng.random(full)).astype(np.float32)
    with _native.thread_tuning(gs_variant=variant, gs_persistent=form):
        call = H.gs_solver(rows, cols, call=pd.cuda_call_jit, math_mode=pd.MathMode.SAFE, steps=steps, halo=halo)
        got = _run_guarded(call, [u, v])
        want = _plain(call, [u, v])
    valid = slice(halo, full[0] - halo) if halo else slice(None)
    for g, w in zip(got, want):
        np.testing.assert_array_equal(g[valid], w[valid])
        if halo:  # rows the call never writes must still hold the sentinel bytes
            untouched = np.r_[0:1, full[0] - 1:full[0]]
            assert (g[untouched].view(np.uint8) == SENTINEL).all()


@pytest.mark.parametrize("n", [1, 129, 5000])
def test_df32_stays_in_bounds(n):
    _, pairs = W.kepler_ensemble(n)
    call = H.kepler_solver(n, call=pd.cuda_call_jit, dt=1e-3, steps=4)
    for g, w in zip(_run_guarded(call, list(pairs)), _plain(call, list(pairs))):
        np.testing.assert_array_equal(g, w)
    args = list(W.lotka_volterra_ensemble(n))
    call = H.lv_solver(n, steps=4, df32=True, call=pd.cuda_call_jit, math_mode=pd.MathMode.SAFE)
    for g, w in zip(_run_guarded(call, args), _plain(call, args)):
        np.testing.assert_array_equal(g, w)
