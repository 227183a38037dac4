"""The halo exchange from inside the stencil kernel (pd_gray_scott_slab_push),
on one GPU: the neighbours' fields are ordinary buffers of the same device, so
the index arithmetic of the pushed rows is checked without a second GPU and
without any kernel waiting on another (launches run one after the other)."""

import numpy as np
import pytest

import oracle
import palladium_b200 as pd
from palladium_b200 import _native, sharded
from palladium_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _state(rows, cols, seed=11):
    size = max(rows, cols)
    u0, v0 = W.gray_scott_initial_state(size, seed=seed, patches=6, patch=16)
    return u0[:rows, :cols].copy(), v0[:rows, :cols].copy()


@pytest.mark.parametrize("rows,cols,halo,steps", [
    (64, 256, 8, 40),     # temporally blocked launches of 4 steps: the push rides on the last one
    (64, 256, 8, 37),     # a partial last cycle (5 steps: 4 + 1, the copy kernel pushes)
    (48, 256, 3, 9),      # launches of 3 steps
    (40, 256, 1, 5),      # one step per call: vec4 kernel + copy kernel
    (40, 100, 4, 12),     # columns not a multiple of 4: per-cell kernel + copy kernel
    (16, 512, 16, 32),    # the slab is exactly one halo deep: top and bottom rows are the same rows
])
@pytest.mark.parametrize("form", [0, 2])   # tiles in shared memory per block / in registers per warp (copy-engine fed)
def test_single_slab_wrapping_onto_itself(rows, cols, halo, steps, form):
    import torch

    u0, v0 = _state(rows, cols)
    slab = sharded.GrayScottSlab(torch.from_numpy(u0).cuda(), torch.from_numpy(v0).cuda(), rows, halo=halo,
                                 constants=dict(oracle.GS_DEFAULTS), math_mode="safe", push=True)
    with _native.thread_tuning(gs_persistent=form):
        slab.advance(steps)
    want_u, want_v = oracle.gray_scott(u0, v0, steps=steps)
    u, v = slab.owned()
    np.testing.assert_array_equal(u.cpu().numpy(), want_u)
    np.testing.assert_array_equal(v.cpu().numpy(), want_v)
    assert slab.exchanges == 1 and slab.pushes == -(-steps // halo)
    slab.close()


@pytest.mark.parametrize("form", [0, 2])
@pytest.mark.parametrize("halo,cycles", [(8, 3), (16, 2), (12, 3)])
def test_two_slabs_of_unequal_height_pushing_into_each_other(halo, cycles, form):
    """Two 'ranks' in one process: A owns rows [0, 48), B owns [48, 128).  Each call
    pushes into the other's output set; the calls run back to back on one stream,
    so A's whole call -- its push into B's ghost rows included -- is over before
    B's call starts: the extreme of one rank running ahead of the other.  With a
    halo of 12 or 16 a call is three or four fused launches, and none but the last
    may touch the output set the neighbour has already pushed into."""
    import torch

    rows_a, rows_b, cols = 48, 80, 256
    u0, v0 = _state(rows_a + rows_b, cols)
    g = oracle.GS_DEFAULTS
    mode = 0

    def slab(lo, hi):
        r = hi - lo
        sets = []
        for _ in range(2):
            sets.append([torch.zeros((r + 2 * halo, cols), device="cuda"), torch.zeros((r + 2 * halo, cols), device="cuda")])
        sets[0][0][halo:halo + r] = torch.from_numpy(u0[lo:hi]).cuda()
        sets[0][1][halo:halo + r] = torch.from_numpy(v0[lo:hi]).cuda()
        return sets

    a, b = slab(0, rows_a), slab(rows_a, rows_a + rows_b)
    # initial ghost rows by hand (periodic ring of two slabs: both neighbours are the other slab)
    for f in range(2):
        a[0][f][:halo] = b[0][f][rows_b:rows_b + halo]
        a[0][f][halo + rows_a:] = b[0][f][halo:2 * halo]
        b[0][f][:halo] = a[0][f][rows_a:rows_a + halo]
        b[0][f][halo + rows_b:] = a[0][f][halo:2 * halo]
    cur = 0
    with _native.thread_tuning(gs_persistent=form):
        for _ in range(cycles):
            out = 1 - cur
            for me, other, rows, other_rows in ((a, b, rows_a, rows_b), (b, a, rows_b, rows_a)):
                params = _native.GrayScottParams(g["du"], g["dv"], g["f"], g["k"], g["dt"], halo, rows, cols, halo)
                nb = _native.GsNeighbours(other[out][0].data_ptr(), other[out][1].data_ptr(), other_rows,
                                          other[out][0].data_ptr(), other[out][1].data_ptr(), other_rows)
                _native.gray_scott_slab_push(params, mode, me[cur][0].data_ptr(), me[cur][1].data_ptr(),
                                             me[out][0].data_ptr(), me[out][1].data_ptr(), nb,
                                             torch.cuda.current_stream().cuda_stream)
            cur = out
    torch.cuda.synchronize()
    want_u, want_v = oracle.gray_scott(u0, v0, steps=cycles * halo)
    got_u = torch.cat([a[cur][0][halo:halo + rows_a], b[cur][0][halo:halo + rows_b]]).cpu().numpy()
    got_v = torch.cat([a[cur][1][halo:halo + rows_a], b[cur][1][halo:halo + rows_b]]).cpu().numpy()
    np.testing.assert_array_equal(got_u, want_u)
    np.testing.assert_array_equal(got_v, want_v)
    assert _native.device_status() == 0


def test_argument_checks():
    import torch

    g = oracle.GS_DEFAULTS
    t = torch.zeros((24, 256), device="cuda")
    ok = _native.GsNeighbours(t.data_ptr(), t.data_ptr(), 8, t.data_ptr(), t.data_ptr(), 8)
    with pytest.raises(pd.DispatchError, match="needs a slab"):
        _native.gray_scott_slab_push(_native.GrayScottParams(g["du"], g["dv"], g["f"], g["k"], g["dt"], 1, 24, 256, 0),
                                     0, t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), ok)
    with pytest.raises(pd.DispatchError, match="cannot serve"):
        _native.gray_scott_slab_push(_native.GrayScottParams(g["du"], g["dv"], g["f"], g["k"], g["dt"], 4, 4, 256, 8),
                                     0, t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), ok)
    bad = _native.GsNeighbours(0, t.data_ptr(), 8, t.data_ptr(), t.data_ptr(), 8)
    with pytest.raises(pd.DispatchError, match="must not be NULL"):
        _native.gray_scott_slab_push(_native.GrayScottParams(g["du"], g["dv"], g["f"], g["k"], g["dt"], 4, 8, 256, 8),
                                     0, t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), bad)
