"""pd_gray_scott_static: the multi-step Gray-Scott entry point for callers that
cannot let the library allocate device memory (a host runtime that owns the
whole GPU memory pool, or a fixed-budget stepping loop that cannot afford the
device-wide synchronisation of cudaMalloc).  Its ping-pong fields live in a
fixed 8 MiB array inside the library instead of allocated scratch.

Checked here through the C ABI: the result must equal, bit for bit, what the
regular entry point (pd_launch with PD_FAMILY_GRAY_SCOTT) produces for the same
inputs -- both run the same kernels, so any difference means the static array
was addressed wrongly -- on two calls in a row, because the second call starts
from whatever the first one left in the shared array.  Collected last so that a
failure here cannot hide the other tests in a stop-at-first-failure run."""

import numpy as np
import pytest

from palladium_b200 import _native
from palladium_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _regular(params, mode, u, v):
    import torch

    uo, vo = torch.empty_like(u), torch.empty_like(v)
    nbytes = u.numel() * 4
    _native.launch(_native.FAMILY_IDS["gray_scott"], params, mode, (params.rows, params.cols), None,
                   [(u.data_ptr(), nbytes), (v.data_ptr(), nbytes)],
                   [(uo.data_ptr(), nbytes), (vo.data_ptr(), nbytes)],
                   stream=torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return uo, vo


def _static(params, mode, u, v):
    import torch

    uo, vo = torch.empty_like(u), torch.empty_like(v)
    _native.gray_scott_static(params, mode, u.data_ptr(), v.data_ptr(), uo.data_ptr(), vo.data_ptr(),
                              stream=torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return uo, vo


@pytest.mark.parametrize("rows,cols,steps,halo", [(256, 256, 6, 0), (100, 60, 5, 0), (64, 512, 3, 4), (128, 128, 1, 0),
                                                  (64, 512, 4, 4), (50, 60, 2, 2)])
def test_static_scratch_matches_regular_entry_point_twice(rows, cols, steps, halo):
    """The even step counts with a halo are the cases where the last ping-pong lands
    back in the caller's output after passing through the shared array while the
    updated row window shrinks by one row per step on each side."""
    import torch

    mode = 0  # SAFE: identical kernels, identical op order -> identical bits
    params = _native.GrayScottParams(0.16, 0.08, 0.035, 0.065, 1.0, steps, rows, cols, halo)
    rng = np.random.default_rng(21)
    shape = (rows + 2 * halo, cols)
    first = (torch.from_numpy((1.0 - 0.5 * rng.random(shape)).astype(np.float32)).cuda(),
             torch.from_numpy((0.25 * rng.random(shape)).astype(np.float32)).cuda())
    second = (torch.from_numpy((1.0 - 0.3 * rng.random(shape)).astype(np.float32)).cuda(),
              torch.from_numpy((0.4 * rng.random(shape)).astype(np.float32)).cuda())
    valid = slice(halo, shape[0] - halo) if halo else slice(None)
    for u, v in (first, second):  # the second call reuses the array the first one dirtied
        want_u, want_v = _regular(params, mode, u, v)
        got_u, got_v = _static(params, mode, u, v)
        assert torch.equal(got_u[valid], want_u[valid])
        assert torch.equal(got_v[valid], want_v[valid])


def test_static_scratch_matches_the_cpu_oracle():
    """Not only equal to the regular entry point (the same kernels) but to the CPU
    restatement of the reference's stencil, bit for bit under SAFE, on two calls in a row."""
    import torch

    import oracle

    rows, cols, steps = 96, 260, 7
    params = _native.GrayScottParams(0.16, 0.08, 0.035, 0.065, 1.0, steps, rows, cols, 0)
    rng = np.random.default_rng(5)
    for _ in range(2):
        u0 = (1.0 - 0.5 * rng.random((rows, cols))).astype(np.float32)
        v0 = (0.25 * rng.random((rows, cols))).astype(np.float32)
        got_u, got_v = _static(params, 0, torch.from_numpy(u0).cuda(), torch.from_numpy(v0).cuda())
        want_u, want_v = oracle.gray_scott(u0, v0, steps=steps)
        np.testing.assert_array_equal(got_u.cpu().numpy(), want_u)
        np.testing.assert_array_equal(got_v.cpu().numpy(), want_v)


def test_static_scratch_rejects_a_grid_it_cannot_launch():
    import torch

    from palladium_b200.errors import DispatchError

    params = _native.GrayScottParams(0.16, 0.08, 0.035, 0.065, 1.0, 2, 1 << 20, 1, 0)   # 2^20 cells, one column
    buf = torch.zeros(16, device="cuda")
    with pytest.raises(DispatchError, match="cannot be launched"):
        _native.gray_scott_static(params, 0, buf.data_ptr(), buf.data_ptr(), buf.data_ptr(), buf.data_ptr())


def test_static_scratch_rejects_more_cells_than_it_holds():
    import torch

    from palladium_b200.errors import DispatchError

    params = _native.GrayScottParams(0.16, 0.08, 0.035, 0.065, 1.0, 2, 1024, 1028, 0)
    buf = torch.zeros(16, device="cuda")
    with pytest.raises(DispatchError, match="exceed the fixed maximum"):
        _native.gray_scott_static(params, 0, buf.data_ptr(), buf.data_ptr(), buf.data_ptr(), buf.data_ptr())


def test_static_scratch_at_its_maximum_size():
    import torch

    size = 1024  # exactly 2^20 cells
    params = _native.GrayScottParams(0.16, 0.08, 0.035, 0.065, 1.0, 4, size, size, 0)
    u0, v0 = W.gray_scott_initial_state(size, patches=8)
    u, v = torch.from_numpy(u0).cuda(), torch.from_numpy(v0).cuda()
    want_u, want_v = _regular(params, 2, u, v)
    got_u, got_v = _static(params, 2, u, v)
    assert torch.equal(got_u, want_u) and torch.equal(got_v, want_v)
