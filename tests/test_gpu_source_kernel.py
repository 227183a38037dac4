"""Complete caller-written kernels (CUDA source + entry-point name, compiled at
run time): the handler contract of native/ffi/palladium_ffi.cpp:110-193 with
CUDA C in place of MSL.  Checked against NumPy, against the oracle, and against
the hand-written families where a kernel restates one of them."""

import numpy as np
import pytest

import oracle
import palladium_b200 as pd
from palladium_b200 import families, pl
from palladium_b200 import workloads as W
from tests import helpers as H

pytestmark = pytest.mark.gpu

SAFE, RELAXED, FAST = pd.MathMode.SAFE, pd.MathMode.RELAXED, pd.MathMode.FAST

SAXPY = '''
extern "C" __global__ void saxpy(const float* a, const float* x, const float* y, float* out,
                                 long long gx, long long gy, long long gz) {
    const long long i = PD_THREAD_X;
    if (i >= gx) return;
    out[i] = a[0] * x[i] + y[i];
}
'''

# The reference's stencil kernel (examples/04_reaction_diffusion.py:61-74) as a user would write it.
GRAY_SCOTT = '''
extern "C" __global__ void gray_scott_cell(const float* u_, const float* v_, const float* c, float* uo, float* vo,
                                           long long cols, long long rows, long long gz) {
    const long long j = PD_THREAD_X, i = PD_THREAD_Y;
    if (i >= rows || j >= cols) return;
    const float DU = c[0], DV = c[1], F = c[2], FK = c[3], DT = c[4];
    const long long ip = (i == rows - 1) ? 0 : i + 1, im = (i == 0) ? rows - 1 : i - 1;
    const long long jp = (j == cols - 1) ? 0 : j + 1, jm = (j == 0) ? cols - 1 : j - 1;
    const float u = u_[i * cols + j], v = v_[i * cols + j];
    const float lap_u = (((u_[ip * cols + j] + u_[im * cols + j]) + u_[i * cols + jp]) + u_[i * cols + jm]) - 4.0f * u;
    const float lap_v = (((v_[ip * cols + j] + v_[im * cols + j]) + v_[i * cols + jp]) + v_[i * cols + jm]) - 4.0f * v;
    const float uvv = (u * v) * v;
    uo[i * cols + j] = u + DT * ((DU * lap_u - uvv) + F * (1.0f - u));
    vo[i * cols + j] = v + DT * ((DV * lap_v + uvv) - FK * v);
}
'''

RANDOM_BITS = '''
extern "C" __global__ void bits(const uint32_t* key, uint32_t* out, long long gx, long long gy, long long gz) {
    const long long i = PD_THREAD_X;
    if (i >= gx) return;
    out[i] = pd_random_bits(key[0], key[1], (uint32_t)i);
}
'''

FMA_PROBE = '''
extern "C" __global__ void probe(const float* a, const float* b, const float* c, float* out,
                                 long long gx, long long gy, long long gz) {
    const long long i = PD_THREAD_X;
    if (i >= gx) return;
    out[i] = a[i] * b[i] + c[i];
}
'''


def shaped(*shape, dtype=np.float32):
    return pl.ShapeDtypeStruct(shape, dtype)


@pytest.mark.parametrize("n", [1, 127, 128, 100_003])
def test_one_dimensional_kernel_with_a_scalar_operand(n, rng):
    x, y = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    a = np.array([2.5], np.float32)
    call = pd.cuda_call(families.source_kernel(SAXPY, "saxpy"), grid=(n,), out_shape=shaped(n), math_mode=SAFE)
    np.testing.assert_array_equal(call(a, x, y), a[0] * x + y)


@pytest.mark.parametrize("threadgroup", [None, (16, 16), (32, 1), (8, 4, 1)])
def test_two_dimensional_stencil_equals_the_family_and_the_oracle(threadgroup):
    rows, cols = 67, 130        # not multiples of any block shape: the edge blocks are trimmed by the kernel
    u0, v0 = W.gray_scott_initial_state(256, seed=11, patches=8, patch=16)
    u0, v0 = u0[:rows, :cols].copy(), v0[:rows, :cols].copy()
    g = oracle.GS_DEFAULTS
    consts = np.array([g["du"], g["dv"], g["f"], g["f"] + g["k"], g["dt"]], np.float64).astype(np.float32)
    call = pd.cuda_call(families.source_kernel(GRAY_SCOTT, "gray_scott_cell"), grid=(cols, rows),
                        out_shape=(shaped(rows, cols), shaped(rows, cols)), math_mode=SAFE, threadgroup=threadgroup)
    u, v = u0, v0
    for _ in range(3):
        u, v = call(u, v, consts)
    want_u, want_v = oracle.gray_scott(u0, v0, steps=3)
    np.testing.assert_array_equal(u, want_u)
    np.testing.assert_array_equal(v, want_v)
    fam_u, fam_v = H.gs_solver(rows, cols, math_mode=SAFE, steps=3)(u0, v0)
    np.testing.assert_array_equal(u, fam_u)
    np.testing.assert_array_equal(v, fam_v)


def test_shared_helpers_are_in_scope_threefry_bits():
    n = 5000
    key = W.gbm_key(7)
    call = pd.cuda_call(families.source_kernel(RANDOM_BITS, "bits"), grid=(n,), out_shape=shaped(n, dtype=np.uint32))
    got = call(key)
    np.testing.assert_array_equal(got, oracle.random_bits(key, n))
    np.testing.assert_array_equal(got, H.threefry_solver("bits", n)(key))


def test_math_mode_reaches_the_compiler():
    """SAFE forbids contraction, RELAXED and FAST fuse a*b+c (the reference checks
    the same through the FFI path, tests/test_11_ffi.py)."""
    a = np.array([1.0 + 2.0 ** -12], np.float32)
    b = np.array([1.0 + 2.0 ** -12], np.float32)
    c = -(a * b)                                  # minus the rounded product
    fam = families.source_kernel(FMA_PROBE, "probe")
    safe = pd.cuda_call(fam, grid=(1,), out_shape=shaped(1), math_mode=SAFE)(a, b, c)
    relaxed = pd.cuda_call(fam, grid=(1,), out_shape=shaped(1), math_mode=RELAXED)(a, b, c)
    fast = pd.cuda_call(fam, grid=(1,), out_shape=shaped(1), math_mode=FAST)(a, b, c)
    assert safe[0] == 0.0                         # two roundings: product rounds, then cancels exactly
    exact = float(np.float64(a[0]) * np.float64(b[0]) + np.float64(c[0]))
    assert exact != 0.0 and relaxed[0] == np.float32(exact) and fast[0] == np.float32(exact)


def test_device_tensors_and_jit_form():
    import torch

    n = 4096
    x = torch.arange(n, dtype=torch.float32, device="cuda")
    y = torch.ones(n, dtype=torch.float32, device="cuda")
    a = torch.tensor([3.0], device="cuda")
    call = pd.cuda_call_jit(families.source_kernel(SAXPY, "saxpy"), grid=(n,), out_shape=shaped(n))
    out = call(a, x, y)
    assert out.is_cuda and torch.equal(out, 3.0 * x + y)


def test_missing_entry_point_is_reported():
    fam = families.source_kernel(SAXPY, "no_such_kernel")
    call = pd.cuda_call(fam, grid=(8,), out_shape=shaped(8))
    with pytest.raises(pd.PalladiumError, match="no kernel named 'no_such_kernel'"):
        call(np.ones(1, np.float32), np.zeros(8, np.float32), np.zeros(8, np.float32))


def test_oversized_threadgroup_is_refused():
    call = pd.cuda_call(families.source_kernel(SAXPY, "saxpy"), grid=(8,), out_shape=shaped(8), threadgroup=(2048,))
    with pytest.raises(pd.PalladiumError, match="exceeds 1024 threads"):
        call(np.ones(1, np.float32), np.zeros(8, np.float32), np.zeros(8, np.float32))
