"""Run-time right-hand sides, the parts that need no GPU: the definition-time
compile check (NVRTC runs without a device), call validation, and the generic
oracle loops against the family-specific ones (which carry the pins)."""

import numpy as np
import pytest

import oracle
import palladium_b200 as pd
from oracle import custom_ode as oracle_custom
from palladium_b200 import families, pl
from palladium_b200 import workloads as W

LV = "dy[0] = p[0]*y[0] - (p[1]*y[0])*y[1];\ndy[1] = (p[2]*y[0])*y[1] - p[3]*y[1];"
VDP = "dy[0] = y[1];\ndy[1] = (p[0]*(1.0f - y[0]*y[0]))*y[1] - y[0];"


def test_generic_oracle_loops_equal_the_pinned_family_oracles():
    ins = W.lotka_volterra_ensemble(500)
    got = oracle_custom.rk4(LV, 2, 4, ins, dt=0.01, steps=300)
    want = oracle.lv_rk4(*ins, dt=0.01, steps=300)
    for g, w in zip(got, want):
        np.testing.assert_array_equal(g, w)
    x0, v0, mu = W.van_der_pol_ensemble(100)
    cfg = dict(t1=2.0, rtol=1e-5, atol=1e-7, dt0=0.01, max_steps=3000)
    for flavour in ("pd", "libm"):
        got = oracle_custom.bs32(VDP, 2, 1, (x0, v0, mu), pow=flavour, **cfg)
        want = oracle.vdp_bs32(x0, v0, mu, pow=flavour, **cfg)
        for g, w in zip(got, want):
            np.testing.assert_array_equal(g, w)


def test_a_faulty_right_hand_side_fails_where_it_is_defined():
    with pytest.raises(pd.EmitError, match=r'rhs\(2\): error: identifier "q" is undefined'):
        families.custom_ode("dy[0] = y[0];\ndy[1] = q;", 2)
    # the check can be skipped (the error then surfaces at the first launch)
    families.custom_ode("dy[0] = q;", 1, check=False)


def test_constructor_argument_checks():
    with pytest.raises(pd.TraceError, match="method"):
        families.custom_ode(LV, 2, 4, method="euler")
    with pytest.raises(pd.TraceError, match="dim"):
        families.custom_ode(LV, 9, 0, check=False)
    with pytest.raises(pd.TraceError, match="nparam"):
        families.custom_ode(LV, 2, 9, check=False)
    with pytest.raises(pd.TraceError, match="non-empty"):
        families.custom_ode("  ", 2, 4)


def test_call_shape_is_validated_like_any_family():
    n = 64
    sh = pl.ShapeDtypeStruct((n,), np.float32)
    fam = families.custom_ode(LV, 2, 4, dt=0.01, steps=10)
    spec = families.trace(fam, dict(grid=(n,), out_shape=(sh, sh)))
    assert len(spec.inputs) == 6 and len(spec.outputs) == 2
    with pytest.raises(pd.TraceError, match="produces 2"):
        families.trace(fam, dict(grid=(n,), out_shape=(sh,)))
    adaptive = families.custom_ode(VDP, 2, 1, method="bs32")
    spec = families.trace(adaptive, dict(grid=(n,), out_shape=(sh,) * 6))
    assert len(spec.inputs) == 3 and len(spec.outputs) == 6
    call = pd.cuda_call(fam, grid=(n,), out_shape=(sh, sh))
    with pytest.raises(pd.DispatchError):
        call(*[np.zeros(n, np.float64)] * 6)
    report = call.explain(*[np.zeros(n, np.float32)] * 6)
    assert "pd_ode_rk4" in str(report)


# ------------------------------------------------------------------ complete caller-written kernels
SAXPY = '''
extern "C" __global__ void saxpy(const float* a, const float* x, const float* y, float* out,
                                 long long gx, long long gy, long long gz) {
    const long long i = PD_THREAD_X;
    if (i >= gx) return;
    out[i] = a[0] * x[i] + y[i];
}
'''


def test_source_kernel_is_checked_where_it_is_defined():
    families.source_kernel(SAXPY, "saxpy")
    with pytest.raises(pd.EmitError, match=r'source\(6\): error: identifier "b" is undefined'):
        families.source_kernel(SAXPY.replace("a[0]", "b[0]"), "saxpy")
    with pytest.raises(pd.TraceError, match="C identifier"):
        families.source_kernel(SAXPY, "not a name")
    with pytest.raises(pd.TraceError, match="non-empty"):
        families.source_kernel("", "saxpy")


def test_source_kernel_takes_its_operands_from_the_call():
    n = 1000
    fam = families.source_kernel(SAXPY, "saxpy")
    args = (np.ones(1, np.float32), np.zeros(n, np.float32), np.zeros(n, np.float32))
    spec = families.trace(fam, dict(grid=(n,), out_shape=pl.ShapeDtypeStruct((n,), np.float32)), *args)
    assert [i.array_shape for i in spec.inputs] == [(1,), (n,), (n,)] and spec.outputs[0].array_shape == (n,)
    call = pd.cuda_call(fam, grid=(n,), out_shape=pl.ShapeDtypeStruct((n,), np.float32), threadgroup=(64,))
    report = call.explain(*args)
    assert report.cuda_kernel == "saxpy" and report.cuda_grid == (16, 1, 1) and report.cuda_block == (64, 1, 1)
    assert report.msl_lines == len(SAXPY.splitlines())
    with pytest.raises(pd.TraceError, match="1 to 3 dimensions"):
        families.trace(fam, dict(grid=(2, 2, 2, 2), out_shape=pl.ShapeDtypeStruct((n,), np.float32)), *args)


def test_debug_msl_shows_the_text_handed_to_the_compiler():
    n = 8
    sh = pl.ShapeDtypeStruct((n,), np.float32)
    fam = families.custom_ode(VDP, 2, 1, method="bs32")
    text = pd.debug_msl(fam, grid=(n,), out_shape=(sh,) * 6, math_mode=pd.MathMode.SAFE)
    assert "#define PD_MODE 0" in text and "#define PD_DIM 2" in text
    assert VDP in text and 'extern "C" __global__' in text and "pd_ode_bs32" in text
    src = families.source_kernel(SAXPY, "saxpy")
    args = (np.ones(1, np.float32), np.zeros(n, np.float32), np.zeros(n, np.float32))
    assert SAXPY in pd.debug_msl(src, *args, grid=(n,), out_shape=sh)


# ------------------------------------------------------------------ the seven-stage 5(4) pairs
def _order_condition_residuals(A, b, c, order):
    """Largest residual of the rooted-tree order conditions up to `order` (at most 5), row sums included."""
    one = np.ones_like(c)
    Ac = A @ c
    r = [np.abs(A @ one - c).max(), b @ one - 1, b @ c - 1 / 2, b @ c**2 - 1 / 3, b @ Ac - 1 / 6, b @ c**3 - 1 / 4,
         b @ (c * Ac) - 1 / 8, b @ (A @ c**2) - 1 / 12, b @ (A @ Ac) - 1 / 24]
    if order >= 5:
        r += [b @ c**4 - 1 / 5, b @ (c**2 * Ac) - 1 / 10, b @ (c * (A @ c**2)) - 1 / 15, b @ (c * (A @ Ac)) - 1 / 30,
              b @ (Ac * Ac) - 1 / 20, b @ (A @ c**3) - 1 / 20, b @ (A @ (c * Ac)) - 1 / 40,
              b @ (A @ (A @ c**2)) - 1 / 60, b @ (A @ (A @ Ac)) - 1 / 120]
    return max(abs(float(v)) for v in r)


@pytest.mark.parametrize("method", ["dopri5", "tsit5"])
def test_tableau_meets_the_order_conditions(method):
    """The published coefficients are typed in, not derived: the 17 conditions for order five on the
    weights, the 8 for order four on weights minus error weights, and the row sums, on the values the
    compiled code holds (float32, hence the 1e-6), catch a wrong digit."""
    A, c, e = oracle_custom.tableau(method)
    b = A[6]
    assert _order_condition_residuals(A, b, c, 5) < 1.5e-6
    assert _order_condition_residuals(A, b - e, c, 4) < 1.5e-6
    assert _order_condition_residuals(A, b - e, c, 5) > 1e-4      # the embedded solution is of order four only
    assert c[5] == 1.0 and c[6] == 1.0                            # the last stage is the slope at the new point


def test_adaptive_pairs_against_a_float64_solution():
    """Van der Pol to t = 2 against scipy's DOP853 at rtol 1e-12: the error follows the tolerance and
    the 5(4) pairs need a fraction of the Bogacki-Shampine steps (measured at rtol 1e-6: 34 against 243)."""
    from scipy.integrate import solve_ivp

    n = 24
    x0, v0, mu = W.van_der_pol_ensemble(n)
    truth = np.array([solve_ivp(lambda t, y, m=float(mu[i]): [y[1], m * (1 - y[0] ** 2) * y[1] - y[0]], (0, 2.0),
                                [float(x0[i]), float(v0[i])], method="DOP853", rtol=1e-12, atol=1e-14).y[:, -1]
                      for i in range(n)])
    for rtol in (1e-4, 1e-5, 1e-6):
        cfg = dict(t1=2.0, rtol=rtol, atol=rtol * 1e-2, dt0=0.01, max_steps=3000)
        low = oracle_custom.bs32(VDP, 2, 1, (x0, v0, mu), **cfg)
        for method in ("dopri5", "tsit5"):
            out = oracle_custom.erk(VDP, 2, 1, (x0, v0, mu), method=method, **cfg)
            assert np.all(out[0] == 2.0)
            err = max(np.abs(out[1] - truth[:, 0]).max(), np.abs(out[2] - truth[:, 1]).max())
            assert err < 5 * rtol, (method, rtol, err)
            assert out[5].mean() < 0.5 * low[5].mean()
            np.testing.assert_array_equal(out[3] + out[4], 3000.0)


def test_adaptive_pairs_trace_like_the_other_adaptive_method():
    n = 64
    sh = pl.ShapeDtypeStruct((n,), np.float32)
    for method in ("dopri5", "tsit5"):
        fam = families.custom_ode(VDP, 2, 1, method=method)
        assert fam.constants["error_order"] == 5
        spec = families.trace(fam, dict(grid=(n,), out_shape=(sh,) * 6))
        assert len(spec.inputs) == 3 and len(spec.outputs) == 6
    assert families.custom_ode(VDP, 2, 1, method="bs32").constants["error_order"] == 3
    assert families.custom_ode(VDP, 2, 1, method="tsit5", error_order=4).constants["error_order"] == 4
