"""Call builders shared by the tests: each mirrors the `make_solver` of the
reference test for that kernel (same grid / in_specs / out_specs / out_shape)."""

import numpy as np

import palladium_b200 as pd
from palladium_b200 import families, pl

F32 = np.float32
SPEC_1 = pl.BlockSpec((1,), lambda i: (i,))


def shaped(*shape, dtype=F32):
    return pl.ShapeDtypeStruct(shape, dtype)


def lv_solver(n, dt=0.01, steps=500, call=None, df32=False, **kw):
    """tests/test_06_capstone_rk4.py:42-53 in the reference."""
    fam = families.lv_rk4_df32(dt, steps) if df32 else families.lv_rk4(dt, steps)
    return (call or pd.cuda_call)(fam, grid=(n,), in_specs=[SPEC_1] * 6, out_specs=(SPEC_1, SPEC_1),
                                  out_shape=(shaped(n), shaped(n)), **kw)


def vdp_solver(n, outputs=6, call=None, math_mode=pd.MathMode.RELAXED, **constants):
    """tests/test_08_adaptive.py:145-154 (5 outputs) / examples/02:173-181 (6)."""
    fam = families.vdp_bs32(**constants)
    if outputs == 3:
        out_shape = (shaped(n, 2), shaped(n, dtype=np.int32), shaped(n, dtype=np.int32))
        out_specs = (pl.BlockSpec((1, 2), lambda i: (i, 0)), SPEC_1, SPEC_1)
    else:
        out_shape = tuple(shaped(n) for _ in range(outputs))
        out_specs = (SPEC_1,) * outputs
    return (call or pd.cuda_call)(fam, grid=(n,), in_specs=[SPEC_1] * 3, out_specs=out_specs, out_shape=out_shape,
                                  math_mode=math_mode)


def gbm_solver(n, with_sums=False, call=None, math_mode=pd.MathMode.FAST, **constants):
    """examples/03_sde_montecarlo.py:122-129."""
    fam = families.gbm_threefry(**constants)
    out_shape = shaped(n)
    out_specs = SPEC_1
    if with_sums:
        out_shape = (shaped(n), shaped(2, dtype=np.float64))
        out_specs = (SPEC_1, pl.BlockSpec((2,), lambda i: (0,)))
    return (call or pd.cuda_call)(fam, grid=(n,), in_specs=[pl.BlockSpec((2,), lambda i: (0,))],
                                  out_specs=out_specs, out_shape=out_shape, math_mode=math_mode)


def gbm_pcg_solver(n, with_sums=False, call=None, math_mode=pd.MathMode.FAST, **constants):
    """The hand-written variant: no inputs (examples/03_sde_montecarlo.py:78-93)."""
    fam = families.gbm_pcg(**constants)
    out_shape = (shaped(n), shaped(2, dtype=np.float64)) if with_sums else shaped(n)
    return (call or pd.cuda_call)(fam, grid=(n,), out_shape=out_shape, math_mode=math_mode)


def gs_solver(rows, cols, call=None, math_mode=pd.MathMode.FAST, **constants):
    """examples/04_reaction_diffusion.py:77-88."""
    fam = families.gray_scott(**constants)
    halo = fam.constants["halo"]
    shape = (rows + 2 * halo, cols)
    full = pl.BlockSpec(shape, lambda i, j: (0, 0))
    return (call or pd.cuda_call)(fam, grid=(rows, cols), in_specs=[full, full], out_specs=(full, full),
                                  out_shape=(shaped(*shape), shaped(*shape)), math_mode=math_mode)


def kepler_solver(n, call=None, **constants):
    fam = families.kepler_rk4_df32(**constants)
    return (call or pd.cuda_call)(fam, grid=(n,), in_specs=[SPEC_1] * 8, out_specs=(SPEC_1,) * 8,
                                  out_shape=tuple(shaped(n) for _ in range(8)), math_mode=pd.MathMode.SAFE)


def threefry_solver(op, n, count=1, call=None):
    fam = families.threefry_bits(op, count)
    if op in ("bits", "pcg"):
        out = shaped(n, dtype=np.uint32)
    elif op == "uniform":
        out = shaped(n)
    elif op == "fold_in":
        out = shaped(n, 2, dtype=np.uint32)
    else:
        out = shaped(n, count)
    return (call or pd.cuda_call)(fam, grid=(n,), out_shape=out, math_mode=pd.MathMode.SAFE)


def custom_solver(n, rhs, dim, nparam, call=None, math_mode=pd.MathMode.SAFE, **constants):
    """A run-time right-hand side behind the usual call shape."""
    fam = families.custom_ode(rhs, dim, nparam, **constants)
    n_out = dim if fam.constants["method"] == "rk4" else dim + 4
    return (call or pd.cuda_call)(fam, grid=(n,), in_specs=[SPEC_1] * (dim + nparam), out_specs=(SPEC_1,) * n_out,
                                  out_shape=tuple(shaped(n) for _ in range(n_out)), math_mode=math_mode)
