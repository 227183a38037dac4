"""`.interpret` provider backed by the CPU oracle: what `call.interpret(*args)`
returns in the reference (the Pallas interpreter's result for the same call),
here computed by oracle/ for each kernel family."""

import numpy as np

import oracle


def interpret(family, pallas_kwargs, *args, pow_flavour="pd"):
    c = family.constants
    name = family.name
    outs = pallas_kwargs.get("out_shape")
    n_out = len(outs) if isinstance(outs, (list, tuple)) else 1
    if name == "lv_rk4":
        return oracle.lv_rk4(*args, dt=c["dt"], steps=c["steps"])
    if name == "lv_rk4_df32":
        return oracle.lv_rk4_df32(*args, dt=c["dt"], steps=c["steps"])
    if name == "vdp_bs32":
        keys = ("t1", "rtol", "atol", "dt0", "pcoeff", "icoeff", "safety", "factor_min", "factor_max",
                "error_order", "max_steps")
        t, x, v, steps, rejected, real = oracle.vdp_bs32(*args, pow=pow_flavour, **{k: c[k] for k in keys})
        if n_out == 6:
            return t, x, v, steps, rejected, real
        if n_out == 5:
            return t, x, v, steps, rejected
        return np.stack([x, v], axis=1), real.astype(np.int32), rejected.astype(np.int32)
    if name == "gbm_threefry":
        grid = pallas_kwargs["grid"]
        n = int(grid[0] if isinstance(grid, (tuple, list)) else grid)
        terminal, payoff = oracle.gbm(args[0], n, s0=c["s0"], strike=c["strike"], r=c["r"], sigma=c["sigma"],
                                      t=c["t"], steps=c["steps"], path_offset=c["path_offset"])
        first = payoff if c["output"] == "payoff" else terminal
        if n_out == 2:
            p64 = payoff.astype(np.float64)
            return first, np.array([p64.sum(), (p64 * p64).sum()])
        return first
    if name == "gbm_pcg":
        grid = pallas_kwargs["grid"]
        n = int(grid[0] if isinstance(grid, (tuple, list)) else grid)
        terminal, payoff = oracle.gbm_pcg(n, s0=c["s0"], strike=c["strike"], r=c["r"], sigma=c["sigma"], t=c["t"],
                                          steps=c["steps"], path_offset=c["path_offset"])
        first = payoff if c["output"] == "payoff" else terminal
        if n_out == 2:
            p64 = payoff.astype(np.float64)
            return first, np.array([p64.sum(), (p64 * p64).sum()])
        return first
    if name == "gray_scott":
        if c["halo"]:
            raise NotImplementedError("the oracle steps whole periodic grids only")
        return oracle.gray_scott(*args, steps=c["steps"], du=c["du"], dv=c["dv"], f=c["f"], k=c["k"], dt=c["dt"])
    if name == "kepler_rk4_df32":
        return oracle.kepler_rk4_df32(args, dt=c["dt"], gm=c["gm"], steps=c["steps"])
    if name == "threefry_bits":
        grid = pallas_kwargs["grid"]
        n = int(grid[0] if isinstance(grid, (tuple, list)) else grid)
        if c["op"] == "pcg":
            return oracle.pcg_hash(n)
        if c["op"] == "bits":
            return oracle.random_bits(args[0], n)
        if c["op"] == "uniform":
            return oracle.uniform(args[0], n)
        if c["op"] == "fold_in":
            return oracle.fold_in(args[0], args[1])
        return oracle.fold_uniform(args[0], n, c["count"])
    raise NotImplementedError(name)
