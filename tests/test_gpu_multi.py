"""Two (or more) GPUs, one process each, NCCL: the Gray-Scott halo exchange and
the Monte Carlo all-reduce with the CUDA kernels.  Skipped on a single GPU."""

import os
import socket

import numpy as np
import pytest

import oracle
from palladium_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


VDP_CFG = dict(t1=2.0, rtol=1e-5, atol=1e-7, dt0=0.01, max_steps=3000)
N_VDP = 20_011


def _sorted_vdp(n):
    x0, v0, mu = W.van_der_pol_ensemble(n)
    return x0, v0, np.sort(mu)


def _worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist

    from palladium_b200 import sharded

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        rows, cols, steps, halo = 250, 512, 18, 4   # 250 rows: unequal slabs on 4 ranks (63, 63, 62, 62)
        u0, v0 = W.gray_scott_initial_state(512, seed=11, patches=16, patch=32)
        u0, v0 = u0[:rows].copy(), v0[:rows].copy()
        lo, hi = sharded.partition(rows, world, rank)
        results = []
        for overlap in (True, False):
            slab = sharded.GrayScottSlab(torch.from_numpy(u0[lo:hi]).cuda(), torch.from_numpy(v0[lo:hi]).cuda(), rows,
                                         halo=halo, constants=dict(oracle.GS_DEFAULTS), math_mode="safe",
                                         overlap=overlap)
            slab.advance(steps)
            results.append(slab.owned())
        assert torch.equal(results[0][0], results[1][0]) and torch.equal(results[0][1], results[1][1])
        # the exchange from inside the kernel: boundary rows stored into the neighbours' memory
        pushed = sharded.GrayScottSlab(torch.from_numpy(u0[lo:hi]).cuda(), torch.from_numpy(v0[lo:hi]).cuda(), rows,
                                       halo=halo, constants=dict(oracle.GS_DEFAULTS), math_mode="safe", push=True)
        pushed.advance(steps)
        pu, pv = (t.clone() for t in pushed.owned())
        assert pushed.exchanges == 1 and pushed.pushes == -(-steps // halo)
        pushed.close()
        assert torch.equal(pu, results[0][0]) and torch.equal(pv, results[0][1])
        # the same with the register-tile kernel (tiles fetched by the copy engine) doing the pushing,
        # forced here because the planner gives a grid this small to the block-tile kernel
        from palladium_b200 import _native

        with _native.thread_tuning(gs_persistent=2):
            pushed = sharded.GrayScottSlab(torch.from_numpy(u0[lo:hi]).cuda(), torch.from_numpy(v0[lo:hi]).cuda(), rows,
                                           halo=halo, constants=dict(oracle.GS_DEFAULTS), math_mode="safe", push=True)
            pushed.advance(steps)
            ru, rv = (t.clone() for t in pushed.owned())
            pushed.close()
        assert torch.equal(ru, results[0][0]) and torch.equal(rv, results[0][1])
        assert _native.device_status() == 0
        u, v = results[0]
        cfg = dict(s0=100.0, strike=100.0, r=0.05, sigma=0.2, t=1.0, steps=64)
        res = sharded.gbm_monte_carlo(W.gbm_key(0), 100_003, cfg, math_mode="safe")
        # adaptive ensemble with the stiffness sorted along the array: interleaved shares,
        # outputs all-gathered on the device and put back in trajectory order
        import palladium_b200 as pd
        from palladium_b200 import families, pl

        def make(n_local):
            sh = pl.ShapeDtypeStruct((n_local,), np.float32)
            return pd.cuda_call_jit(families.vdp_bs32(**VDP_CFG), grid=(n_local,), out_shape=(sh,) * 6,
                                    math_mode="safe")

        ins = [torch.from_numpy(a).cuda() for a in _sorted_vdp(N_VDP)]
        ens = {}
        for interleave in (False, True):
            outs, _ = sharded.run_ensemble(make, ins, interleave=interleave, gather=True)
            ens[interleave] = [o.cpu().numpy() for o in outs]
        for a, b in zip(ens[False], ens[True]):
            np.testing.assert_array_equal(a, b)
        torch.cuda.synchronize()
        np.savez(os.path.join(out_dir, f"r{rank}.npz"), u=u.cpu().numpy(), v=v.cpu().numpy(), lo=lo, hi=hi,
                 price=res.price, sums=np.array(res.sums), out=res.local_output.cpu().numpy(), plo=res.local_lo,
                 **{f"vdp{i}": a for i, a in enumerate(ens[True])})
    finally:
        dist.destroy_process_group()


def test_two_gpus_halo_exchange_and_all_reduce(tmp_path):
    import torch
    import torch.multiprocessing as mp

    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    rows, steps = 250, 18
    u0, v0 = W.gray_scott_initial_state(512, seed=11, patches=16, patch=32)
    want_u, want_v = oracle.gray_scott(u0[:rows].copy(), v0[:rows].copy(), steps=steps)
    cfg = dict(s0=100.0, strike=100.0, r=0.05, sigma=0.2, t=1.0, steps=64)
    terminal, payoff = oracle.gbm(W.gbm_key(0), 100_003, **cfg)
    p64 = payoff.astype(np.float64)
    want_vdp = oracle.vdp_bs32(*_sorted_vdp(N_VDP), pow="pd", **VDP_CFG)
    outs = []
    for rank in range(world):
        part = np.load(tmp_path / f"r{rank}.npz")
        lo, hi = int(part["lo"]), int(part["hi"])
        np.testing.assert_array_equal(part["u"], want_u[lo:hi])
        np.testing.assert_array_equal(part["v"], want_v[lo:hi])
        np.testing.assert_allclose(part["sums"][0], p64.sum(), rtol=1e-5)
        outs.append(part["out"])
        for i, want in enumerate(want_vdp):
            np.testing.assert_array_equal(part[f"vdp{i}"], want)
    np.testing.assert_allclose(np.concatenate(outs), terminal, rtol=1e-5)
