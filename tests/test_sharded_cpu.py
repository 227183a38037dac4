"""Multi-rank host logic on CPU ranks (gloo): partitioning, the Gray-Scott halo
exchange pattern, and the Monte Carlo reduction.  The step / path functions are
the oracle's, so what is tested is exactly the code that decides who owns what,
what is sent where, and how partial results combine."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from oracle import oracle_np
from palladium_b200 import sharded
from palladium_b200 import workloads as W
from palladium_b200.errors import DispatchError


def test_partition_covers_everything_once():
    for n in (0, 1, 7, 100, 100_000):
        for world in (1, 2, 3, 8):
            slabs = [sharded.partition(n, world, r) for r in range(world)]
            assert slabs[0][0] == 0 and slabs[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(slabs, slabs[1:]))
            sizes = [hi - lo for lo, hi in slabs]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharded.partition(10, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _np_slab_step(u, v, steps, halo, rows, cols, constants, math_mode):
    nu, nv = oracle_np.gray_scott_slab(u.numpy(), v.numpy(), steps=steps, halo=halo, **constants)
    return torch.from_numpy(nu), torch.from_numpy(nv)


def _oracle_paths(key, lo, n_local, constants, math_mode, output):
    terminal, payoff = oracle.gbm(key, n_local, path_offset=lo, **constants)
    p64 = payoff.astype(np.float64)
    return torch.from_numpy(terminal), np.array([p64.sum(), (p64 * p64).sum()])


def _worker(rank, world, port, case, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        if case == "gray_scott":
            rows, cols, steps, halo = 48, 20, 11, 3
            u0, v0 = W.gray_scott_initial_state(rows, seed=11, patches=3, patch=8)
            u0, v0 = u0[:, :cols].copy(), v0[:, :cols].copy()
            lo, hi = sharded.partition(rows, world, rank)
            slab = sharded.GrayScottSlab(torch.from_numpy(u0[lo:hi]), torch.from_numpy(v0[lo:hi]), rows, halo=halo,
                                         constants=dict(oracle.GS_DEFAULTS), step_fn=_np_slab_step)
            slab.advance(steps)
            u, v = slab.owned()
            np.savez(os.path.join(out_dir, f"gs_{rank}.npz"), u=u.numpy(), v=v.numpy(), lo=lo, hi=hi,
                     exchanges=slab.exchanges)
        elif case.startswith("ensemble"):
            n = 1001
            ins = W.lotka_volterra_ensemble(n)
            make = lambda n_local: (lambda *a: oracle.lv_rk4(*a, dt=0.01, steps=20))
            interleave = case.endswith("interleave")
            (x, y), idx = sharded.run_ensemble(make, ins, interleave=interleave, gather=True)
            (lx, ly), _ = sharded.run_ensemble(make, ins, interleave=interleave)
            np.savez(os.path.join(out_dir, f"ens_{rank}.npz"), x=x, y=y, lx=lx, ly=ly,
                     idx=np.arange(n)[idx])
        elif case == "leave":
            # rank 2 returns from the stepping loop after its first exchange (between steps, nothing of
            # its own in flight); the others find out through the bounded wait of their next exchange
            rows, cols, halo = 48, 20, 3
            u0, v0 = W.gray_scott_initial_state(rows, seed=11, patches=3, patch=8)
            u0, v0 = u0[:, :cols].copy(), v0[:, :cols].copy()
            lo, hi = sharded.partition(rows, world, rank)
            slab = sharded.GrayScottSlab(torch.from_numpy(u0[lo:hi]), torch.from_numpy(v0[lo:hi]), rows, halo=halo,
                                         constants=dict(oracle.GS_DEFAULTS), step_fn=_np_slab_step, timeout=1.5)
            store = dist.distributed_c10d._get_default_store()
            message = ""
            if rank == 2:
                slab.advance(halo)                       # one exchange, then it leaves
                store.wait(["leave_case/0", "leave_case/1"])   # stays alive, on the host, until the others are done
            else:
                try:
                    slab.advance(3 * halo)
                except DispatchError as exc:
                    message = str(exc)
                store.set(f"leave_case/{rank}", "done")
            with open(os.path.join(out_dir, f"leave_{rank}.txt"), "w") as fh:
                fh.write(f"{slab.exchanges}\n{message}")
            os._exit(0)    # the group is unusable after a collective that timed out: no orderly teardown
        elif case == "gbm":
            cfg = dict(s0=100.0, strike=100.0, r=0.05, sigma=0.2, t=1.0, steps=32)
            res = sharded.gbm_monte_carlo(W.gbm_key(0), 1001, cfg, path_fn=_oracle_paths)
            np.savez(os.path.join(out_dir, f"gbm_{rank}.npz"), price=res.price, stderr=res.stderr, lo=res.local_lo,
                     hi=res.local_hi, out=res.local_output.numpy(), sums=np.array(res.sums))
    finally:
        dist.destroy_process_group()


def _run(world, case, tmp_path):
    mp.spawn(_worker, args=(world, _free_port(), case, str(tmp_path)), nprocs=world, join=True)


@pytest.mark.parametrize("world", [2, 3])
def test_gray_scott_slabs_with_halo_exchange_equal_the_periodic_grid(world, tmp_path):
    _run(world, "gray_scott", tmp_path)
    rows, cols, steps = 48, 20, 11
    u0, v0 = W.gray_scott_initial_state(rows, seed=11, patches=3, patch=8)
    want_u, want_v = oracle.gray_scott(u0[:, :cols].copy(), v0[:, :cols].copy(), steps=steps)
    for rank in range(world):
        part = np.load(tmp_path / f"gs_{rank}.npz")
        lo, hi = int(part["lo"]), int(part["hi"])
        np.testing.assert_array_equal(part["u"], want_u[lo:hi])
        np.testing.assert_array_equal(part["v"], want_v[lo:hi])
        assert int(part["exchanges"]) == 4  # ceil(11 / 3)


@pytest.mark.parametrize("world,case", [(2, "ensemble"), (3, "ensemble_interleave")])
def test_ensemble_shares_and_gather_restore_trajectory_order(world, case, tmp_path):
    _run(world, case, tmp_path)
    n = 1001
    want_x, want_y = oracle.lv_rk4(*W.lotka_volterra_ensemble(n), dt=0.01, steps=20)
    seen = []
    for rank in range(world):
        part = np.load(tmp_path / f"ens_{rank}.npz")
        np.testing.assert_array_equal(part["x"], want_x)      # gathered: whole ensemble, original order
        np.testing.assert_array_equal(part["y"], want_y)
        np.testing.assert_array_equal(part["lx"], want_x[part["idx"]])   # local share only
        np.testing.assert_array_equal(part["ly"], want_y[part["idx"]])
        seen.append(part["idx"])
    assert sorted(np.concatenate(seen).tolist()) == list(range(n))
    if case.endswith("interleave"):
        assert seen[1][:3].tolist() == [1, 1 + world, 1 + 2 * world]


def test_ensemble_indices():
    assert sharded.ensemble_indices(10, 2, 1) == slice(5, 10)
    assert sharded.ensemble_indices(10, 3, 2, interleave=True) == slice(2, 10, 3)
    with pytest.raises(ValueError):
        sharded.ensemble_indices(10, 2, 2, interleave=True)


def test_gray_scott_single_rank_wraps_its_own_halo():
    rows, cols, steps = 32, 16, 7
    u0, v0 = W.gray_scott_initial_state(rows, patches=2, patch=8)
    u0, v0 = u0[:, :cols].copy(), v0[:, :cols].copy()
    slab = sharded.GrayScottSlab(torch.from_numpy(u0), torch.from_numpy(v0), rows, halo=4,
                                 constants=dict(oracle.GS_DEFAULTS), step_fn=_np_slab_step)
    slab.advance(steps)
    want = oracle.gray_scott(u0, v0, steps=steps)
    np.testing.assert_array_equal(slab.owned()[0].numpy(), want[0])
    np.testing.assert_array_equal(slab.owned()[1].numpy(), want[1])


def test_slab_argument_checks():
    u = torch.zeros(8, 4)
    with pytest.raises(ValueError, match="push=True needs the CUDA step function"):
        sharded.GrayScottSlab(u, u, 8, halo=2, step_fn=_np_slab_step, push=True)
    with pytest.raises(ValueError, match="expected fields of shape"):
        sharded.GrayScottSlab(u, u, 16, halo=2, step_fn=_np_slab_step)
    with pytest.raises(ValueError, match="cannot serve"):
        sharded.GrayScottSlab(u, u, 8, halo=9, step_fn=_np_slab_step)


def test_gbm_all_reduce_matches_single_rank(tmp_path):
    _run(2, "gbm", tmp_path)
    cfg = dict(s0=100.0, strike=100.0, r=0.05, sigma=0.2, t=1.0, steps=32)
    single = sharded.gbm_monte_carlo(W.gbm_key(0), 1001, cfg, path_fn=_oracle_paths)
    parts = [np.load(tmp_path / f"gbm_{r}.npz") for r in range(2)]
    for part in parts:
        np.testing.assert_allclose(part["sums"], single.sums, rtol=1e-13)
        np.testing.assert_allclose(float(part["price"]), single.price, rtol=1e-13)
    # the slabs are contiguous and the per-path results do not depend on the rank count
    assert int(parts[0]["lo"]) == 0 and int(parts[0]["hi"]) == int(parts[1]["lo"]) and int(parts[1]["hi"]) == 1001
    np.testing.assert_array_equal(np.concatenate([p["out"] for p in parts]), single.local_output.numpy())


def test_a_rank_that_leaves_between_steps_ends_the_others_wait_with_its_name(tmp_path):
    """World 3 on gloo: rank 2 returns after its first exchange.  The other two
    ranks' next exchange runs into the bounded wait and raises DispatchError
    naming rank 2, instead of waiting forever."""
    _run(3, "leave", tmp_path)
    gone = (tmp_path / "leave_2.txt").read_text().splitlines()
    assert gone[0] == "1"
    for rank in (0, 1):
        exchanges, message = (tmp_path / f"leave_{rank}.txt").read_text().split("\n", 1)
        assert int(exchanges) == 2                       # the first exchange completed, the second did not
        assert "did not complete within 1.5 s" in message
        assert "rank(s) [2] never arrived" in message
