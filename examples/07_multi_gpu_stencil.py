"""The reaction-diffusion stepping loop on several GPUs (no counterpart among the
reference's examples: it is single-device; this extends examples/04).

    python examples/07_multi_gpu_stencil.py                         # one GPU
    torchrun --nproc-per-node 4 examples/07_multi_gpu_stencil.py    # one process per GPU

The periodic grid is cut into row slabs, one per rank.  Each slab carries `HALO`
ghost rows per side; a call advances `HALO` steps, and its last launch stores the
slab's boundary rows straight into the neighbours' ghost rows (their device memory,
over NVLink), so the only collective is a one-element all-reduce per call.
"""

import os
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))  # run from a source checkout

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from palladium_b200 import sharded, workloads  # noqa: E402

ROWS_PER_GPU, COLS, HALO, STEPS = 2048, 4096, 16, 640
CONSTANTS = dict(du=0.16, dv=0.08, f=0.035, k=0.065, dt=1.0)


def main():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rows_total = ROWS_PER_GPU * world
    lo, hi = sharded.partition(rows_total, world, rank)
    # every rank builds the same seeded initial state and keeps its own rows
    u0, v0 = workloads.gray_scott_initial_state(max(rows_total, COLS), seed=11, patches=16, patch=32)
    u = torch.from_numpy(u0[lo:hi, :COLS].copy()).cuda()
    v = torch.from_numpy(v0[lo:hi, :COLS].copy()).cuda()
    slab = sharded.GrayScottSlab(u, v, rows_total, halo=HALO, constants=CONSTANTS, math_mode="fast", push=True)
    slab.advance(HALO)                                  # warm-up: kernels loaded, ghost rows primed
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    slab.advance(STEPS)
    end.record()
    end.synchronize()
    ms = start.elapsed_time(end)
    uo, vo = slab.owned()
    total_v = torch.tensor([float(vo.double().sum())], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(total_v)
    if rank == 0:
        cells = rows_total * COLS
        print(f"Gray-Scott {rows_total} x {COLS} on {world} GPU(s): {STEPS} steps in {ms:.1f} ms "
              f"({ms / STEPS * 1e3:.1f} us per step, {cells * STEPS / ms / 1e6:.0f} G cell-steps/s), "
              f"{slab.pushes} in-kernel exchanges, sum(v) = {total_v.item():.3f}")
    slab.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
