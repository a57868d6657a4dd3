"""Worker of tests/test_multirank_cpu.py: one data-parallel rank on the CPU (gloo).

Each rank takes the batch rows the host mirror's get_partition() assigns to it,
runs forward / backward on those rows with the oracle's GEMM, sums the weight
gradients over ranks with an all-reduce and applies SGD - the same decomposition
the GPU ranks use with NCCL.  Rank 0 writes the resulting weights to argv[1]."""
import ctypes as C
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
from helpers import make_problem  # noqa: E402
from oracle import oracle as O  # noqa: E402
from tbb_test_b200 import build  # noqa: E402


def main():
    out_path, batch = sys.argv[1], int(sys.argv[2])
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    host = C.CDLL(build.HOST_LIB)
    rng = (C.c_int * 2)()
    host.b2h_get_partition(world, batch, rank, 1, 0, rng)
    b0, b1 = rng[0], rng[1]
    nf, lr, steps = [48, 64, 32], 0.05, 3
    ws, x, t = make_problem(O, nf, batch)
    L = len(nf) - 1
    for _ in range(steps):
        acts = [x[b0:b1]]
        for l in range(L):
            z = O.sgemm(False, True, acts[l], ws[l]) if b1 > b0 else np.zeros((0, nf[l + 1]), np.float32)
            acts.append(np.maximum(z, 0) if l < L - 1 else z)
        dz = (acts[L] - t[b0:b1]) * np.float32(1.0 / batch)
        new_ws = list(ws)
        for l in range(L - 1, -1, -1):
            dw = O.sgemm(True, False, dz, acts[l]) if b1 > b0 else np.zeros_like(ws[l])
            g = torch.from_numpy(dw.copy())
            dist.all_reduce(g, op=dist.ReduceOp.SUM)
            if l > 0:
                da = O.sgemm(False, False, dz, ws[l]) if b1 > b0 else np.zeros((0, nf[l]), np.float32)
                dz = da * (acts[l] > 0)
            new_ws[l] = (ws[l] - np.float32(lr) * g.numpy()).astype(np.float32)
        ws = new_ws
    # the timing rule of the benchmark: a value is the max over ranks
    tmax = torch.tensor([float(rank + 1)], dtype=torch.float64)
    dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    assert tmax.item() == world
    if rank == 0:
        np.savez(out_path, *ws, rows=np.array([b0, b1]))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
