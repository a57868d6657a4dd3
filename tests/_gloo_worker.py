"""Worker of tests/test_multirank_cpu.py: one data-parallel rank on the CPU (gloo).

Each rank takes the batch rows the host mirror's get_partition() assigns to it,
runs forward / backward on those rows with the oracle's GEMM, sums the weight
gradients over ranks with an all-reduce and applies SGD - the same decomposition
the GPU ranks use with NCCL.  With argv[3] = "shard" the update takes the library's
sharded route instead, on the library's own slab layout, bucket rule and slice
ownership (csrc/bucket_plan.h through the host library): reduce the gradient slab
bucket by bucket so that each rank holds the sum of its slice, SGD on that slice,
allgather of the updated weights.  Rank 0 writes the resulting weights to argv[1]."""
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
    shard = len(sys.argv) > 3 and sys.argv[3] == "shard"
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    host = C.CDLL(build.HOST_LIB)
    rng = (C.c_int * 2)()
    host.b2h_get_partition(world, batch, rank, 1, 0, rng)
    b0, b1 = rng[0], rng[1]
    nf, lr, steps = [48, 64, 32], 0.05, 3
    ws, x, t = make_problem(O, nf, batch)
    L = len(nf) - 1
    if shard:
        elems = (C.c_size_t * L)(*[nf[l + 1] * nf[l] for l in range(L)])
        off, pad = (C.c_size_t * L)(), (C.c_size_t * L)()
        host.b2h_slab_layout.restype = C.c_size_t
        total = host.b2h_slab_layout(elems, L, world, off, pad)
        low, high = (C.c_int * L)(), (C.c_int * L)()
        # one bucket for both layers (target 1 MiB), so that slices cross the layer boundary
        host.b2h_plan_buckets((C.c_size_t * L)(*[4 * e for e in elems]), L, world, 1, 1, C.c_double(0.0), low, high)
        w_slab = np.zeros(total, np.float32)
        for l in range(L):
            w_slab[off[l]:off[l] + elems[l]] = ws[l].ravel()
    for _ in range(steps):
        if shard:
            ws = [w_slab[off[l]:off[l] + elems[l]].reshape(nf[l + 1], nf[l]).copy() for l in range(L)]
        acts = [x[b0:b1]]
        for l in range(L):
            z = O.sgemm(False, True, acts[l], ws[l]) if b1 > b0 else np.zeros((0, nf[l + 1]), np.float32)
            acts.append(np.maximum(z, 0) if l < L - 1 else z)
        dz = (acts[L] - t[b0:b1]) * np.float32(1.0 / batch)
        new_ws = list(ws)
        g_slab = np.zeros(total, np.float32) if shard else None
        for l in range(L - 1, -1, -1):
            dw = O.sgemm(True, False, dz, acts[l]) if b1 > b0 else np.zeros_like(ws[l])
            g = torch.from_numpy(dw.copy())
            if shard:
                g_slab[off[l]:off[l] + elems[l]] = dw.ravel()
                if low[l] == l:  # the bucket is complete: reduce-scatter, SGD on the own slice, allgather
                    rng4 = (C.c_size_t * 4)()
                    host.b2h_bucket_slice(off, pad, l, high[l], world, rank, rng4)
                    begin, count, sb, sc = rng4[0], rng4[1], rng4[2], rng4[3]
                    assert count % world == 0 and sc * world == count
                    mine = None
                    for r in range(world):  # gloo has no reduce-scatter: one rooted reduction per slice
                        part = torch.from_numpy(g_slab[begin + r * sc:begin + (r + 1) * sc].copy())
                        dist.reduce(part, dst=r, op=dist.ReduceOp.SUM)
                        if r == rank:
                            mine = part.numpy()
                    w_slab[sb:sb + sc] = (w_slab[sb:sb + sc] - np.float32(lr) * mine).astype(np.float32)
                    pieces = [torch.zeros(sc, dtype=torch.float32) for _ in range(world)]
                    dist.all_gather(pieces, torch.from_numpy(w_slab[sb:sb + sc].copy()))
                    for r in range(world):
                        w_slab[begin + r * sc:begin + (r + 1) * sc] = pieces[r].numpy()
            else:
                dist.all_reduce(g, op=dist.ReduceOp.SUM)
            if l > 0:
                da = O.sgemm(False, False, dz, ws[l]) if b1 > b0 else np.zeros((0, nf[l]), np.float32)
                dz = da * (acts[l] > 0)
            if not shard:
                new_ws[l] = (ws[l] - np.float32(lr) * g.numpy()).astype(np.float32)
        if not shard:
            ws = new_ws
    if shard:
        ws = [w_slab[off[l]:off[l] + elems[l]].reshape(nf[l + 1], nf[l]).copy() for l in range(L)]
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
