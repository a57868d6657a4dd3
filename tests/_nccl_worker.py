"""Worker of tests/test_multigpu_gpu.py: one rank (one GPU) of a data-parallel job.

Runs the reference's allreduce+SGD known-answer test across the ranks and a few
training steps, and checks both against the CPU oracle configured with the same
number of ranks. Exits non-zero on any mismatch."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
from helpers import make_problem, rel_fro  # noqa: E402
from oracle import oracle as O  # noqa: E402
from tbb_test_b200 import _capi as K  # noqa: E402
from tbb_test_b200.mlp import MLP, nccl_unique_id  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")  # only carries the NCCL id and the verdicts

    def fresh_id():
        # an NCCL unique id founds exactly one communicator: every handle gets its own
        box = [nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        return box[0]


    # 1. the reference's self-check (mlp_omp.cc:325-373) with one GPU per socket
    nrows, ncols = 256, 512
    w, g, e = O.kat(world, nrows, ncols)
    # through both routes: reduce-scatter + SGD on the owned slice + allgather of the weights (the
    # reference's own, mlp_omp.cc:90-146,240-258), and allreduce + SGD on every rank; fp32 operands
    # and bf16 operands (where the allgather carries the bf16 copy and the download gathers the masters)
    for shard in (1, 0):
        for prec in (K.PREC_FP32, K.PREC_BF16):
            dev = MLP([ncols, nrows], 8 * world, rank=rank, world_size=world, device=local, lr=1.0,
                      nccl_id=fresh_id(), shard_update=shard, precision=prec)
            dev.upload_weights(0, w[rank])
            dev.upload_weight_grad(0, g[rank])
            dev.update_weight(0)
            got = dev.weights(0)
            assert np.array_equal(got, e), f"rank {rank}: allreduce+SGD known-answer test failed (shard {shard})"
            if shard == 1 and prec == K.PREC_FP32:
                ms, checksum = dev.allreduce_bench(1 << 20, K.DTYPE_F32, 2, 5)
                ref = sum(O.fill_uniform(1, 4096, r, -1.0, 1.0).astype(np.float64).sum() for r in range(world))
                assert abs(checksum - ref) <= 1e-3, (checksum, ref)
                # the same sum on a caller-owned device buffer (configuration 2 through the boundary)
                buf = torch.from_numpy(O.fill_uniform(1, 70001, rank, -1.0, 1.0).ravel().copy()).cuda()
                dev.allreduce(buf.data_ptr(), buf.numel(), K.DTYPE_F32)
                want = np.zeros(70001, np.float64)
                for r in range(world):
                    want += O.fill_uniform(1, 70001, r, -1.0, 1.0).ravel()
                assert np.abs(buf.cpu().numpy() - want).max() <= 1e-5  # the reference's own bound, mlp_omp.cc:360
            dev.close()

    # 1b. the same known-answer test and a few steps of the deep narrow shape through the
    # peer-memory path (gradient sums of up to 4 MiB bypass NCCL), against the NCCL path
    # (on two ranks always; on four and eight, where it has not run yet, with B2_TEST_P2P=1)
    if world == 2 or os.environ.get("B2_TEST_P2P") == "1":
        def connected(dev):
            descs = [None] * world
            dist.all_gather_object(descs, dev.p2p_describe())
            dev.p2p_connect(descs, 4 << 20)
            dist.barrier()
            return dev

        dev = connected(MLP([ncols, nrows], 8 * world, rank=rank, world_size=world, device=local, lr=1.0,
                            nccl_id=fresh_id()))
        dev.upload_weights(0, w[rank])
        dev.upload_weight_grad(0, g[rank])
        dev.update_weight(0)
        assert np.array_equal(dev.weights(0), e), f"rank {rank}: known-answer test through peer memory failed"
        dist.barrier()
        dev.close()
        nf_s, batch_s = [128, 512, 512, 64], 64 * world + 3
        ws_s, x_s, t_s = make_problem(O, nf_s, batch_s)
        results = []
        for p2p in (False, True):
            dev = MLP(nf_s, batch_s, rank=rank, world_size=world, device=local, precision=K.PREC_FP32, lr=0.01,
                      nccl_id=fresh_id(), ar_bucket_mb=0, shard_update=0)
            if p2p:
                connected(dev)
            for l in range(3):
                dev.upload_weights(l, ws_s[l])
            dev.upload_input(x_s)
            dev.upload_target(t_s)
            dev.step(4)
            results.append([dev.weights(l) for l in range(3)] + [dev.weight_grad(l) for l in range(3)])
            dist.barrier()
            dev.close()
        for a, b in zip(*results):  # same sums, possibly in another order
            assert rel_fro(b, a) <= 1e-6
        # every rank holds identical weights after the peer-memory steps
        box = [None] * world
        dist.all_gather_object(box, [float(np.float64(x).sum()) for x in results[1][:3]])
        assert all(b == box[0] for b in box)

    # 2. training steps: every precision, ragged batch split, against the oracle with `world` ranks
    nf, batch, steps = [256, 512, 256, 128], 200 + world, 3
    ws, x, t = make_problem(O, nf, batch)
    for prec, rounding, tol in ((K.PREC_FP32, O.ROUND_NONE, dict(state=2e-5, grad=2e-5)),
                                (K.PREC_BF16, O.ROUND_BF16, dict(state=5e-3, grad=1e-1))):
        # two-stream schedule with the default gradient buckets, with one collective per layer,
        # and the serial schedule; sharded update (default) and allreduce + full update
        # ... and, one bucket per layer, the two other allgather orders of the sharded update
        for overlap, bucket, shard, ag_order in ((True, -1, 1, None), (True, 0, 1, None), (False, -1, 1, None),
                                                 (True, -1, 0, None), (False, 0, 0, None),
                                                 (True, 0, 1, "eager"), (True, 0, 1, "grouped")):
            if ag_order:
                os.environ["B2_AG_ORDER"] = ag_order
            else:
                os.environ.pop("B2_AG_ORDER", None)
            dev = MLP(nf, batch, rank=rank, world_size=world, device=local, precision=prec, lr=0.01,
                      nccl_id=fresh_id(), overlap=overlap, ar_bucket_mb=bucket, shard_update=shard)
            orc = O.Oracle(nf, batch, nranks=world, mode=O.MODE_BASELINE, rounding=rounding, lr=0.01)
            for l in range(3):
                dev.upload_weights(l, ws[l])
                orc.set_weights(l, ws[l])
            dev.upload_input(x)
            dev.upload_target(t)
            orc.set_input(x)
            orc.set_target(t)
            dev.step(steps)
            orc.step(steps)
            b0, b1 = dev.rows
            assert (b0, b1) == O.batch_range(batch, world, rank)
            assert rel_fro(dev.activation(3), orc.activation(3)[b0:b1]) <= tol["state"]
            for l in range(3):
                assert rel_fro(dev.weights(l) - ws[l], orc.weights(l) - ws[l]) <= max(tol["state"], 3e-2 if prec else 0), l
                if shard == 0:  # summed over ranks (with the sharded update no rank holds the whole sum)
                    assert rel_fro(dev.weight_grad(l), orc.weight_grad(l)) <= tol["grad"], l
            loss = torch.tensor([dev.loss()], dtype=torch.float64)
            dist.all_reduce(loss)
            assert abs(loss.item() - orc.loss()) <= 2e-3 * abs(orc.loss())
            dev.close()
            orc.close()
    os.environ.pop("B2_AG_ORDER", None)
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank}: ok")


if __name__ == "__main__":
    main()
