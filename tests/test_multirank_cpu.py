"""The N > 1 path without GPUs: world_size-2 and -3 `gloo` jobs on the CPU."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from helpers import make_problem, rel_fro

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def torchrun(nproc, script_args, port, timeout=300):
    env = dict(os.environ, OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port)] + script_args
    return subprocess.run(cmd, env=env, cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                          timeout=timeout)


@pytest.mark.parametrize("world,batch,route", [(2, 50, "allreduce"), (3, 50, "allreduce"), (2, 50, "shard"),
                                               (3, 50, "shard")])
def test_sharded_ranks_reproduce_the_single_job(native, oracle, tmp_path, world, batch, route):
    """Batch shards per rank, gradients summed over ranks: by allreduce + SGD everywhere, or by
    the reference's route (mlp_omp.cc:90-146,240-258) on the library's slab layout - reduce-scatter
    per bucket, SGD on the owned slice, allgather of the weights."""
    out = str(tmp_path / "w.npz")
    r = torchrun(world, [os.path.join(ROOT, "tests", "_gloo_worker.py"), out, str(batch), route],
                 29731 + world + (10 if route == "shard" else 0))
    assert r.returncode == 0, r.stdout[-2000:]
    got = np.load(out)
    nf = [48, 64, 32]
    ws, x, t = make_problem(oracle, nf, batch)
    o = oracle.Oracle(nf, batch, nranks=world, mode=oracle.MODE_BASELINE, lr=0.05)
    for l in range(2):
        o.set_weights(l, ws[l])
    o.set_input(x)
    o.set_target(t)
    o.step(3)
    for l in range(2):
        assert rel_fro(got[f"arr_{l}"] - ws[l], o.weights(l) - ws[l]) < 1e-4
    assert tuple(got["rows"]) == oracle.batch_range(batch, world, 0)


def test_reference_arm_prints_one_line_from_rank_zero(native, oracle):
    """bench.py --impl reference under a 2-rank launch: rank 0 times the reference's CPU
    path and prints the JSON line, the other rank exits quietly."""
    ref = os.path.join(ROOT, "oracle", "_ref", "mlp_omp_c1")
    if not os.path.exists(ref):
        pytest.skip("oracle/_ref not built (no reference sources on this machine)")
    r = torchrun(2, [os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--workload", "c1",
                     "--steps", "2", "--warmup", "1"], 29741)
    assert r.returncode == 0, r.stdout[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "samples/s" and d["value"] > 0
    assert d["cpu_baseline"]["kind"] in ("reference", "port")
    assert d["e2e"]["h2d_bytes_per_step"] == 0
