"""Several configurations of the training step in ONE multi-rank job (one process start-up and
one NCCL bootstrap per rank instead of one per configuration): for comparing schedules.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        tbb_test_b200/step_sweep.py c4|c5 ['{"shard_update": 0}' '{"comm_sms": 0, "env": {"B2_AG_ORDER": "eager"}}' ...]

Every argument after the workload is a JSON object of MLP keyword arguments (shard_update,
comm_sms, ar_bucket_mb, allreduce, ...) plus an optional "env" object of environment switches
read by b2_create. Rank 0 prints one JSON line per configuration: milliseconds per step (CUDA
events inside the library, max over ranks, SWEEP_STEPS steps after 5 warm-up steps) and samples/s.
Bf16 operands; seeded synthetic data as in bench.py. No checks beyond the loss: bench.py is the
benchmark, this is the comparison tool."""
import os, sys, json, time
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # repository root
import numpy as np, torch, torch.distributed as dist
from tbb_test_b200 import _capi as K
from tbb_test_b200.mlp import MLP, nccl_unique_id
import bench as B
rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dist.init_process_group("nccl", device_id=torch.device("cuda", local))
wl = sys.argv[1] if len(sys.argv) > 1 else "c4"
nf, batch, winit, desc = B.WORKLOADS[wl]
L = len(nf) - 1
steps = int(os.environ.get("SWEEP_STEPS", 30))
def fresh():
    box = [nccl_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    return box[0]
def mx(v):
    t = torch.tensor([v], dtype=torch.float64, device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MAX); return float(t.item())
x = None
configs = [dict(shard_update=1), dict(shard_update=0), dict(shard_update=1, comm_sms=0), dict(shard_update=1, comm_sms=12),
           dict(shard_update=1, comm_sms=32), dict(shard_update=1, ar_bucket_mb=0), dict(shard_update=1, ar_bucket_mb=64),
           dict(shard_update=1, ar_bucket_mb=128), dict(shard_update=1, ar_bucket_mb=256),
           dict(shard_update=1, env={"B2_BUCKET_GROWTH": "1.0"}), dict(shard_update=1, env={"B2_BUCKET_GROWTH": "2.0"}),
           dict(allreduce=False)]
if len(sys.argv) > 2:
    configs = [json.loads(a) for a in sys.argv[2:]]
for cfg in configs:
    cfg = dict(cfg)
    env = cfg.pop("env", {})
    for k, v in env.items(): os.environ[k] = v
    kw = dict(rank=rank, world_size=world, device=local, precision=K.PREC_BF16, lr=0.01, grad_bf16=(wl == "c5"))
    kw.update(cfg)
    if kw.get("allreduce", True): kw["nccl_id"] = fresh()
    try:
        dev = MLP(nf, batch, **kw)
    except Exception as e:
        for k in env: os.environ.pop(k, None)
        if rank == 0: print(json.dumps({"wl": wl, "cfg": cfg, "env": env, "error": str(e)[:200]}), flush=True)
        continue
    for k in env: os.environ.pop(k, None)
    rng = np.random.default_rng(0)
    for l in range(L): dev.upload_weights(l, B.draw_weights(rng, winit, (nf[l + 1], nf[l])))
    b0, b1 = dev.rows
    if x is None:
        x = np.zeros((batch, nf[0]), np.float32); t = np.zeros((batch, nf[-1]), np.float32)
        x[b0:b1] = np.random.default_rng([1, rank]).standard_normal((b1 - b0, nf[0]), dtype=np.float32)
        t[b0:b1] = np.where(np.random.default_rng([2, rank]).random((b1 - b0, nf[-1])) < 0.5, -1.0, 1.0)
    dev.upload_input(x); dev.upload_target(t)
    dev.step(5); dev.reset_timing()
    torch.cuda.synchronize(); dist.barrier()
    dev.step(steps)
    _, ms, n = dev.timing()
    ms = mx(ms / n)
    loss = dev.loss()
    dev.close()
    if rank == 0:
        print(json.dumps({"wl": wl, "cfg": cfg, "env": env, "ms_per_step": round(ms, 4), "samples_per_s": round(batch / ms * 1e3), "loss0": loss}), flush=True)
dist.barrier(); dist.destroy_process_group()
