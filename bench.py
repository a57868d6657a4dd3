#!/usr/bin/env python
"""Benchmark of the MLP training step (samples/s) on 1..8 B200s of one box.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c4|c1|c3] [--precision bf16|tf32|fp32]

One process per GPU (torchrun sets RANK / LOCAL_RANK / WORLD_SIZE); rank 0 prints
ONE JSON line.  A step is one pass of the hot path (forward, output gradient,
weight-gradient + input-gradient GEMMs per layer, gradient allreduce, SGD) over
one global batch of seeded synthetic data.  The default workload is the widest
configuration that fits one GPU: 8 layers of 4096x4096, global batch 8192,
bf16 tensor-core operands with fp32 accumulation and fp32 master weights; with
N GPUs the global batch is split evenly (strong scaling) and each layer's 64 MiB
fp32 gradient is summed with NCCL on a side stream.

kat       before anything is timed every rank runs the reference's own start-up
          self-check (allreduce + SGD known-answer test, mlp_omp.cc:325-373) through
          b2_allreduce_sgd; after the timed steps the ranks compare fingerprints of
          their weights. A failed check ends the run with a non-zero exit code.
value     global batch * K / device time of K steps (CUDA events on the launching
          stream inside the library; max over ranks), inputs resident in HBM, no
          per-phase events in the timed steps
e2e       same metric through b2_train_step_host_async: every step copies that
          step's inputs and targets from pinned host memory and reads the loss back
roofline  the GEMMs: 2mnk flops of all GEMM launches / the time during which a GEMM
          was running, from a second, shorter run with per-phase events, against the
          measured cuBLAS bf16 peak of MEASURED_PEAKS.json (burst figure: the timed
          region is well under a second; the sustained figure is quoted beside it)
cpu_baseline / --impl reference
          the reference's own mlp_omp (oracle/_ref, built from the unmodified
          sources with only the workload literals replaced) timed on the host cores
"""
import argparse
import json
import os
import re
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (layer widths, global batch, weight init, description)
    "c1": ([1024] * 6, 1024, ("uniform", 1.0 / 32), "5 x 1024^2, batch 1024"),
    "c3": ([512] * 21, 2048, ("uniform", 512 ** -0.5), "20 x 512^2, batch 2048"),
    "c4": ([4096] * 9, 8192, ("uniform", 1.0 / 64), "8 x 4096^2, batch 8192"),
    # bf16 operands and bf16 weight gradients, fp32 master weights (implies --grad-bf16)
    "c5": ([8192] * 17, 16384, ("normal", 8192 ** -0.5), "16 x 8192^2, batch 16384, bf16 gradients"),
}


def gradient_buckets(layer_bytes, world, bucket_mb, sharded=False):
    """Bytes of each gradient collective of one step, in issue order, from the library's own
    rule (csrc/bucket_plan.h through the host library)."""
    import ctypes as C
    from tbb_test_b200 import build as B
    H = C.CDLL(B.HOST_LIB)
    n = len(layer_bytes)
    low, high = (C.c_int * n)(), (C.c_int * n)()
    growth = float(os.environ.get("B2_BUCKET_GROWTH", 0.0))
    if sharded:
        H.b2h_plan_buckets_sharded((C.c_size_t * n)(*layer_bytes), n, world, bucket_mb, C.c_double(growth), low, high)
    else:
        H.b2h_plan_buckets((C.c_size_t * n)(*layer_bytes), n, world, 1, bucket_mb, C.c_double(growth), low, high)
    out, l = [], n - 1
    while l >= 0:
        out.append(sum(layer_bytes[low[l]:high[l] + 1]))
        l = low[l] - 1
    return out


def draw_weights(rng, winit, shape):
    """Seeded weights of one layer: U(-a, a) or N(0, a^2)."""
    import numpy as np
    kind, a = winit
    if kind == "normal":
        return (rng.standard_normal(shape, dtype=np.float32) * np.float32(a)).astype(np.float32)
    return rng.uniform(-a, a, shape).astype(np.float32)


def env_int(name, default):
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def has_avx512():
    try:
        with open("/proc/cpuinfo") as f:
            return "avx512f" in f.read()
    except Exception:
        return False


def pick_sockets_threads(cores):
    """(sockets, threads/socket) for mlp_omp: the reference's self-check only passes for
    1, 2 or 8 sockets with several threads each, and its thread table stops at 28
    (mlp_bench_common.h:40-48). Choose the pair with the most GEMM threads."""
    comm = lambda t: 0 if t < 5 else 1 if t < 10 else 2 if t < 20 else 4
    best = (1, max(1, min(cores, 28)))
    best_score = best[1] - comm(best[1])
    for s in (2, 8):
        t = min(cores // s, 28)
        if t >= 5:
            score = s * (t - comm(t))
            if score > best_score:
                best, best_score = (s, t), score
    return best


REF_ITERS = {"c1": (3, 20), "c3": (3, 20), "c4": (1, 4)}  # most (warm-up, timed) steps a CPU sample may take


def run_reference_cpu(workload, batch, warmup=None, steps=None):
    """Times oracle/_ref/mlp_omp_<workload> on the host cores. Returns a dict or None."""
    exe = os.path.join(ROOT, "oracle", "_ref", f"mlp_omp_{workload}")
    if not os.path.exists(exe) or not has_avx512():
        return None
    cores = host_cores()
    s, t = pick_sockets_threads(cores)
    cap_w, cap_k = REF_ITERS.get(workload, (1, 2))
    nwarm = max(1, min(cap_w, warmup if warmup is not None else cap_w))
    niter = max(1, min(cap_k, steps if steps is not None else cap_k))
    env = dict(os.environ, OMP_PROC_BIND="close", OMP_PLACES="cores", OPENBLAS_NUM_THREADS="1",
               OMP_NUM_THREADS=str(s * t), B2_REF_NWARMUP=str(nwarm), B2_REF_NITER=str(niter))
    t0 = time.time()
    try:
        r = subprocess.run([exe, str(s), str(t)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                           text=True, timeout=900)
    except subprocess.TimeoutExpired:
        return None
    m = re.search(r"wall clock time ([0-9.eE+-]+) ms/iter", r.stdout)
    if r.returncode != 0 or not m:
        return None
    ms = float(m.group(1))
    return {"value": batch / (ms / 1e3), "ms_per_step": ms, "cores": s * t, "sockets": s, "kind": "reference",
            "unit": "samples/s", "wall_s": round(time.time() - t0, 1), "steps": niter, "warmup": nwarm,
            "sample": f"unmodified mlp_omp built with this workload's widths/batch, {s} socket(s) x {t} threads, "
                      f"OpenBLAS sgemm, {nwarm} warm-up + {niter} timed steps of the full workload"}


def run_port_cpu(nf, batch, steps=1):
    """Fallback CPU baseline: the oracle port with OpenBLAS on all cores (bounded sample)."""
    from oracle import oracle as O
    import numpy as np
    cores = host_cores()
    O.use_openblas(threads=cores)
    rows = min(batch, 1024)  # bounded sample: a 1024-row slice of the batch
    orc = O.Oracle(nf, rows, mode=O.MODE_REF, lr=1e-10)
    rng = np.random.default_rng(0)
    for l in range(len(nf) - 1):
        orc.set_weights(l, rng.uniform(-0.01, 0.01, (nf[l + 1], nf[l])).astype(np.float32))
    orc.set_input(rng.standard_normal((rows, nf[0]), dtype=np.float32))
    orc.step(1)
    t0 = time.time()
    orc.step(steps)
    dt = (time.time() - t0) / steps
    O.use_builtin_gemm()
    return {"value": rows / dt, "ms_per_step": dt * 1e3, "cores": cores, "kind": "port", "unit": "samples/s",
            "steps": steps, "warmup": 1,
            "sample": f"oracle port (OpenBLAS, {cores} threads) on a {rows}-row slice of the batch, {steps} step(s)"}


class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.p = None
        self.idx = gpu_index
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                       "-lms", "100", "-i", str(gpu_index)], stdout=subprocess.PIPE,
                                      stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.p = None

    def stop(self):
        if not self.p:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        try:
            out, _ = self.p.communicate(timeout=5)
        except Exception:
            self.p.kill()
            out = ""
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        hi = [v for v in sm if v >= 0.5 * max(sm)]  # samples under load
        return {"sm_mhz": statistics.median(hi), "sm_max_mhz": max(smax), "reasons": sorted(reasons),
                "samples": len(sm)}


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return p, "measured"
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def profiled_traffic(precision, rows, nf):
    """DRAM bytes (read + write) per GEMM launch from the ncu summary kept for this shape under
    profiles/ (a line `dram_bytes_per_launch: fwd=.. wgrad=.. dgrad=..`), mean over the three
    forms, or None when the shape was not profiled."""
    if not all(f == nf[0] for f in nf):
        return None, "no ncu capture for this shape"
    name = f"gemm_tc_kernel_{rows}x{nf[0]}x{nf[0]}_{precision}_ncu.md"
    path = os.path.join(ROOT, "profiles", name)
    try:
        with open(path) as f:
            m = re.search(r"dram_bytes_per_launch:\s*fwd=([0-9.eE+]+)\s+wgrad=([0-9.eE+]+)\s+dgrad=([0-9.eE+]+)", f.read())
    except OSError:
        m = None
    if not m:
        return None, "no ncu capture for this shape"
    vals = [float(v) for v in m.groups()]
    alg = (2 * rows * nf[0] + nf[0] * nf[0]) * (2 if precision == "bf16" else 4)
    return sum(vals) / 3, (f"mean of fwd/wgrad/dgrad DRAM read+write bytes per launch from profiles/{name}; "
                           f"operands + result of one launch: about {alg:.3g} bytes")


def allreduce_sweep(args, rank, world, local_rank):
    """Configuration 2: fp32 buffers of 4 KB .. 1 GB (powers of two), U(-1,1) from seed = rank,
    summed over all GPUs with the library's gradient allreduce; bus bandwidth
    bytes * 2(G-1)/G / t per size (the reference counts the same bytes per socket for its
    reduce-scatter + allgather, mlp_omp.cc:163,288). The CPU side is the reference's own ring
    (update_weight) on host threads acting as sockets, on a bounded set of sizes."""
    sizes = [1 << p for p in range(12, 31)]
    if args.impl == "reference" or world < 2:
        if rank != 0:
            return 0
        from oracle import oracle as O
        cores = host_cores()
        socks = 8 if cores >= 8 else 2
        table = []
        try:
            R = O.RefLib()
            for nbytes in (1 << 12, 1 << 16, 1 << 20, 1 << 24, 1 << 26):
                ncols = 1008  # ld = 1024 floats
                nrows = max(1, nbytes // 4 // ncols)
                iters = 20 if nbytes <= (1 << 20) else 3
                t = R.time_update_weight(socks, 1, nrows, ncols, iters)
                real = nrows * ncols * 4
                table.append({"bytes": real, "ms": t * 1e3, "busbw_gbs": real * 2 * (socks - 1) / socks / t / 1e9})
            kind = "reference"
        except Exception as e:  # no prebuilt reference on this machine
            table, kind = [{"error": str(e)}], "unavailable"
        best = max((r.get("busbw_gbs", 0.0) for r in table), default=0.0)
        # the TwistedHyperCube addressing as a data path (recursive halving + doubling between host
        # threads; the reference declares the interface only): this repository's host code
        cube = []
        try:
            import ctypes as C
            from tbb_test_b200 import build as B
            H = C.CDLL(B.HOST_LIB)
            H.b2h_time_hypercube_allreduce.restype = C.c_double
            H.b2h_time_hypercube_allreduce.argtypes = [C.c_int, C.c_int, C.c_int, C.c_size_t, C.c_int]
            for nbytes in (1 << 12, 1 << 16, 1 << 20, 1 << 24, 1 << 26):
                t = H.b2h_time_hypercube_allreduce(1 if socks == 8 else 0, socks, 0, nbytes // 4,
                                                   50 if nbytes <= (1 << 20) else 3)
                cube.append({"bytes": nbytes, "ms": t * 1e3,
                             "busbw_gbs": nbytes * 2 * (socks - 1) / socks / t / 1e9 if t > 0 else None})
        except (OSError, AttributeError) as e:
            cube = [{"error": str(e)}]
        cpu = {"value": best, "unit": "GB/s", "cores": socks, "kind": kind,
               "sample": f"reference update_weight (ring reduce-scatter + SGD + allgather), {socks} sockets x 1 "
                         "thread on the host cores, sizes 4 KB .. 64 MB", "table": table,
               "twisted_hypercube_host_path": cube}
        line = {"impl": "reference", "metric": "allreduce_busbw", "value": best, "unit": "GB/s", "n_gpus": 0,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": None, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": "c2: gradient allreduce sweep, fp32"}, "cpu_baseline": cpu,
                "e2e": {"value": best, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        if args.impl != "reference":
            line.pop("impl")
            line["note"] = "the sweep needs 2 or more GPUs; only the CPU side was run"
        print(json.dumps(line))
        return 0

    import torch
    import torch.distributed as dist
    from tbb_test_b200 import _capi as K
    from tbb_test_b200.mlp import MLP, nccl_unique_id
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    box = [nccl_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    dev = MLP([16, 16], 16 * world, rank=rank, world_size=world, device=local_rank, nccl_id=box[0])
    table = []
    for nbytes in sizes:
        iters = max(5, min(args.steps, 200 if nbytes <= (1 << 22) else 20))
        torch.cuda.synchronize()
        dist.barrier()
        ms, _ = dev.allreduce_bench(nbytes // 4, K.DTYPE_F32, max(args.warmup, 3), iters)
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        table.append({"bytes": nbytes, "ms": ms, "busbw_gbs": nbytes * 2 * (world - 1) / world / (ms / 1e3) / 1e9})
    launches = dev.launch_counts()[0]
    dev.close()
    if rank == 0:
        top = table[-1]
        line = {"metric": "allreduce_busbw", "value": top["busbw_gbs"], "unit": "GB/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": top["ms"],
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": {"workload": f"c2: gradient allreduce sweep, fp32, {world} GPUs, "
                                                "value = bus bandwidth at 1 GiB", "table": table},
                "roofline": {"bound": "nvlink", "achieved": top["busbw_gbs"], "peak": 770.0, "unit": "GB/s",
                             "frac": top["busbw_gbs"] / 770.0, "traffic": None,
                             "peak_source": "measured peer copy per direction on this pool (900 nominal)"},
                "cpu_baseline": None, "e2e": None, "gpu_launches": launches * world}
        print(json.dumps(line))
    dist.barrier()
    dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c4", choices=sorted(WORKLOADS) + ["c2"],
                    help="c2 = the gradient-allreduce sweep alone (needs 2 or more GPUs)")
    ap.add_argument("--precision", default="bf16", choices=["bf16", "tf32", "fp32", "fp32tc"],
                    help="fp32tc = fp32-class results on the tensor cores (three tf32 MMAs on split operands)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--comm-sms", type=int, default=-1,
                    help="SMs the GEMM kernels leave to the collective (-1 = library default)")
    ap.add_argument("--bucket-mb", type=int, default=-1,
                    help="gradient allreduce granularity in MiB (0 = per layer, -1 = library default)")
    ap.add_argument("--grad-bf16", action="store_true", help="bf16 weight gradients (configuration 5 style)")
    ap.add_argument("--shard-update", type=int, default=-1,
                    help="1 = reduce-scatter + SGD on the owned slice + allgather of the weights (default on 2 or "
                         "more GPUs), 0 = allreduce + SGD on every rank")
    ap.add_argument("--p2p-bytes", type=int, default=0,
                    help="gradient sums up to this many bytes go through peer memory instead of NCCL (0 = off)")
    ap.add_argument("--trace", default=None,
                    help="write rank 0's Chrome trace (per-kernel intervals of the timed steps) to this file")
    ap.add_argument("--graph", action="store_true",
                    help="replay each step as one CUDA graph (latency-bound workloads c1/c3); per-phase "
                         "events are not available then and the roofline line uses the whole step time")
    args = ap.parse_args()
    if args.graph and args.gpus > 1:
        ap.error("--graph is for single-GPU runs: the library refuses graph replay together with the allreduce")

    rank, world = env_int("RANK", 0), env_int("WORLD_SIZE", 1)
    local_rank = env_int("LOCAL_RANK", 0)
    if args.workload == "c2":
        return allreduce_sweep(args, rank, world, local_rank)
    nf, batch, winit, desc = WORKLOADS[args.workload]
    if args.workload == "c5":
        if args.precision != "bf16":
            ap.error("workload c5 is defined for bf16 operands")
        args.grad_bf16 = True
    warmup = max(args.warmup, 3)
    L = len(nf) - 1
    cfg_common = {"workload": f"{args.workload}: MLP {desc}, ReLU, +-1 targets, SGD lr 0.01; "
                              f"global batch split over {world} GPU(s)",
                  "global_batch": batch, "layers": L, "width": nf[0],
                  "parallelism": f"dp{world}", "l2": "working set per step exceeds the 126 MB L2 "
                  "(weights + activations of all layers are re-read every step)"}

    if args.impl == "reference":
        if rank != 0:
            return 0
        ref = run_reference_cpu(args.workload, batch, warmup=args.warmup, steps=args.steps)
        if ref is None:
            ref = run_port_cpu(nf, batch)
        # steps / warmup: what was really timed (a bounded sample of the requested run)
        line = {"impl": "reference", "metric": "mlp_train_samples_per_sec", "value": ref["value"],
                "unit": "samples/s", "n_gpus": 0, "steps": ref["steps"], "warmup": ref["warmup"],
                "requested": {"steps": args.steps, "warmup": args.warmup},
                "ms_per_step": ref["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg_common,
                "cpu_baseline": {k: ref[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": ref["value"], "unit": "samples/s", "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return 0

    import numpy as np
    import torch
    from tbb_test_b200 import _capi as K
    from tbb_test_b200.mlp import MLP, nccl_unique_id, pinned_array

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def fresh_id():
        """An NCCL id founds one communicator: every handle of the job gets its own."""
        if dist is None:
            return None
        box = [nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        return box[0]

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce_over_ranks(v, op):
        if dist is None:
            return v
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=op)
        return float(t.item())

    max_over_ranks = lambda v: reduce_over_ranks(v, dist.ReduceOp.MAX if dist else None)
    sum_over_ranks = lambda v: reduce_over_ranks(v, dist.ReduceOp.SUM if dist else None)

    def fail_all(what):
        """Every rank learns of a failed check; the job ends with a non-zero exit code."""
        if rank == 0:
            print(json.dumps({"metric": "mlp_train_samples_per_sec", "value": None, "n_gpus": world,
                              "error": what}))
        sys.exit(3)

    prec = {"bf16": K.PREC_BF16, "tf32": K.PREC_TF32, "fp32": K.PREC_FP32, "fp32tc": K.PREC_FP32_TC}[args.precision]

    # ---- the reference's start-up self-check (mlp_omp.cc:325-373, 413-416) on every rank ---------
    # grad(s*R + i, j) = s + i + j, w = i*j, alpha = 1  ->  w = i*j - ((i + j)*N + N(N-1)/2), exact in fp32
    kat_rows, kat_cols = 256, 512
    ii, jj = np.meshgrid(np.arange(kat_rows), np.arange(kat_cols), indexing="ij")
    kat = MLP([kat_cols, kat_rows], 8 * world, rank=rank, world_size=world, device=local_rank, lr=1.0,
              nccl_id=fresh_id(), precision=prec, shard_update=args.shard_update)
    kat.upload_weights(0, (ii * jj).astype(np.float32))
    kat.upload_weight_grad(0, (rank + ii + jj).astype(np.float32))
    kat.update_weight(0)
    kat_ok = bool(np.array_equal(kat.weights(0),
                                 (ii * jj - ((ii + jj) * world + world * (world - 1) // 2)).astype(np.float32)))
    kat.close()
    if sum_over_ranks(0.0 if kat_ok else 1.0) > 0:
        fail_all("allreduce + SGD known-answer test failed")

    def make(**kw):
        opts = dict(rank=rank, world_size=world, device=local_rank, mode=K.MODE_BASELINE, precision=prec, lr=0.01,
                    comm_sms=args.comm_sms, grad_bf16=args.grad_bf16, ar_bucket_mb=args.bucket_mb,
                    shard_update=args.shard_update)
        opts.update(kw)
        if opts.get("allreduce", True):
            opts["nccl_id"] = fresh_id()
        m = MLP(nf, batch, **opts)
        rng_w = np.random.default_rng(0)  # every rank draws the same weights
        for l in range(L):
            m.upload_weights(l, draw_weights(rng_w, winit, (nf[l + 1], nf[l])))
        return m

    dev = make(use_graph=args.graph)
    b0, b1 = dev.rows
    if args.p2p_bytes > 0 and world > 1:
        descs = [None] * world
        dist.all_gather_object(descs, dev.p2p_describe())
        dev.p2p_connect(descs, args.p2p_bytes)
        dist.barrier()

    # seeded synthetic data (weights seed 0, inputs seed 1, targets seed 2), drawn in blocks of 256
    # rows from generators keyed by the block number: the global batch is the same whatever the
    # number of ranks, and a rank only draws its own rows
    # pinned, and on the NUMA node of this rank's GPU (the reference binds each socket's matrices to
    # its node, mlp_omp.cc:27-47)
    numa_nodes = []
    x_host = pinned_array((batch, nf[0]), device=local_rank, node_out=numa_nodes)
    t_host = pinned_array((batch, nf[-1]), device=local_rank, node_out=numa_nodes)
    for blk in range(b0 // 256, (b1 + 255) // 256):
        r0, r1 = blk * 256, min(batch, blk * 256 + 256)
        xb = np.random.default_rng([1, blk]).standard_normal((r1 - r0, nf[0]), dtype=np.float32)
        tb = np.where(np.random.default_rng([2, blk]).random((r1 - r0, nf[-1])) < 0.5, -1.0, 1.0).astype(np.float32)
        lo, hi = max(r0, b0), min(r1, b1)
        x_host[lo:hi] = xb[lo - r0:hi - r0]
        t_host[lo:hi] = tb[lo - r0:hi - r0]
    dev.upload_input(x_host)
    dev.upload_target(t_host)

    # ---- device-resident timing (no per-phase events in these steps) ----------------------------
    sampler = ClockSampler(local_rank) if rank == 0 else None  # started early: nvidia-smi needs a moment
    dev.step(warmup)
    dev.reset_timing()
    l0, tc0 = dev.launch_counts()
    barrier()
    dev.step(args.steps)
    barrier()
    clocks = sampler.stop() if sampler else None  # idle samples are dropped, see ClockSampler.stop
    _, step_ms, nsteps = dev.timing()
    l1, tc1 = dev.launch_counts()
    ms_per_step = max_over_ranks(step_ms / max(nsteps, 1))
    value = batch / (ms_per_step / 1e3)
    launches = int(sum_over_ranks(l1 - l0))
    loss = sum_over_ranks(dev.loss())

    # ---- the replicas still hold the same weights (what the reference checks by eye on its
    # print_checksum lines): fingerprints of every layer, equal on all ranks
    fps = [dev.weights_fingerprint(l) for l in range(L)]
    replicas_identical = True
    if dist is not None:
        box = [None] * world
        dist.all_gather_object(box, fps)
        replicas_identical = all(b == box[0] for b in box)
        if not replicas_identical:
            fail_all("the ranks' weights differ after the timed steps")
    if not np.isfinite(loss):
        fail_all("the loss is not finite")

    # ---- per-phase breakdown: a second, short run of the same handle with an event pair around
    # every kernel (it costs ~150 extra runtime calls per step, hence not in the timed steps above)
    bl = b1 - b0
    peaks, peak_kind = measured_peaks()
    phase_steps = max(3, min(args.steps, 10))
    per_phase, gemm_ms, achieved_tf = {}, 0.0, 0.0
    gemm_flops_step = sum(3 * 2.0 * bl * nf[l] * nf[l + 1] for l in range(L))
    if not args.graph:
        dev.set_timing(True)
        dev.reset_timing()
        barrier()
        dev.step(phase_steps)
        if args.trace and rank == 0:
            dev.write_trace(args.trace)
        barrier()
        phase_ms, timed_ms, n_ph = dev.timing()
        gemm_ms = dev.gemm_busy_ms()
        per_phase = {n: float(phase_ms[:, i].sum() / max(n_ph, 1)) for n, i in
                     (("fwd_ms", K.T_FWD), ("wgrad_ms", K.T_WGT_GRAD), ("dgrad_ms", K.T_BWD),
                      ("sgd_ms", K.T_WGT_UPDATE), ("allreduce_ms", K.T_ALLREDUCE), ("allgather_ms", K.T_ALLGATHER))}
        per_phase["step_ms_with_events"] = timed_ms / max(n_ph, 1)
        achieved_tf = gemm_flops_step * n_ph / (gemm_ms / 1e3) / 1e12 if gemm_ms > 0 else 0.0
        dev.set_timing(False)
    whole_step_tf = gemm_flops_step / (ms_per_step / 1e3) / 1e12  # every flop of the step / the whole step
    if args.graph:
        achieved_tf = whole_step_tf
    peak_burst = peaks.get("bf16_tflops", 1590.0)
    peak_sust = peaks.get("bf16_tflops_sustained", 1400.0)
    n_params = sum(nf[l] * nf[l + 1] for l in range(L))
    traffic, traffic_note = profiled_traffic(args.precision, bl, nf)
    roofline = {"bound": "tensor",
                "kernel": "gemm_tc_kernel (fwd + wgrad + dgrad launches; flops / time with a GEMM running, "
                          f"{phase_steps}-step run with per-phase events)",
                "achieved": achieved_tf, "peak": peak_burst, "unit": "TFLOP/s",
                "frac": achieved_tf / peak_burst if peak_burst else None,
                "frac_of_sustained_peak": achieved_tf / peak_sust if peak_sust else None,
                "whole_step_tflops": whole_step_tf, "whole_step_frac": whole_step_tf / peak_burst if peak_burst else None,
                "traffic": traffic, "traffic_note": traffic_note,
                "peak_source": f"{peak_kind}: cuBLAS bf16 burst (best of 10; the timed region lasts "
                               f"{ms_per_step * args.steps / 1e3:.2f} s); sustained figure {peak_sust}",
                "per_step_ms": per_phase}
    # the SGD kernel alone on cold data (one layer's parameters; rotating sets larger than the L2)
    big = max(nf[l] * nf[l + 1] for l in range(L))
    sgd_ms, sgd_bytes = dev.sgd_bench(big, K.DTYPE_BF16 if args.grad_bf16 else K.DTYPE_F32,
                                      with_bf16_copy=(args.precision == "bf16"))
    sgd_gbs = sgd_bytes / (sgd_ms / 1e3) / 1e9
    roofline["sgd"] = {"bound": "hbm", "isolated": {"achieved": sgd_gbs, "peak": peaks.get("hbm_gbs"), "unit": "GB/s",
                                                    "frac": sgd_gbs / peaks["hbm_gbs"] if peaks.get("hbm_gbs") else None,
                                                    "bytes_per_launch": sgd_bytes, "ms_per_launch": sgd_ms,
                                                    "note": "sgd_kernel alone, CUDA events, operands not in L2"},
                       "in_step_ms": per_phase.get("sgd_ms"),
                       "note": "in the step it runs on the update stream next to the GEMMs"}

    if world > 1 and not args.graph:
        # The collectives alone (same sizes as the step's buckets), the step without any collective
        # (the reference's NO_ALL_REDUCE build, mlp_omp.cc:21), and from the three:
        # hidden fraction = 1 - (t_step - t_step,no collectives) / t_collectives,alone
        es = 2 if args.grad_bf16 else 4
        ws = 2 if args.precision == "bf16" else 4  # bytes per weight the allgather carries
        shard = args.shard_update != 0
        buckets = gradient_buckets([nf[l] * nf[l + 1] * es for l in range(L)], world, args.bucket_mb, sharded=shard)
        t_alone, wire = 0.0, 0.0
        for b in buckets:
            cnt = (b // es + 128 * world - 1) // (128 * world) * (128 * world)
            barrier()
            if shard:
                t_alone += max_over_ranks(dev.collective_bench(1, cnt, K.DTYPE_BF16 if args.grad_bf16 else K.DTYPE_F32))
                barrier()
                t_alone += max_over_ranks(dev.collective_bench(2, cnt, K.DTYPE_BF16 if ws == 2 else K.DTYPE_F32))
                wire += cnt * (es + ws) * (world - 1) / world
            else:
                t_alone += max_over_ranks(dev.collective_bench(0, cnt, K.DTYPE_BF16 if args.grad_bf16 else K.DTYPE_F32))
                wire += cnt * es * 2 * (world - 1) / world
        noar = make(allreduce=False)
        noar.upload_input(x_host)
        noar.upload_target(t_host)
        noar.step(warmup)
        noar.reset_timing()
        barrier()
        noar.step(args.steps)
        barrier()
        _, ms_noar, n_noar = noar.timing()
        noar.close()
        t_noar = max_over_ranks(ms_noar / max(n_noar, 1))
        in_step = per_phase.get("allreduce_ms", 0.0) + per_phase.get("allgather_ms", 0.0)
        nvlink = 900.0
        roofline["allreduce"] = {
            "bound": "nvlink", "route": "reduce-scatter + owned-slice SGD + allgather" if shard else "allreduce",
            "wire_bytes_per_gpu_per_step": wire, "buckets_bytes": buckets,
            "alone_ms_per_step": t_alone, "busbw_alone_gbs": wire / (t_alone / 1e3) / 1e9 if t_alone > 0 else None,
            "in_step_ms": in_step, "busbw_in_step_gbs": wire / (in_step / 1e3) / 1e9 if in_step > 0 else None,
            "peak": nvlink, "unit": "GB/s", "frac_alone": wire / (t_alone / 1e3) / 1e9 / nvlink if t_alone > 0 else None,
            "peak_source": "nominal NVLink 5 bandwidth per direction per GPU",
            "step_ms_without_allreduce": t_noar,
            "hidden_fraction": 1.0 - (ms_per_step - t_noar) / t_alone if t_alone > 0 else None}

    # ---- end to end through the host-facing call --------------------------------
    # Every step: this step's inputs and targets are copied from pinned host memory
    # (copy stream, two input slots, so the copy of step i+1 overlaps the compute of
    # step i) and the step's loss is read back to the host.
    e2e = None
    if not args.no_e2e:
        dev.close()
        dev = make()
        xp = x_host.ctypes.data_as(K._fp)
        tp = t_host.ctypes.data_as(K._fp)

        def pipelined(n):
            last = None
            for i in range(n):
                dev.train_step_host_async(xp, nf[0], tp, nf[-1])
                if i >= 1:
                    last = dev.wait_loss()
            return dev.wait_loss() if n else last

        pipelined(3)
        barrier()
        t0 = time.perf_counter()
        e2e_loss = pipelined(args.steps)
        torch.cuda.synchronize()
        dt = max_over_ranks(time.perf_counter() - t0)
        # the host link alone: every rank copies its rows of the pinned input matrix, all ranks at once
        barrier()
        t1 = time.perf_counter()
        for _ in range(5):
            dev.upload_input(x_host)
        h2d_s = max_over_ranks((time.perf_counter() - t1) / 5)
        e2e = {"value": batch * args.steps / dt, "unit": "samples/s",
               "h2d_bytes_per_step": batch * (nf[0] + nf[-1]) * 4, "d2h_bytes_per_step": 8 * world,
               "ms_per_step": dt / args.steps * 1e3, "loss_share_rank0": e2e_loss,
               "h2d_alone_gbs_all_gpus": batch * nf[0] * 4 / h2d_s / 1e9,
               "h2d_alone_note": "input rows only, pinned memory, every rank copying at the same time "
                                 "(incl. the bf16 conversion kernel): the host link's share of a step is "
                                 "h2d_bytes_per_step / this rate",
               "host_numa_node_rank0": numa_nodes[0] if numa_nodes else None,
               "call": "b2_train_step_host_async + b2_wait_loss, fp32 host matrices in pinned memory"}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = run_reference_cpu(args.workload, batch) or run_port_cpu(nf, batch)
        cpu = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}

    dev.close()
    if rank == 0:
        line = {"metric": "mlp_train_samples_per_sec", "value": value, "unit": "samples/s", "n_gpus": world,
                "steps": args.steps, "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": args.precision, "data": "synthetic",
                "config": cfg_common, "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
                "gpu_launches": launches, "clocks": clocks, "loss": loss,
                "kat": "pass", "replicas_identical": replicas_identical,
                "weights_fingerprint": [f"{v:016x}" for v in fps[:4]],
                "gemm_tflops_per_gpu": achieved_tf}
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
