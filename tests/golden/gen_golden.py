"""Regenerates the golden fixtures of this directory from the UNMODIFIED reference.

Needs the reference sources (where oracle/build_ref.sh finds them) and oracle/_ref built by
oracle/build_ref.sh; run once, commit the outputs:

    python tests/golden/gen_golden.py

Outputs
  partition_topology.json  get_partition / get_intra_socket_2dpartition /
                           get_2dpartition (Partition.cc), HyperCube and
                           TwistedHyperCube peer/recv/send tables
                           (TwistedHyperCube.cc), get_my_ring_info
                           (mlp_bench_common.cc:170-190)
  ring_update.npz          update_weight (mlp_omp.cc:297-323) run by the reference
                           on seeded data for 1/2/4/8 sockets, one thread each
  ref_mode_run.npz         state of the reference's globals after its own
                           `mlp_omp 1 8` run (16+256 steps): sampled entries and
                           norms of the output, the propagated gradients, the
                           weight gradients and the final weights
The script also checks the CPU oracle against each of them and prints the
deviations (the same checks run in tests/test_oracle_pins.py).
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import oracle as O  # noqa: E402

SAMPLE = 512


def sample_idx(n, count=SAMPLE):
    """Deterministic spread of `count` flat indices over [0, n)."""
    if n <= count:
        return np.arange(n, dtype=np.int64)
    return (np.arange(count, dtype=np.int64) * 2654435761 + 12345) % n


def gen_partition_topology(R):
    out = {"get_partition": [], "intra_socket_2d": [], "partition_2d": [], "hypercube": [],
           "ring_info": []}
    for nsock in (1, 2, 3, 4, 8):
        for work in (1, 7, 1000, 1024, 2048, 8192, 16384):
            for nthr in (1, 3, 8):
                for sid in range(nsock):
                    for tid in range(nthr):
                        out["get_partition"].append(
                            [nsock, work, sid, nthr, tid] + R.get_partition(nsock, work, sid, nthr, tid))
    shapes = [(1024, 1024), (512, 512), (4096, 4096), (1024, 1), (100, 36), (2048, 8192), (17, 1000)]
    for (m, n) in shapes:
        for ar in (4.0, 0.5):
            for m_align in (0, 1):
                for nthr in (1, 4, 7, 8, 16, 24, 27):
                    for tid in sorted({0, 1 % nthr, nthr // 2, nthr - 1}):
                        out["intra_socket_2d"].append(
                            [m, n, ar, m_align, nthr, tid] + R.intra_socket_2d(m, n, ar, m_align, nthr, tid))
    for nsock in (1, 2, 4, 8):
        for (m, n) in ((1024 * nsock, 1024), (8192, 4096), (1000, 512)):
            for ar, m_align in ((4.0, 0), (0.5, 0)):
                for nthr in (7, 24):
                    for sid in sorted({0, nsock - 1}):
                        for tid in (0, nthr - 1):
                            out["partition_2d"].append(
                                [nsock, m, n, ar, m_align, sid, nthr, tid] +
                                R.partition_2d(nsock, m, n, ar, m_align, sid, nthr, tid))
    for twisted in (0, 1):
        for n in (2, 4, 8):
            dims = {2: 1, 4: 2, 8: 3}[n]
            for shift in range(dims):
                for dim in range(dims):
                    for node in range(n):
                        out["hypercube"].append([twisted, n, shift, node, dim] +
                                                R.hypercube(twisted, n, shift, node, dim))
    for nsock in (1, 2, 3, 4, 8):
        for sid in range(nsock):
            for task in (0, 1, 2, 3):
                out["ring_info"].append([nsock, sid, task] + R.ring_info(nsock, sid, task))
    with open(os.path.join(HERE, "partition_topology.json"), "w") as f:
        json.dump(out, f, separators=(",", ":"))
    print("partition_topology.json:", {k: len(v) for k, v in out.items()})


def ring_inputs(n, nrows=32, ncols=48):
    w0 = O.fill_uniform(nrows, ncols, 100 + n, -1.0, 1.0)
    w = np.repeat(w0[None], n, axis=0)
    g = np.stack([O.fill_uniform(nrows, ncols, 200 + 10 * n + s, -1.0, 1.0) for s in range(n)])
    return w, g


def gen_ring(R):
    out = {}
    for n in (1, 2, 4, 8):
        w, g = ring_inputs(n)
        ref = R.update_weight(w, g, 0.37, 1)
        mine = O.ring_update(w, g, 0.37)
        print(f"ring_update n={n}: oracle bit-exact vs reference: {np.array_equal(ref, mine)}")
        out[f"n{n}"] = ref
    np.savez_compressed(os.path.join(HERE, "ring_update.npz"), **out)


def ref_mode_initial_state(nf, batch):
    """Inputs and weights exactly as the reference's init_matrices() draws them from
    the stand-in stream (seed 3, consumed row by row: mlp_bench_common.cc:16-33)."""
    pos = 0
    x = O.fill_uniform(batch, nf[0], 3, 0.0, 1.0, start=pos)
    pos += batch * nf[0]
    ws = []
    for l in range(len(nf) - 1):
        ws.append(O.fill_uniform(nf[l + 1], nf[l], 3, -0.1, 0.1, start=pos))
        pos += nf[l + 1] * nf[l]
    return x, ws


def gen_ref_mode(R):
    nf = R.nfeatures()
    L = len(nf) - 1
    print("running the reference benchmark (mlp_omp 1 8): 272 steps ...", flush=True)
    R.run_main(1, 8)
    tensors = {"y": R.activation(L), "dinput": R.activation(L + 1)}
    for l in range(1, L):
        tensors[f"da{l}"] = R.activation(l)
    for l in range(L):
        tensors[f"dw{l}"] = R.weight_grad(l)
        tensors[f"w{l}"] = R.weights(l)
    batch = tensors["y"].shape[0]
    R.reinit()
    x0, w0 = ref_mode_initial_state(nf, batch)
    assert np.array_equal(x0, R.activation(0)), "stand-in stream reproduction (input) failed"
    for l in range(L):
        assert np.array_equal(w0[l], R.weights(l)), "stand-in stream reproduction (weights) failed"
    out = {"nfeatures": np.array(nf), "batch": np.array(batch), "steps": np.array(272),
           "lr": np.array(1e-10)}
    for k, t in tensors.items():
        flat = t.reshape(-1)
        idx = sample_idx(flat.size)
        out[k + "_idx"] = idx
        out[k + "_val"] = flat[idx]
        out[k + "_norm"] = np.array(np.sqrt(np.sum(flat.astype(np.float64) ** 2)))
        out[k + "_sum"] = np.array(np.sum(flat.astype(np.float64)))
    np.savez_compressed(os.path.join(HERE, "ref_mode_run.npz"), **out)

    # pin report: the oracle on the same initial state
    print("running the oracle in ref mode, 272 steps ...", flush=True)
    O.use_openblas(threads=os.cpu_count())
    o = O.Oracle(nf, batch, nranks=1, mode=O.MODE_REF, lr=1e-10)
    o.set_input(x0)
    for l in range(L):
        o.set_weights(l, w0[l])
    o.step(272)
    mine = {"y": o.activation(L), "dinput": o.input_grad()}
    for l in range(1, L):
        mine[f"da{l}"] = o.dz(l - 1)
    for l in range(L):
        mine[f"dw{l}"] = o.weight_grad(l)
        mine[f"w{l}"] = o.weights(l)
    for k in sorted(tensors):
        a, b = mine[k].astype(np.float64), tensors[k].astype(np.float64)
        rel = np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300)
        print(f"  {k:8s} rel_fro {rel:.3e}")
    O.use_builtin_gemm()


if __name__ == "__main__":
    R = O.RefLib()
    gen_partition_topology(R)
    gen_ring(R)
    gen_ref_mode(R)
