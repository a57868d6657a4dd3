"""The CPU oracle against the golden vectors generated from the unmodified
reference (tests/golden/gen_golden.py) and against the reference's own
known-answer test."""
import os

import numpy as np
import pytest

from helpers import rel_fro

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_gemm_forms_against_numpy(oracle):
    rs = np.random.RandomState(0)
    for (m, n, k) in [(17, 33, 29), (128, 64, 256)]:
        a = rs.randn(m, k).astype(np.float32)
        b = rs.randn(k, n).astype(np.float32)
        ref = a.astype(np.float64) @ b.astype(np.float64)
        assert rel_fro(oracle.sgemm(False, False, a, b), ref) < 1e-6
        assert rel_fro(oracle.sgemm(False, True, a, np.ascontiguousarray(b.T)), ref) < 1e-6
        assert rel_fro(oracle.sgemm(True, False, np.ascontiguousarray(a.T), b), ref) < 1e-6


def test_builtin_gemm_matches_openblas(oracle):
    if oracle.find_openblas() is None:
        pytest.skip("no OpenBLAS in this image")
    a = oracle.fill_uniform(96, 200, 1, -1.0, 1.0)
    b = oracle.fill_uniform(200, 72, 2, -1.0, 1.0)
    mine = oracle.sgemm(False, False, a, b)
    oracle.use_openblas(threads=2)
    try:
        blas = oracle.sgemm(False, False, a, b)
    finally:
        oracle.use_builtin_gemm()
    assert rel_fro(mine, blas) < 1e-6


def test_known_answer_allreduce_sgd(oracle):
    """mlp_omp.cc:325-373: exact for every socket count, on every replica."""
    for n in (1, 2, 3, 4, 8):
        w, g, e = oracle.kat(n, 32, 48)
        got = oracle.ring_update(w, g, 1.0)
        for s in range(n):
            assert np.array_equal(got[s], e), (n, s)


def test_ring_update_bit_exact_against_reference(oracle):
    import importlib.util
    spec = importlib.util.spec_from_file_location("gen_golden", os.path.join(GOLD, "gen_golden.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    gold = np.load(os.path.join(GOLD, "ring_update.npz"))
    for n in (1, 2, 4, 8):
        w, g = gen.ring_inputs(n)
        assert np.array_equal(oracle.ring_update(w, g, 0.37), gold[f"n{n}"]), n


def test_ref_mode_against_reference_binary_run(oracle):
    """272 REF-mode steps from the reference's initial state land on what the
    unmodified mlp_omp left in its globals (sampled entries + norms), within fp32
    GEMM-order noise."""
    if oracle.find_openblas() is None:
        pytest.skip("needs OpenBLAS to finish in seconds")
    import importlib.util
    spec = importlib.util.spec_from_file_location("gen_golden", os.path.join(GOLD, "gen_golden.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    gold = np.load(os.path.join(GOLD, "ref_mode_run.npz"))
    nf = [int(v) for v in gold["nfeatures"]]
    batch, steps = int(gold["batch"]), int(gold["steps"])
    L = len(nf) - 1
    x0, w0 = gen.ref_mode_initial_state(nf, batch)
    oracle.use_openblas(threads=os.cpu_count())
    try:
        o = oracle.Oracle(nf, batch, nranks=1, mode=oracle.MODE_REF, lr=float(gold["lr"]))
        o.set_input(x0)
        for l in range(L):
            o.set_weights(l, w0[l])
        o.step(steps)
        mine = {"y": o.activation(L), "dinput": o.input_grad()}
        for l in range(1, L):
            mine[f"da{l}"] = o.dz(l - 1)
        for l in range(L):
            mine[f"dw{l}"] = o.weight_grad(l)
            mine[f"w{l}"] = o.weights(l)
        o.close()
    finally:
        oracle.use_builtin_gemm()
    for k, t in mine.items():
        flat = t.reshape(-1)
        idx = gold[k + "_idx"]
        assert rel_fro(flat[idx], gold[k + "_val"]) <= 5e-5, k
        norm = np.sqrt(np.sum(flat.astype(np.float64) ** 2))
        assert abs(norm - float(gold[k + "_norm"])) <= 5e-5 * float(gold[k + "_norm"]), k


def test_rank_split_is_sum_of_shards(oracle):
    """Data parallelism is a split of the weight-gradient contraction over batch rows:
    the oracle with G ranks equals the single-rank oracle up to summation order, for
    even and ragged splits (Partition.cc:34-51 shards)."""
    from helpers import make_problem
    nf, batch = [48, 64, 32], 50
    ws, x, t = make_problem(oracle, nf, batch)
    res = []
    for g in (1, 2, 4, 8):
        o = oracle.Oracle(nf, batch, nranks=g, mode=oracle.MODE_BASELINE, lr=0.05)
        for l in range(2):
            o.set_weights(l, ws[l])
        o.set_input(x)
        o.set_target(t)
        o.step(3)
        res.append([o.weights(l) for l in range(2)] + [o.activation(2)])
        o.close()
    for r in res[1:]:
        for a, b in zip(r, res[0]):
            assert rel_fro(a, b) < 1e-5
    assert oracle.batch_range(50, 8, 7) == (49, 50)
    assert oracle.batch_range(1000, 4, 3) == (750, 1000)
    assert oracle.batch_range(3, 8, 5) == (3, 3)  # empty shard


def test_bf16_rounding_helper(oracle):
    import torch
    x = oracle.fill_normal(64, 64, 9, 3.0)
    ref = torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.array_equal(oracle.round_bf16(x), ref)


def test_checksum_matches_print_checksum_arithmetic(oracle):
    w = oracle.fill_uniform(40, 24, 3, -0.1, 0.1)
    l1, l2, tr = oracle.checksum(w)
    assert abs(l1 - np.abs(w.astype(np.float64)).sum()) < 1e-9 * max(1, l1)
    assert abs(l2 - np.sqrt((w.astype(np.float32) ** 2).astype(np.float64).sum())) < 1e-9
    assert abs(tr - np.trace(w[:24, :24].astype(np.float64))) < 1e-12
