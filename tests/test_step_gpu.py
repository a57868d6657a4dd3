"""GPU parity of the whole training step against the CPU oracle, through the C ABI.

Tolerances (relative Frobenius error per tensor, after 10 SGD steps with lr 0.01
on seeded inputs, compared on activations, propagated gradients, weight gradients
of the last step and the weight change W10 - W0):
  fp32  2e-5  against the fp32 oracle (only the order of fp32 additions differs)
  tf32  4e-3  against the fp32 oracle (10-bit operand mantissas)
  bf16  3e-2  against the fp32 oracle and against the oracle that rounds operands
              to bf16 at the same points (8-bit operand mantissas; reduction order
              and single-ulp rounding flips compound over the steps)
"""
import numpy as np
import pytest

from helpers import make_problem, rel_fro

pytestmark = pytest.mark.gpu

TOL = {"fp32": 2e-5, "tf32": 4e-3, "bf16": 3e-2}


def _prec(name):
    from tbb_test_b200 import _capi as K
    return {"fp32": K.PREC_FP32, "tf32": K.PREC_TF32, "bf16": K.PREC_BF16}[name]


def run_pair(O, nf, batch, prec, mode, steps, lr, rounding=None, **kw):
    from tbb_test_b200 import _capi as K
    from tbb_test_b200.mlp import MLP
    ws, x, t = make_problem(O, nf, batch)
    L = len(nf) - 1
    dev = MLP(nf, batch, mode=mode, precision=_prec(prec), lr=lr, **kw)
    orc = O.Oracle(nf, batch, nranks=1, mode=mode, lr=lr,
                   rounding=O.ROUND_NONE if rounding is None else rounding)
    for l in range(L):
        dev.upload_weights(l, ws[l])
        orc.set_weights(l, ws[l])
    dev.upload_input(x)
    orc.set_input(x)
    dev.upload_target(t)
    orc.set_target(t)
    dev.step(steps)
    orc.step(steps)
    out = {}
    out["y"] = (dev.activation(L), orc.activation(L))
    for l in range(1, L):
        out[f"act{l}"] = (dev.activation(l), orc.activation(l))
    for l in range(L):
        out[f"dz{l}"] = (dev.dz(l), orc.dz(l))
        out[f"dw{l}"] = (dev.weight_grad(l), orc.weight_grad(l))
        out[f"dW_total{l}"] = (dev.weights(l) - ws[l], orc.weights(l) - ws[l])
    out["dinput"] = (dev.input_grad(), orc.input_grad())
    out["loss"] = (np.array([dev.loss()]), np.array([orc.loss()]))
    counts = dev.launch_counts()
    dev.close()
    orc.close()
    return out, counts


@pytest.mark.parametrize("prec", ["fp32", "tf32", "bf16"])
def test_baseline_mode_10_steps(native, oracle, prec):
    """Config-1-shaped job scaled to 256 wide: ReLU MLP, +-1 targets, lr 0.01, 10 steps."""
    from tbb_test_b200 import _capi as K
    nf = [256] * 6
    out, (total, tc) = run_pair(oracle, nf, 256, prec, K.MODE_BASELINE, 10, 0.01)
    for name, (a, b) in out.items():
        assert rel_fro(a, b) <= TOL[prec], f"{name}: {rel_fro(a, b):.3e}"
    if prec != "fp32":
        assert tc >= 10 * 15, "the step did not run on the tensor-core kernels"


def test_bf16_against_rounding_oracle(native, oracle):
    from tbb_test_b200 import _capi as K
    nf = [256, 512, 256, 128]
    out, _ = run_pair(oracle, nf, 384, "bf16", K.MODE_BASELINE, 3, 0.01, rounding=oracle.ROUND_BF16)
    for name, (a, b) in out.items():
        assert rel_fro(a, b) <= TOL["bf16"], f"{name}: {rel_fro(a, b):.3e}"


@pytest.mark.parametrize("prec", ["fp32", "tf32"])
def test_ref_mode_matches_reference_semantics(native, oracle, prec):
    """REF mode = the C++ reference as written: no ReLU, the forward output fed back
    as the gradient, tiny lr (mlp_omp.cc:565,609,655)."""
    from tbb_test_b200 import _capi as K
    nf = [128, 256, 128, 64]
    out, _ = run_pair(oracle, nf, 200, prec, K.MODE_REF, 4, 1e-6)
    for name, (a, b) in out.items():
        assert rel_fro(a, b) <= TOL[prec], f"{name}: {rel_fro(a, b):.3e}"


def test_reference_topology_with_unit_tail(native, oracle):
    """The reference's own widths end in a 1-wide layer (mlp_bench_common.h:26)."""
    from tbb_test_b200 import _capi as K
    nf = [128, 128, 128, 1]
    for prec in ("fp32", "bf16"):
        out, _ = run_pair(oracle, nf, 96, prec, K.MODE_REF, 2, 1e-8,
                          rounding=oracle.ROUND_BF16 if prec == "bf16" else None)
        for name, (a, b) in out.items():
            assert rel_fro(a, b) <= TOL[prec], f"{prec} {name}: {rel_fro(a, b):.3e}"


@pytest.mark.parametrize("kw", [dict(overlap=False), dict(use_graph=True), dict(collect_timing=True),
                                dict(input_grad=False)], ids=lambda d: next(iter(d)))
def test_schedule_variants_agree(native, oracle, kw):
    """Serial schedule, CUDA-graph replay and timed mode give the same numbers as the
    overlapped two-stream schedule."""
    from tbb_test_b200 import _capi as K
    nf = [128, 256, 128]
    out, _ = run_pair(oracle, nf, 128, "fp32", K.MODE_BASELINE, 5, 0.01, **kw)
    for name, (a, b) in out.items():
        if name == "dinput" and kw.get("input_grad") is False:
            continue
        assert rel_fro(a, b) <= TOL["fp32"], f"{name}: {rel_fro(a, b):.3e}"


def test_allreduce_sgd_known_answer(native, oracle):
    """The reference's self-check (mlp_omp.cc:325-373) for one socket: grad = i + j,
    w = i*j, alpha = 1 -> w = i*j - (i + j), exact in fp32."""
    from tbb_test_b200 import _capi as K
    from tbb_test_b200.mlp import MLP
    nrows, ncols = 1024, 1024
    w, g, e = oracle.kat(1, nrows, ncols)
    dev = MLP([ncols, nrows], 8, lr=1.0)
    dev.upload_weights(0, w[0])
    dev.upload_weight_grad(0, g[0])
    dev.update_weight(0)
    got = dev.weights(0)
    dev.close()
    assert np.array_equal(got, e)
    assert np.abs(got - e).max() <= 1e-5  # the reference's own threshold


def test_sgd_bit_exact_against_ring_oracle(native, oracle):
    """w = fma(-lr, g, w) on random data equals the restated AVX-512 update bit for bit."""
    from tbb_test_b200.mlp import MLP
    nrows, ncols = 96, 80
    w = oracle.fill_uniform(nrows, ncols, 5, -1.0, 1.0)
    g = oracle.fill_uniform(nrows, ncols, 6, -1.0, 1.0)
    dev = MLP([ncols, nrows], 8, lr=0.37)
    dev.upload_weights(0, w)
    dev.upload_weight_grad(0, g)
    dev.update_weight(0)
    got = dev.weights(0)
    dev.close()
    ref = oracle.ring_update(w[None], g[None], 0.37)[0]
    assert np.array_equal(got, ref)


def test_golden_ref_mode_first_step(native, oracle):
    """One REF-mode step from the reference's own initial state reproduces, layer by
    layer, what the oracle (pinned to the reference binary) computes; 7 layers of
    1024 ending in the 1-wide tail, batch 1024."""
    import os
    from tbb_test_b200 import _capi as K
    from tbb_test_b200.mlp import MLP
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_mode_run.npz"))
    nf = [int(v) for v in gold["nfeatures"]]
    batch = int(gold["batch"])
    L = len(nf) - 1
    pos = 0
    x = oracle.fill_uniform(batch, nf[0], 3, 0.0, 1.0, start=pos)
    pos += batch * nf[0]
    ws = []
    for l in range(L):
        ws.append(oracle.fill_uniform(nf[l + 1], nf[l], 3, -0.1, 0.1, start=pos))
        pos += nf[l + 1] * nf[l]
    oracle.use_openblas()
    try:
        orc = oracle.Oracle(nf, batch, mode=oracle.MODE_REF, lr=1e-10)
        dev = MLP(nf, batch, mode=K.MODE_REF, precision=K.PREC_FP32, lr=1e-10)
        for l in range(L):
            orc.set_weights(l, ws[l])
            dev.upload_weights(l, ws[l])
        orc.set_input(x)
        dev.upload_input(x)
        orc.step(1)
        dev.step(1)
        assert rel_fro(dev.activation(L), orc.activation(L)) <= 2e-5
        for l in range(L):
            assert rel_fro(dev.weight_grad(l), orc.weight_grad(l)) <= 2e-5, l
        assert rel_fro(dev.input_grad(), orc.input_grad()) <= 2e-5
        dev.close()
        orc.close()
    finally:
        oracle.use_builtin_gemm()


def test_bad_arguments_are_reported_not_fatal(native):
    """Errors come back as status codes with a message (the reference asserts/exits)."""
    from tbb_test_b200 import _capi as K
    from tbb_test_b200.mlp import MLP
    with pytest.raises(K.B2Error) as e:
        MLP([16, 0, 16], 8)
    assert e.value.code == K.ERR_INVALID
    with pytest.raises(K.B2Error):
        MLP([16, 16], 8, rank=3, world_size=2)
    with pytest.raises(K.B2Error):
        MLP([16, 16], 8, grad_bf16=True, precision=K.PREC_FP32)
    import ctypes as C
    m = MLP([16, 16], 8)
    buf = (C.c_float * 256)()
    assert m.lib.b2_download_weights(m._h, 5, buf, 16) == K.ERR_INVALID
    assert b"out of range" in m.lib.b2_last_error(m._h)
    assert m.lib.b2_download_weights(m._h, 0, None, 16) == K.ERR_INVALID
    assert m.lib.b2_step(m._h, -1) == K.ERR_INVALID
    m.close()
