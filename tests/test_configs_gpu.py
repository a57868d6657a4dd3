"""GPU parity at the benchmark's own configurations, at their literal sizes.

  configuration 1   5 x 1024^2, batch 1024, W ~ U(-1/32, 1/32), 10 steps, lr 0.01
  configuration 3   20 x 512^2, batch 2048, W ~ U(-1/sqrt(512), 1/sqrt(512))
  configuration 4   8 x 4096^2, batch 8192, W ~ U(-1/64, 1/64), bf16 operands
  configuration 5   16 x 8192^2 over 8 GPUs = 2048 rows per GPU; a 2-layer slice of it with
                    bf16 weight gradients, W ~ N(0, 1/8192)
(Configuration 2, the allreduce sweep, needs two or more GPUs: tests/test_multigpu_gpu.py.)

Two kinds of checks, because at these sizes the configurations are sensitive to the ORDER of
fp32 additions: a ReLU mask that flips, or a bf16 store that rounds the other way, for one
element in a million already moves a weight gradient by 1e-4 .. 1e-3, and over several steps
the difference feeds itself (a flipped mask changes one weight row, which shifts that unit's
pre-activation for every sample, which flips more masks).  Two CPU oracle runs that differ
ONLY in the order of additions (every GEMM summed in four partial sums) are, after ONE step,
1e-6 (fp32, no flip) to 1.4e-4 (fp32, one flip) apart on configuration 1's gradients, 6e-3
with bf16 storage, and 5e-2 on the lowest layers of configuration 3 with bf16 storage.

  1. every GEMM of the step alone, at its literal shape, fed with the oracle's operands
     (test_literal_shape_gemms): nothing can flip, bounds 2e-5 (fp32), 5e-5 (bf16 operands,
     fp32 result), 2e-3 (tf32)
  2. whole steps against the oracle: a tensor passes if its relative Frobenius error is within
     the stated bound OR within FLOOR_FACTOR x the distance between the two oracle runs above
     (measured in the same test, on the same data); the 10 iterations of configuration 1 are
     run one at a time from the oracle's weights (so every iteration is checked from a state
     both sides share) and once freely, where the loss must agree and the state is reported.
"""
import numpy as np
import pytest

from helpers import check_errors, make_problem, problem_weights, rel_fro, run_step_pair, worst_errors

pytestmark = pytest.mark.gpu

# bounds without the noise floor: fp32 state 2e-5. Gradients of one step contain flipped ReLU
# masks: a pre-activation z is summed over K = 1024 terms to about sqrt(K) * 2^-24 |z| = 2e-6 |z|
# in either order, so of configuration 1's 4 M masked elements about 2 * 2e-6 * 0.7 * 4e6 = 10
# have the other sign in the other order, each worth about 3e-4 of a weight gradient.
FP32_STEP = dict(state=2e-5, total=1e-2, grad=1e-2)
# fp32-class tensor-core mode: 2e-5 per GEMM; over the layers of a step the truncating accumulation of the
# tensor core adds up as a bias (20 layers of configuration 3: 2.6e-5 on the output)
FP32TC_STEP = dict(state=1e-4, total=1e-2, grad=1e-2)
SAME_ROUNDING_STEP = dict(state=2e-3, total=2e-3, grad=2e-3)
FLOOR_FACTOR = 8.0


def _prec(name):
    from tbb_test_b200 import _capi as K
    return {"fp32": K.PREC_FP32, "fp32tc": K.PREC_FP32_TC, "tf32": K.PREC_TF32, "bf16": K.PREC_BF16}[name]


def _report(tag, out, floor=None):
    fmt = lambda v: f"{v[0]:.2e} ({v[1]}" + (f", oracle-to-oracle {v[2]:.1e})" if len(v) > 2 else ")")
    print(tag, {k: fmt(v) for k, v in worst_errors(out, floor).items()})


SHAPES = {
    # configuration: (batch rows on one GPU, width)
    "c1": (1024, 1024), "c3": (2048, 512), "c4": (8192, 4096), "c4_8gpu": (1024, 4096), "c5_8gpu": (2048, 8192),
}


@pytest.mark.parametrize("cfg", sorted(SHAPES))
@pytest.mark.parametrize("prec,tol", [("bf16", 5e-5), ("tf32", 2e-3), ("fp32", 2e-5), ("fp32tc", 2e-5)])
def test_literal_shape_gemms(native, oracle, cfg, prec, tol):
    """Forward (ReLU epilogue), weight-gradient and input-gradient (mask epilogue) GEMM of one
    layer at the configuration's literal shape, on the oracle's operands."""
    from tbb_test_b200 import _capi as K
    from tbb_test_b200.mlp import MLP
    b, f = SHAPES[cfg]
    if prec == "fp32" and b * f * f > 2048 * 1024 * 1024:
        pytest.skip("the CUDA-core fp32 kernel is the parity mode of the small configurations")
    rnd = oracle.round_bf16 if prec == "bf16" else (lambda v: v)
    a = rnd(oracle.fill_normal(b, f, 21))
    w = rnd(oracle.fill_uniform(f, f, 22, -f ** -0.5, f ** -0.5))
    dz = rnd(oracle.fill_normal(b, f, 23))
    dev = MLP([16, 16], 16)
    oracle.use_openblas()
    try:
        fwd = dev.sgemm_host(_prec(prec), False, True, a, w, epilogue=K.EPI_RELU)
        ref = np.maximum(oracle.sgemm(False, True, a, w), 0.0)
        if prec == "bf16":  # the fused ReLU output is stored as a bf16 activation
            assert rel_fro(fwd, oracle.round_bf16(ref)) <= 2e-3
            assert np.mean(fwd != oracle.round_bf16(ref)) <= 2e-2  # other way at a rounding boundary
        else:
            assert rel_fro(fwd, ref) <= tol
        wg = dev.sgemm_host(_prec(prec), True, False, dz, a)
        assert rel_fro(wg, oracle.sgemm(True, False, dz, a)) <= tol
        dg = dev.sgemm_host(_prec(prec), False, False, dz, w, epilogue=K.EPI_MASK, aux=a)
        ref = oracle.sgemm(False, False, dz, w) * (a > 0)
        if prec == "bf16":
            assert rel_fro(dg, oracle.round_bf16(ref)) <= 2e-3
        else:
            assert rel_fro(dg, ref) <= tol
        total, tc = dev.launch_counts()
        assert (tc >= 3) == (prec != "fp32")
        if prec == "fp32tc":  # same tolerance class as the CUDA-core fp32 kernel, per row as well
            row = np.linalg.norm(wg - oracle.sgemm(True, False, dz, a), axis=1)
            assert row.max() <= 1e-4 * np.linalg.norm(wg, axis=1).max()
    finally:
        oracle.use_builtin_gemm()
        dev.close()


@pytest.mark.parametrize("prec", ["fp32", "fp32tc", "bf16"])
def test_configuration_1_ten_iterations_from_shared_state(native, oracle, prec):
    """The 10 iterations of configuration 1, each started from the oracle's weights."""
    from tbb_test_b200 import _capi as K
    from tbb_test_b200.mlp import MLP
    nf, batch, L = [1024] * 6, 1024, 5
    ws, x, t = make_problem(oracle, nf, batch, wdist=("uniform", 1.0 / 32))
    rounding = oracle.ROUND_BF16 if prec == "bf16" else oracle.ROUND_NONE
    # this configuration's own distance between two summation orders, measured once (step 1)
    _, _, floor = run_step_pair(oracle, nf, batch, _prec(prec), K.MODE_BASELINE, 1, 0.01, rounding=rounding,
                                wdist=("uniform", 1.0 / 32), openblas=True, taps="weights", floor_ksplit=4)
    tol = {"fp32": FP32_STEP, "fp32tc": FP32TC_STEP}.get(prec, SAME_ROUNDING_STEP)
    oracle.use_openblas()
    try:
        dev = MLP(nf, batch, precision=_prec(prec), lr=0.01)
        orc = oracle.Oracle(nf, batch, mode=oracle.MODE_BASELINE, rounding=rounding, lr=0.01)
        for l in range(L):
            orc.set_weights(l, ws[l])
        dev.upload_input(x)
        dev.upload_target(t)
        orc.set_input(x)
        orc.set_target(t)
        worst = {}
        for it in range(10):
            before = [orc.weights(l) for l in range(L)]
            for l in range(L):
                dev.upload_weights(l, before[l])
            dev.step(1)
            orc.step(1)
            out = {"y": (dev.activation(L), orc.activation(L)),
                   "loss": (np.array([dev.loss()]), np.array([orc.loss()]))}
            for l in range(L):
                out[f"dw{l}"] = (dev.weight_grad(l), orc.weight_grad(l))
                out[f"dW_total{l}"] = (dev.weights(l) - before[l], orc.weights(l) - before[l])
            check_errors(out, tol, floor=floor, factor=FLOOR_FACTOR, weights=before)
            for k, v in worst_errors(out).items():
                worst[k] = max(worst.get(k, (0.0, "")), v)
        print(f"c1 {prec} 10 iterations from shared state", {k: f"{v[0]:.2e} ({v[1]})" for k, v in worst.items()},
              "oracle-to-oracle", {k: f"{floor[k]:.1e}" for k in ("y", "dw0", "dw4")})
        dev.close()
        orc.close()
    finally:
        oracle.use_builtin_gemm()


@pytest.mark.parametrize("prec", ["fp32", "fp32tc", "tf32", "bf16"])
def test_configuration_1_ten_steps_free_running(native, oracle, prec):
    """10 steps without re-synchronisation: the loss agrees; the state is compared with loose
    bounds because differences between any two implementations feed themselves here."""
    from tbb_test_b200 import _capi as K
    out, (total, tc) = run_step_pair(oracle, [1024] * 6, 1024, _prec(prec), K.MODE_BASELINE, 10, 0.01,
                                     wdist=("uniform", 1.0 / 32), openblas=True)
    _report(f"c1 {prec} free running vs fp32 oracle", out)
    loss_d, loss_o = out["loss"][0][0], out["loss"][1][0]
    assert abs(loss_d - loss_o) <= {"fp32": 1e-5, "fp32tc": 1e-4}.get(prec, 1e-3) * abs(loss_o)
    check_errors(out, dict(state=2e-2, total=2e-1, grad=3e-1))
    if prec != "fp32":
        assert tc >= 10 * 15, "the step did not run on the tensor-core kernels"


@pytest.mark.parametrize("prec", ["fp32", "fp32tc"])
def test_configuration_3_one_step_fp32(native, oracle, prec):
    from tbb_test_b200 import _capi as K
    out, _, floor = run_step_pair(oracle, [512] * 21, 2048, _prec(prec), K.MODE_BASELINE, 1, 0.01,
                                  wdist=("uniform", 512 ** -0.5), openblas=True, floor_ksplit=4)
    _report(f"c3 {prec}", out, floor)
    check_errors(out, FP32_STEP if prec == "fp32" else FP32TC_STEP, floor=floor, factor=FLOOR_FACTOR,
                 weights=problem_weights(oracle, [512] * 21, 2048, ("uniform", 512 ** -0.5)))


def test_configuration_3_three_steps_fp32_loss(native, oracle):
    from tbb_test_b200 import _capi as K
    out, _ = run_step_pair(oracle, [512] * 21, 2048, K.PREC_FP32, K.MODE_BASELINE, 3, 0.01,
                           wdist=("uniform", 512 ** -0.5), openblas=True, taps="weights")
    _report("c3 fp32 three steps", out)
    assert abs(out["loss"][0][0] - out["loss"][1][0]) <= 1e-5 * abs(out["loss"][1][0])
    check_errors(out, dict(state=1e-3, total=1e-1, grad=1e-1),
                 weights=problem_weights(oracle, [512] * 21, 2048, ("uniform", 512 ** -0.5)))


def test_configuration_3_one_step_bf16_same_rounding(native, oracle):
    from tbb_test_b200 import _capi as K
    out, (total, tc), floor = run_step_pair(oracle, [512] * 21, 2048, K.PREC_BF16, K.MODE_BASELINE, 1, 0.01,
                                            rounding=oracle.ROUND_BF16, wdist=("uniform", 512 ** -0.5),
                                            openblas=True, floor_ksplit=4)
    _report("c3 bf16 same rounding", out, floor)
    check_errors(out, SAME_ROUNDING_STEP, floor=floor, factor=FLOOR_FACTOR,
                 weights=problem_weights(oracle, [512] * 21, 2048, ("uniform", 512 ** -0.5)))
    assert tc >= 60


def test_configuration_4_one_step_bf16_same_rounding(native, oracle):
    """The shape and kernel variant the benchmark times (256-row tiles, 8192 x 4096 x 4096)."""
    from tbb_test_b200 import _capi as K
    out, (total, tc), floor = run_step_pair(oracle, [4096] * 9, 8192, K.PREC_BF16, K.MODE_BASELINE, 1, 0.01,
                                            rounding=oracle.ROUND_BF16, wdist=("uniform", 1.0 / 64),
                                            openblas=True, taps="weights", floor_ksplit=4)
    _report("c4 bf16 same rounding", out, floor)
    check_errors(out, SAME_ROUNDING_STEP, floor=floor, factor=FLOOR_FACTOR,
                 weights=problem_weights(oracle, [4096] * 9, 8192, ("uniform", 1.0 / 64)))
    assert tc >= 24


def test_configuration_5_slice_bf16_gradients(native, oracle):
    """Two 8192 x 8192 layers on one GPU's 2048 rows of configuration 5, bf16 weight gradients,
    fp32 master weights."""
    from tbb_test_b200 import _capi as K
    out, (total, tc), floor = run_step_pair(oracle, [8192] * 3, 2048, K.PREC_BF16, K.MODE_BASELINE, 1, 0.01,
                                            rounding=oracle.ROUND_BF16, wdist=("normal", 8192 ** -0.5),
                                            openblas=True, taps="weights", grad_bf16=True, floor_ksplit=4)
    _report("c5 slice", out, floor)
    for l in range(2):
        g = out[f"dw{l}"][0]
        assert np.array_equal(g, oracle.round_bf16(g)), "gradient buffer is not bf16-valued"
    check_errors(out, dict(state=2e-3, total=5e-3, grad=5e-3), floor=floor, factor=FLOOR_FACTOR)
    assert tc >= 6
