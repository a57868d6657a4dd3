"""GPU parity of the three GEMM call forms (mlp_omp.cc:474,566,657) against the CPU
oracle, through the C ABI (b2_sgemm_host), for every precision and epilogue."""
import numpy as np
import pytest

from helpers import rel_fro

pytestmark = pytest.mark.gpu

FORMS = {"fwd_NT": (False, True), "dgrad_NN": (False, False), "wgrad_TN": (True, False)}
# (m, n, k): one tile / several tiles / ragged edges in every dimension / the 1024 layer
SHAPES = [(128, 256, 64), (256, 512, 256), (384, 320, 200), (104, 72, 136), (1024, 1024, 1024)]
# fp32: FMA order only; tf32: 10-bit operand mantissa, checked against the fp32 oracle;
# bf16: operands pre-rounded on both sides, so only accumulation order (fp32 output)
# or one final bf16 rounding (bf16 output) may differ.
TOL = {"fp32": 2e-5, "tf32": 2e-3, "bf16_f32out": 5e-5, "bf16_bf16out": 6e-3}


@pytest.fixture(scope="module")
def dev(native):
    from tbb_test_b200.mlp import MLP
    m = MLP([16, 16], 16)
    yield m
    m.close()


def operands(O, form, m, n, k, seed):
    ta, tb = FORMS[form]
    a = O.fill_uniform(k if ta else m, m if ta else k, seed, -1.0, 1.0)
    b = O.fill_uniform(n if tb else k, k if tb else n, seed + 1, -1.0, 1.0)
    return ta, tb, a, b


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("form", list(FORMS))
def test_fp32(dev, oracle, form, shape):
    from tbb_test_b200 import _capi as K
    m, n, k = shape
    ta, tb, a, b = operands(oracle, form, m, n, k, 11)
    c = dev.sgemm_host(K.PREC_FP32, ta, tb, a, b)
    ref = oracle.sgemm(ta, tb, a, b)
    assert rel_fro(c, ref) <= TOL["fp32"]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("form", list(FORMS))
def test_tf32_tensor_core(dev, oracle, form, shape):
    from tbb_test_b200 import _capi as K
    m, n, k = shape
    ta, tb, a, b = operands(oracle, form, m, n, k, 21)
    before = dev.launch_counts()[1]
    c = dev.sgemm_host(K.PREC_TF32, ta, tb, a, b)
    assert dev.launch_counts()[1] == before + 1, "tensor-core kernel was not used"
    ref = oracle.sgemm(ta, tb, a, b)
    assert rel_fro(c, ref) <= TOL["tf32"]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("form", list(FORMS))
def test_bf16_tensor_core(dev, oracle, form, shape):
    from tbb_test_b200 import _capi as K
    m, n, k = shape
    ta, tb, a, b = operands(oracle, form, m, n, k, 31)
    before = dev.launch_counts()[1]
    c = dev.sgemm_host(K.PREC_BF16, ta, tb, a, b)
    assert dev.launch_counts()[1] == before + 1, "tensor-core kernel was not used"
    ref = oracle.sgemm(ta, tb, oracle.round_bf16(a), oracle.round_bf16(b))
    assert rel_fro(c, ref) <= TOL["bf16_f32out"]


@pytest.mark.parametrize("shape", SHAPES + [(4096, 1024, 136), (2048, 512, 512)], ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("form", list(FORMS))
def test_fp32_class_tensor_core(dev, oracle, form, shape):
    """B2_PREC_FP32_TC: three tf32 MMAs per k-step on operands split into high and low parts;
    the fp32 bound of the CUDA-core kernel applies (and the plain tf32 kernel misses it by 30x)."""
    from tbb_test_b200 import _capi as K
    m, n, k = shape
    ta, tb, a, b = operands(oracle, form, m, n, k, 23)
    before = dev.launch_counts()[1]
    c = dev.sgemm_host(K.PREC_FP32_TC, ta, tb, a, b)
    assert dev.launch_counts()[1] == before + 1, "tensor-core kernel was not used"
    oracle.use_openblas()
    try:
        ref = oracle.sgemm(ta, tb, a, b)
    finally:
        oracle.use_builtin_gemm()
    assert rel_fro(c, ref) <= TOL["fp32"]
    row_err = np.linalg.norm(c - ref, axis=1) / np.maximum(np.linalg.norm(ref, axis=1), 1e-30)
    assert row_err.max() <= 1e-4


# Shapes wide enough for the 256-row tile mode (two accumulators per CTA sharing each
# B slab): an exact multiple of the tile grid, and a ragged one whose tile count leaves
# a partial last wave that is handed out as 128-row halves.
BIG_SHAPES = [(4096, 4096, 192), (7944, 4096, 136)]


@pytest.mark.parametrize("prec", ["bf16", "tf32"])
@pytest.mark.parametrize("shape", BIG_SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("form", list(FORMS))
def test_large_tile_mode(dev, oracle, form, shape, prec):
    from tbb_test_b200 import _capi as K
    m, n, k = shape
    ta, tb, a, b = operands(oracle, form, m, n, k, 81)
    before = dev.launch_counts()[1]
    c = dev.sgemm_host(K.PREC_BF16 if prec == "bf16" else K.PREC_TF32, ta, tb, a, b)
    assert dev.launch_counts()[1] == before + 1, "tensor-core kernel was not used"
    oracle.use_openblas()
    try:
        if prec == "bf16":
            ref = oracle.sgemm(ta, tb, oracle.round_bf16(a), oracle.round_bf16(b))
        else:
            ref = oracle.sgemm(ta, tb, a, b)
    finally:
        oracle.use_builtin_gemm()
    # per-row check as well, so that a wrong or missing 128-row block cannot hide in the norm
    assert rel_fro(c, ref) <= (TOL["bf16_f32out"] if prec == "bf16" else TOL["tf32"])
    row_err = np.linalg.norm(c - ref, axis=1) / np.maximum(np.linalg.norm(ref, axis=1), 1e-30)
    assert row_err.max() <= (1e-4 if prec == "bf16" else 4e-3)


@pytest.mark.parametrize("prec", ["fp32", "fp32tc", "tf32", "bf16"])
@pytest.mark.parametrize("shape", [(256, 512, 256), (104, 72, 136)], ids=lambda s: "x".join(map(str, s)))
def test_relu_and_mask_epilogues(dev, oracle, prec, shape):
    from tbb_test_b200 import _capi as K
    P = {"fp32": K.PREC_FP32, "fp32tc": K.PREC_FP32_TC, "tf32": K.PREC_TF32, "bf16": K.PREC_BF16}[prec]
    m, n, k = shape
    rnd = oracle.round_bf16 if prec == "bf16" else (lambda x: x)
    tol = {"fp32": TOL["fp32"], "fp32tc": TOL["fp32"], "tf32": TOL["tf32"], "bf16": TOL["bf16_bf16out"]}[prec]
    # forward with fused ReLU
    ta, tb, a, b = operands(oracle, "fwd_NT", m, n, k, 41)
    c = dev.sgemm_host(P, ta, tb, a, b, epilogue=K.EPI_RELU)
    ref = np.maximum(oracle.sgemm(ta, tb, rnd(a), rnd(b)), 0)
    assert (c >= 0).all()
    assert rel_fro(c, rnd(ref)) <= tol
    # input gradient masked by the sign of the stored activation
    ta, tb, a, b = operands(oracle, "dgrad_NN", m, n, k, 51)
    act = np.maximum(oracle.fill_uniform(m, n, 61, -1.0, 1.0), 0)
    c = dev.sgemm_host(P, ta, tb, a, b, epilogue=K.EPI_MASK, aux=act)
    ref = oracle.sgemm(ta, tb, rnd(a), rnd(b)) * (rnd(act) > 0)
    assert np.array_equal(c != 0, (ref != 0) & (c != 0))  # nothing leaks through the mask
    assert rel_fro(c, rnd(ref)) <= tol


def test_unaligned_shape_falls_back_to_cuda_cores(dev, oracle):
    """Leading dimensions that TMA cannot address (not a multiple of 16 bytes) and the
    N = 1 tail layer of the reference topology are served by the CUDA-core kernel."""
    from tbb_test_b200 import _capi as K
    for (m, n, k) in [(33, 1, 1024), (50, 30, 27)]:
        ta, tb, a, b = operands(oracle, "fwd_NT", m, n, k, 71)
        before = dev.launch_counts()[1]
        c = dev.sgemm_host(K.PREC_BF16, ta, tb, a, b)
        assert dev.launch_counts()[1] == before
        ref = oracle.sgemm(ta, tb, oracle.round_bf16(a), oracle.round_bf16(b))
        assert rel_fro(c, ref) <= TOL["bf16_f32out"]


@pytest.mark.parametrize("variant", ["B2_TC_STREAMK", "B2_TC_PAIR", "B2_TC_HALF_K"])
def test_optional_tile_schedules(dev, oracle, variant, monkeypatch):
    """The opt-in schedules of the tensor-core kernel - stream-K on the tail wave (k-blocks of
    a tile shared between CTAs through an fp32 workspace), CTA pairs (cta_group::2) and
    half-size k-blocks (64-byte swizzle) - give the same results as the default one."""
    from tbb_test_b200 import _capi as K
    monkeypatch.setenv(variant, "1")
    oracle.use_openblas()
    try:
        for form in FORMS:
            for (m, n, k) in [(4096, 4096, 192), (7944, 4096, 136), (1024, 1024, 1024), (256, 512, 2048)]:
                ta, tb, a, b = operands(oracle, form, m, n, k, 91)
                for _ in range(2):  # twice: the workspace flags must be re-armed by the first run
                    c = dev.sgemm_host(K.PREC_BF16, ta, tb, a, b)
                    ref = oracle.sgemm(ta, tb, oracle.round_bf16(a), oracle.round_bf16(b))
                    assert rel_fro(c, ref) <= TOL["bf16_f32out"], (variant, form, m, n, k)
                    row_err = np.linalg.norm(c - ref, axis=1) / np.maximum(np.linalg.norm(ref, axis=1), 1e-30)
                    assert row_err.max() <= 1e-4
    finally:
        oracle.use_builtin_gemm()
