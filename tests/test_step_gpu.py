"""GPU parity of the whole training step against the CPU oracle, through the C ABI.

Tolerances are relative Frobenius errors per tensor and are stated per precision
and per kind of tensor, because two different mechanisms are at work:

  state      activations, network output, loss, weights, and the weight change
             W_k - W_0: errors are those of the operand precision (fp32 add order,
             10-bit tf32 or 8-bit bf16 mantissas) and stay small.
  gradients  dZ, dW of the last step, input gradient: in BASELINE mode they pass
             through ReLU masks. An activation that is slightly positive in one
             arithmetic and slightly negative in the other flips its mask, which
             changes that gradient element by 100 %; with a fraction p of flipped
             masks per layer the error is about sqrt(p * layers) - several percent
             for bf16/tf32 against fp32 even after ONE step, although every single
             GEMM agrees to 1e-7. They are therefore checked tightly where no flips
             can occur (one step against the oracle that rounds operands at the same
             points; REF mode, which has no ReLU) and loosely elsewhere.

                        state     W_k - W_0   gradients
  fp32  vs fp32 oracle  2e-5      2e-5        2e-5
  fp32tc vs fp32 oracle 3e-4      1e-2        5e-2     (3 x tf32 on split operands: 2e-5 per GEMM; over 10
                        steps a handful of ReLU masks differ from the fp32 run and feed themselves; REF
                        mode, no masks: 3e-4 everywhere)
  tf32  vs fp32 oracle  1e-2      5e-2        1.5e-1   (REF mode, no masks: 1e-2)
                        (the tensor core truncates fp32 operands to tf32, which shrinks
                        every product by about 1e-3 on average: a bias that adds up
                        layer by layer instead of averaging out)
  bf16  vs fp32 oracle  2e-2      1e-1        2.5e-1
  bf16 / tf32, one step, vs the oracle rounding operands identically: 2e-3 everywhere
"""
import numpy as np
import pytest

from helpers import make_problem, rel_fro

pytestmark = pytest.mark.gpu

TOL = {"fp32": dict(state=2e-5, total=2e-5, grad=2e-5),
       # fp32-class tensor-core mode: every GEMM is within the fp32 bound, but the tensor core
       # truncates (does not round) when it adds into its accumulator - a bias, which adds up layer
       # by layer and step by step instead of averaging out
       "fp32tc": dict(state=3e-4, total=1e-2, grad=5e-2),
       "tf32": dict(state=1e-2, total=5e-2, grad=1.5e-1),
       "bf16": dict(state=2e-2, total=1e-1, grad=2.5e-1)}
SAME_ROUNDING_TOL = 2e-3


def kind(name):
    if name.startswith(("dz", "dw", "dinput")):
        return "grad"
    if name.startswith("dW_total"):
        return "total"
    return "state"


def check(out, tol, skip=()):
    for name, (a, b) in out.items():
        if name in skip:
            continue
        t = tol if isinstance(tol, float) else tol[kind(name)]
        assert rel_fro(a, b) <= t, f"{name}: {rel_fro(a, b):.3e} > {t}"


def _prec(name):
    from tbb_test_b200 import _capi as K
    return {"fp32": K.PREC_FP32, "fp32tc": K.PREC_FP32_TC, "tf32": K.PREC_TF32, "bf16": K.PREC_BF16}[name]


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


@pytest.mark.parametrize("prec", ["fp32", "fp32tc", "tf32", "bf16"])
def test_baseline_mode_10_steps(native, oracle, prec):
    """Config-1-shaped job scaled to 256 wide: ReLU MLP, +-1 targets, lr 0.01, 10 steps."""
    from tbb_test_b200 import _capi as K
    nf = [256] * 6
    out, (total, tc) = run_pair(oracle, nf, 256, prec, K.MODE_BASELINE, 10, 0.01)
    check(out, TOL[prec])
    if prec != "fp32":
        assert tc >= 10 * 15, "the step did not run on the tensor-core kernels"


@pytest.mark.parametrize("prec", ["bf16", "tf32"])
def test_one_step_against_same_rounding_oracle(native, oracle, prec):
    """One step from identical state against the oracle that rounds GEMM operands at the
    same points (bf16: round-to-nearest-even at every store; tf32: the tensor core drops
    the 13 low mantissa bits of fp32 operands): every tensor, gradients included."""
    from tbb_test_b200 import _capi as K
    nf = [256, 512, 256, 128]
    rounding = oracle.ROUND_BF16 if prec == "bf16" else oracle.ROUND_TF32
    out, _ = run_pair(oracle, nf, 384, prec, K.MODE_BASELINE, 1, 0.01, rounding=rounding)
    check(out, SAME_ROUNDING_TOL)


def test_bf16_three_steps_against_rounding_oracle(native, oracle):
    from tbb_test_b200 import _capi as K
    nf = [256, 512, 256, 128]
    out, _ = run_pair(oracle, nf, 384, "bf16", K.MODE_BASELINE, 3, 0.01, rounding=oracle.ROUND_BF16)
    check(out, dict(state=5e-3, total=3e-2, grad=1e-1))


@pytest.mark.parametrize("prec", ["fp32", "fp32tc", "tf32"])
def test_ref_mode_matches_reference_semantics(native, oracle, prec):
    """REF mode = the C++ reference as written: no ReLU, the forward output fed back
    as the gradient, tiny lr (mlp_omp.cc:565,609,655)."""
    from tbb_test_b200 import _capi as K
    nf = [128, 256, 128, 64]
    out, _ = run_pair(oracle, nf, 200, prec, K.MODE_REF, 4, 1e-6)
    check(out, TOL["fp32"] if prec == "fp32" else 3e-4 if prec == "fp32tc" else dict(state=1e-2, total=1e-2, grad=1e-2))


def test_cuda_core_substitution_is_reported(native):
    """A site the tensor-core kernel cannot address is served by the CUDA-core kernel - and says so."""
    from tbb_test_b200 import _capi as K
    from tbb_test_b200.mlp import MLP
    m = MLP([128, 128, 1], 64, precision=K.PREC_BF16)
    tc, cc, why = m.site_report()
    assert tc > 0 and cc > 0 and ("N < 16" in why or "16-byte aligned" in why) and "x 1 x" in why
    m.close()
    m = MLP([128, 128, 128], 64, precision=K.PREC_BF16)
    assert m.site_report()[1] == 0
    m.close()


def test_reference_topology_with_unit_tail(native, oracle):
    """The reference's own widths end in a 1-wide layer (mlp_bench_common.h:26)."""
    from tbb_test_b200 import _capi as K
    nf = [128, 128, 128, 1]
    for prec in ("fp32", "fp32tc", "bf16"):
        out, _ = run_pair(oracle, nf, 96, prec, K.MODE_REF, 2, 1e-8,
                          rounding=oracle.ROUND_BF16 if prec == "bf16" else None)
        check(out, TOL["fp32"] if prec == "fp32" else 3e-4 if prec == "fp32tc" else SAME_ROUNDING_TOL)


@pytest.mark.parametrize("kw", [dict(overlap=False), dict(use_graph=True), dict(collect_timing=True),
                                dict(input_grad=False)], ids=lambda d: next(iter(d)))
def test_schedule_variants_agree(native, oracle, kw):
    """Serial schedule, CUDA-graph replay and timed mode give the same numbers as the
    overlapped two-stream schedule."""
    from tbb_test_b200 import _capi as K
    nf = [128, 256, 128]
    out, _ = run_pair(oracle, nf, 128, "fp32", K.MODE_BASELINE, 5, 0.01, **kw)
    check(out, TOL["fp32"], skip=("dinput",) if kw.get("input_grad") is False else ())


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


@pytest.mark.parametrize("prec", ["fp32", "bf16"])
def test_pipelined_host_fed_steps_equal_the_blocking_call(native, oracle, prec):
    """b2_train_step_host_async/b2_wait_loss (copy of step i+1 overlapped with step i, two
    input slots) computes exactly what a sequence of blocking b2_train_step_host calls
    computes, on a stream of different batches."""
    import ctypes as C
    from tbb_test_b200 import _capi as K
    from tbb_test_b200.mlp import MLP
    nf, batch, steps = [128, 256, 64], 96, 5
    ws, _, _ = make_problem(oracle, nf, batch)
    xs = [oracle.fill_normal(batch, nf[0], 100 + i) for i in range(steps)]
    ts = [oracle.fill_sign(batch, nf[-1], 200 + i) for i in range(steps)]
    fp = C.POINTER(C.c_float)

    def fresh():
        m = MLP(nf, batch, precision=_prec(prec), lr=0.02)
        for l in range(2):
            m.upload_weights(l, ws[l])
        return m

    a, b = fresh(), fresh()
    loss_a = [a.train_step_host(xs[i].ctypes.data_as(fp), nf[0], ts[i].ctypes.data_as(fp), nf[-1])
              for i in range(steps)]
    loss_b = []
    for i in range(steps):
        b.train_step_host_async(xs[i].ctypes.data_as(fp), nf[0], ts[i].ctypes.data_as(fp), nf[-1])
        if i >= 1:
            loss_b.append(b.wait_loss())
    loss_b.append(b.wait_loss())
    # the loss is summed with floating-point atomics: equal up to the order of additions
    assert np.allclose(loss_a, loss_b, rtol=1e-12, atol=0)
    for l in range(2):
        assert np.array_equal(a.weights(l), b.weights(l))
    # a third step in flight is refused, and so is b2_step while steps are pending
    b.train_step_host_async(xs[0].ctypes.data_as(fp), nf[0], ts[0].ctypes.data_as(fp), nf[-1])
    b.train_step_host_async(xs[1].ctypes.data_as(fp), nf[0], ts[1].ctypes.data_as(fp), nf[-1])
    assert b.lib.b2_train_step_host_async(b._h, xs[2].ctypes.data_as(fp), nf[0], None, 0) == K.ERR_STATE
    assert b.lib.b2_step(b._h, 1) == K.ERR_STATE
    b.wait_loss()
    b.wait_loss()
    assert b.lib.b2_wait_loss(b._h, None) == K.ERR_STATE
    # the loss decreases over a few steps of the same batch through the oracle's eyes
    orc = oracle.Oracle(nf, batch, mode=oracle.MODE_BASELINE, lr=0.02,
                        rounding=oracle.ROUND_BF16 if prec == "bf16" else oracle.ROUND_NONE)
    for l in range(2):
        orc.set_weights(l, ws[l])
    orc.set_input(xs[0])
    orc.set_target(ts[0])
    orc.step(1)
    assert abs(loss_a[0] - orc.loss()) <= 1e-3 * abs(orc.loss())
    a.close()
    b.close()
    orc.close()


def test_bf16_gradients_mode(native, oracle):
    """Configuration-5 style: weight gradients produced, summed and read by SGD in bf16
    (fp32 master weights). One step against the oracle that rounds the same way; the
    gradient itself differs by bf16 rounding only."""
    from tbb_test_b200 import _capi as K
    from tbb_test_b200.mlp import MLP
    nf, batch = [256, 512, 256], 256
    ws, x, t = make_problem(oracle, nf, batch)
    dev = MLP(nf, batch, precision=K.PREC_BF16, grad_bf16=True, lr=0.01)
    orc = oracle.Oracle(nf, batch, mode=oracle.MODE_BASELINE, rounding=oracle.ROUND_BF16, grad_bf16=True, lr=0.01)
    for l in range(2):
        dev.upload_weights(l, ws[l])
        orc.set_weights(l, ws[l])
    dev.upload_input(x)
    dev.upload_target(t)
    orc.set_input(x)
    orc.set_target(t)
    dev.step(1)
    orc.step(1)
    for l in range(2):
        g = dev.weight_grad(l)
        assert np.array_equal(g, oracle.round_bf16(g)), "gradient buffer is not bf16-valued"
        assert rel_fro(g, orc.weight_grad(l)) <= 5e-3
        assert rel_fro(dev.weights(l) - ws[l], orc.weights(l) - ws[l]) <= 5e-3
    dev.close()
    orc.close()


def test_chrome_trace_of_a_timed_step(native, oracle, tmp_path):
    import json
    from tbb_test_b200 import _capi as K
    from tbb_test_b200.mlp import MLP
    nf, batch = [128, 256, 128], 128
    ws, x, t = make_problem(oracle, nf, batch)
    dev = MLP(nf, batch, collect_timing=True)
    for l in range(2):
        dev.upload_weights(l, ws[l])
    dev.upload_input(x)
    dev.upload_target(t)
    dev.step(2)
    path = tmp_path / "trace.json"
    dev.write_trace(path)
    ev = json.loads(path.read_text())
    names = {e["name"] for e in ev}
    assert {"fwd 0", "fwd 1", "wgt_grad 0", "wgt_grad 1", "bwd 0", "bwd 1", "wgt_update 0", "wgt_update 1"} <= names
    assert all(e["ph"] == "X" and e["dur"] >= 0 and e["ts"] >= 0 for e in ev)
    assert {e["args"]["step"] for e in ev} == {0, 1}
    phases, total, steps = dev.timing()
    assert steps == 2 and total > 0 and phases[:, K.T_FWD].sum() > 0
    plain = MLP(nf, batch)
    assert plain.lib.b2_write_trace(plain._h, str(path).encode()) == K.ERR_STATE
    plain.close()
    dev.close()


def test_measurement_entry_points(native, oracle):
    """The micro-benchmarks and checks the benchmark relies on: SGD alone on cold data, one GEMM
    form alone, the collectives' sweep on one rank (nothing to exchange: time 0, data unchanged),
    the timing switch and the weight fingerprint."""
    import torch
    from tbb_test_b200 import _capi as K
    from tbb_test_b200.mlp import MLP
    nf, batch = [128, 256, 128], 128
    ws, x, t = make_problem(oracle, nf, batch)
    dev = MLP(nf, batch, precision=K.PREC_BF16)
    for l in range(2):
        dev.upload_weights(l, ws[l])
    dev.upload_input(x)
    dev.upload_target(t)
    ms, nbytes = dev.sgd_bench(1 << 20, K.DTYPE_F32, with_bf16_copy=True, iters=5)
    assert ms > 0 and nbytes == (1 << 20) * 14
    assert dev.gemm_bench(0, 512, 256, 256, K.PREC_BF16, K.EPI_RELU, K.DTYPE_BF16, iters=3) > 0
    assert dev.gemm_bench(1, 256, 256, 512, K.PREC_FP32_TC, iters=3) > 0
    for kind in (0, 1, 2):
        assert dev.collective_bench(kind, 4096, K.DTYPE_F32, 1, 2) == 0.0
    # the fingerprint is the wrap-around sum of the 32-bit words of the bf16 operand copy
    fp0 = dev.weights_fingerprint(0)
    words = oracle.round_bf16(ws[0]).view(np.uint32) >> 16  # bf16 bit patterns
    pairs = (words.ravel()[0::2].astype(np.uint64) | (words.ravel()[1::2].astype(np.uint64) << np.uint64(16)))
    assert fp0 == int(pairs.sum(dtype=np.uint64))
    dev.step(1)
    assert dev.weights_fingerprint(0) != fp0  # the update changed the weights
    # per-phase events can be switched on for a few steps and off again
    dev.set_timing(True)
    dev.reset_timing()
    dev.step(2)
    phases, total, steps = dev.timing()
    assert steps == 2 and phases[:, K.T_FWD].sum() > 0 and dev.gemm_busy_ms() > 0
    dev.set_timing(False)
    # in-place sum on a caller-owned device buffer: one rank leaves it as it is
    buf = torch.arange(1000, dtype=torch.float32, device="cuda")
    dev.allreduce(buf.data_ptr(), buf.numel(), K.DTYPE_F32)
    assert torch.equal(buf.cpu(), torch.arange(1000, dtype=torch.float32))
    host = np.zeros(16, np.float32)
    assert dev.lib.b2_allreduce(dev._h, host.ctypes.data, 16, K.DTYPE_F32) == K.ERR_INVALID
    dev.close()


def test_pinned_memory_near_the_gpu(native):
    """b2_host_alloc_near: pinned pages from the NUMA node of the GPU (the reference's
    create_matrix_with_numa_aware_allocation, mlp_omp.cc:27-47). The node is whatever sysfs says
    (-1 where it says nothing); the memory is usable, the thread's CPU affinity is as before, and
    a host-fed step from it gives the same loss as one fed from plain pinned memory."""
    import os
    from tbb_test_b200 import _capi as K
    from tbb_test_b200.mlp import MLP, pinned_array
    before = os.sched_getaffinity(0)
    nodes = []
    x = pinned_array((256, 128), device=0, node_out=nodes)
    t = pinned_array((256, 64), device=0, node_out=nodes)
    assert os.sched_getaffinity(0) == before
    assert len(nodes) == 2 and nodes[0] == nodes[1] and nodes[0] >= -1
    rng = np.random.default_rng(5)
    x[:] = rng.standard_normal(x.shape, dtype=np.float32)
    t[:] = np.sign(rng.standard_normal(t.shape)).astype(np.float32)
    x2, t2 = pinned_array(x.shape), pinned_array(t.shape)
    x2[:], t2[:] = x, t
    losses = []
    for xs, ts in ((x, t), (x2, t2)):
        dev = MLP([128, 96, 64], 256, precision=K.PREC_BF16, mode=K.MODE_BASELINE, lr=0.01)
        for l, (fo, fi) in enumerate([(96, 128), (64, 96)]):
            dev.upload_weights(l, np.random.default_rng(l).uniform(-0.1, 0.1, (fo, fi)).astype(np.float32))
        losses.append(dev.train_step_host(xs.ctypes.data_as(K._fp), 128, ts.ctypes.data_as(K._fp), 64))
        dev.close()
    assert losses[0] == losses[1] and np.isfinite(losses[0])
