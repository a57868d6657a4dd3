"""Shared helpers of the parity tests."""
import numpy as np


def rel_fro(x, ref):
    x = np.asarray(x, np.float64)
    ref = np.asarray(ref, np.float64)
    d = np.linalg.norm(x - ref)
    n = np.linalg.norm(ref)
    return d / n if n > 0 else d


def rel_max(x, ref):
    x = np.asarray(x, np.float64)
    ref = np.asarray(ref, np.float64)
    m = np.max(np.abs(ref))
    return np.max(np.abs(x - ref)) / (m if m > 0 else 1.0)


def make_problem(O, nf, batch, wdist=("uniform", None), seed_w=0, seed_x=1, seed_t=2):
    """Seeded weights / inputs / targets in the style of the benchmark configurations:
    weights U(-a, a) (default a = 1/sqrt(fan_in)) or N(0, s), inputs N(0,1), targets +-1."""
    L = len(nf) - 1
    ws = []
    for l in range(L):
        kind, par = wdist
        if kind == "uniform":
            a = par if par is not None else 1.0 / np.sqrt(nf[l])
            ws.append(O.fill_uniform(nf[l + 1], nf[l], seed_w + 1000 * l, -a, a))
        else:
            ws.append(O.fill_normal(nf[l + 1], nf[l], seed_w + 1000 * l, par))
    x = O.fill_normal(batch, nf[0], seed_x)
    t = O.fill_sign(batch, nf[-1], seed_t)
    return ws, x, t


def run_step_pair(O, nf, batch, precision, mode, steps, lr, rounding=None, wdist=("uniform", None),
                  openblas=False, taps="all", floor_ksplit=0, **kw):
    """The same seeded job on the GPU (through the C ABI) and in the CPU oracle; returns
    {tensor name: (device value, oracle value)} and the device's launch counters.
    `taps` = "all" compares every activation, dZ, dW, weight change, the input gradient and
    the loss; "weights" only the network output, dW, the weight change and the loss (for
    shapes whose activations take long to copy back).
    floor_ksplit > 1 also runs a second oracle that adds every GEMM up in `floor_ksplit`
    partial sums (another fp32 order, nothing else changed) and returns, as a third value,
    {tensor name: relative error between the two oracles}: the distance at which two correct
    implementations of this very configuration already are."""
    from tbb_test_b200.mlp import MLP
    ws, x, t = make_problem(O, nf, batch, wdist=wdist)
    L = len(nf) - 1
    if openblas:
        O.use_openblas()

    def taps_of(m):
        out = {"y": m.activation(L)}
        for l in range(L):
            out[f"dw{l}"] = m.weight_grad(l)
            out[f"dW_total{l}"] = m.weights(l) - ws[l]
        if taps == "all":
            for l in range(1, L):
                out[f"act{l}"] = m.activation(l)
            for l in range(L):
                out[f"dz{l}"] = m.dz(l)
            out["dinput"] = m.input_grad()
        out["loss"] = np.array([m.loss()])
        return out

    def oracle_run(ksplit):
        O.set_ksplit(ksplit)
        try:
            orc = O.Oracle(nf, batch, nranks=1, mode=mode, lr=lr,
                           rounding=O.ROUND_NONE if rounding is None else rounding,
                           grad_bf16=bool(kw.get("grad_bf16", False)))
            for l in range(L):
                orc.set_weights(l, ws[l])
            orc.set_input(x)
            orc.set_target(t)
            orc.step(steps)
            res = taps_of(orc)
            orc.close()
        finally:
            O.set_ksplit(1)
        return res

    try:
        dev = MLP(nf, batch, mode=mode, precision=precision, lr=lr, **kw)
        for l in range(L):
            dev.upload_weights(l, ws[l])
        dev.upload_input(x)
        dev.upload_target(t)
        dev.step(steps)
        got = taps_of(dev)
        counts = dev.launch_counts()
        dev.close()
        ref = oracle_run(1)
        out = {k: (got[k], ref[k]) for k in ref}
        floor = None
        if floor_ksplit > 1:
            alt = oracle_run(floor_ksplit)
            floor = {k: rel_fro(alt[k], ref[k]) for k in ref}
    finally:
        if openblas:
            O.use_builtin_gemm()
    if floor_ksplit > 1:
        return out, counts, floor
    return out, counts


def problem_weights(O, nf, batch, wdist):
    """The initial weights run_step_pair uses for this problem."""
    return make_problem(O, nf, batch, wdist=wdist)[0]


def tensor_kind(name):
    if name.startswith(("dz", "dw", "dinput")):
        return "grad"
    if name.startswith("dW_total"):
        return "total"
    return "state"


def worst_errors(out, floor=None):
    """Largest relative Frobenius error per kind of tensor, with the tensor's name (and the
    oracle-to-oracle distance of that tensor when `floor` is given)."""
    worst = {}
    for name, (a, b) in out.items():
        e = rel_fro(a, b)
        k = tensor_kind(name)
        if k not in worst or e > worst[k][0]:
            worst[k] = (e, name) + ((floor[name],) if floor else ())
    return worst


def check_errors(out, tol, skip=(), floor=None, factor=1.0, weights=None):
    """tol: one bound for all tensors or {"state","total","grad"} bounds. With `floor`
    (oracle-to-oracle distances from run_step_pair) a tensor passes if its error is within
    tol or within factor * floor, whichever is larger. With `weights` (the initial weight
    matrices) a weight change dW_total<l> = W_k - W_0 is also allowed to be off by one fp32
    rounding of the weights themselves, 2^-23 * ||W_0||: where lr * dW is smaller than the
    spacing of fp32 numbers around W, the change IS that rounding on either side."""
    for name, (a, b) in out.items():
        if name in skip:
            continue
        t = tol if isinstance(tol, float) else tol[tensor_kind(name)]
        if floor is not None:
            t = max(t, factor * floor[name])
        a64, b64 = np.asarray(a, np.float64), np.asarray(b, np.float64)
        diff, ref = np.linalg.norm(a64 - b64), np.linalg.norm(b64)
        allow = t * ref if ref > 0 else t
        if weights is not None and name.startswith("dW_total"):
            allow += 2.0 ** -23 * np.linalg.norm(np.asarray(weights[int(name[8:])], np.float64))
        assert diff <= allow, f"{name}: |diff| {diff:.3e} > {allow:.3e} (relative {diff / ref if ref else diff:.3e}, bound {t:.3e})"
