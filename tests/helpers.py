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
