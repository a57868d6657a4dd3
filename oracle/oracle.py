"""ctypes loaders for the checker binaries of this directory.

TEST INFRASTRUCTURE ONLY.  `Oracle` wraps liboracle.so (the C restatement in
mlp_oracle.c); `RefLib` wraps oracle/_ref/libref_mlp_omp.so (the unmodified
reference sources plus ref_harness.cc) where it has been built.  Only tests,
the smoke check and the CPU-baseline leg of the benchmark may import this.
"""
import ctypes as C
import glob
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libref_mlp_omp.so")

MODE_REF, MODE_BASELINE = 0, 1
ROUND_NONE, ROUND_TF32, ROUND_BF16 = 0, 1, 2

_fp = C.POINTER(C.c_float)
_ip = C.POINTER(C.c_int)


def build(force=False):
    """Compile liboracle.so (and oracle/_ref when the reference sources exist)."""
    if force or not os.path.exists(ORACLE_SO) or (
            os.path.getmtime(ORACLE_SO) < os.path.getmtime(os.path.join(HERE, "mlp_oracle.c"))):
        subprocess.run(["bash", os.path.join(HERE, "build_ref.sh")], check=True,
                       stdout=subprocess.DEVNULL)


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_fp)


def find_openblas():
    env = os.environ.get("B2_OPENBLAS_PATH")
    pats = [env] if env else []
    try:
        import scipy
        pats.append(os.path.join(os.path.dirname(os.path.dirname(scipy.__file__)), "scipy.libs",
                                 "libscipy_openblas-*.so"))
    except Exception:
        pass
    for p in pats:
        hits = sorted(glob.glob(p))
        if hits:
            return hits[0]
    return None


class _Cfg(C.Structure):
    _fields_ = [("nlayers", C.c_int), ("nfeatures", _ip), ("batch", C.c_int), ("nranks", C.c_int),
                ("mode", C.c_int), ("rounding", C.c_int), ("grad_bf16", C.c_int), ("lr", C.c_float)]


_lib = None
_blas = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(ORACLE_SO)
        L.orc_create.restype = C.c_void_p
        L.orc_create.argtypes = [C.POINTER(_Cfg)]
        L.orc_destroy.argtypes = [C.c_void_p]
        for name in ("orc_set_weights", "orc_get_weights", "orc_get_activation", "orc_get_dz",
                     "orc_get_weight_grad"):
            getattr(L, name).argtypes = [C.c_void_p, C.c_int, _fp, C.c_size_t]
        for name in ("orc_set_input", "orc_set_target", "orc_get_input_grad"):
            getattr(L, name).argtypes = [C.c_void_p, _fp, C.c_size_t]
        L.orc_step.argtypes = [C.c_void_p, C.c_int]
        L.orc_loss.restype = C.c_double
        L.orc_loss.argtypes = [C.c_void_p]
        L.orc_sgemm.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, _fp, C.c_int,
                                _fp, C.c_int, C.c_float, _fp, C.c_int]
        L.orc_set_sgemm.argtypes = [C.c_void_p]
        L.orc_set_ksplit.argtypes = [C.c_int]
        L.orc_batch_range.argtypes = [C.c_int, C.c_int, C.c_int, _ip, _ip]
        L.orc_kat_fill.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, _fp, _fp, C.c_size_t]
        L.orc_kat_expected.argtypes = [C.c_int, C.c_int, C.c_int, _fp, C.c_size_t]
        L.orc_ring_update.argtypes = [C.c_int, C.c_int, C.c_int, C.c_size_t, _fp, _fp, _fp, C.c_float]
        L.orc_checksum.argtypes = [_fp, C.c_int, C.c_int, C.c_size_t, C.POINTER(C.c_double)]
        L.orc_fill_uniform.argtypes = [_fp, C.c_int, C.c_int, C.c_size_t, C.c_uint64, C.c_uint64,
                                       C.c_float, C.c_float]
        L.orc_fill_normal.argtypes = [_fp, C.c_int, C.c_int, C.c_size_t, C.c_uint64, C.c_uint64,
                                      C.c_float]
        L.orc_fill_sign.argtypes = [_fp, C.c_int, C.c_int, C.c_size_t, C.c_uint64, C.c_uint64]
        L.orc_round_bf16.restype = C.c_float
        L.orc_round_bf16.argtypes = [C.c_float]
        _lib = L
    return _lib


def use_openblas(threads=None):
    """Route the oracle's GEMMs through scipy's OpenBLAS (same arithmetic order as
    the reference build of oracle/_ref uses per tile). Returns the library path or
    None when it is not present (the built-in loops stay in use)."""
    global _blas
    path = find_openblas()
    if path is None:
        return None
    if _blas is None:
        _blas = C.CDLL(path)
    if threads is not None:
        _blas.scipy_openblas_set_num_threads(int(threads))
    lib().orc_set_sgemm(C.cast(_blas.scipy_cblas_sgemm, C.c_void_p))
    return path


def use_builtin_gemm():
    lib().orc_set_sgemm(None)


def set_ksplit(s):
    """s > 1: the oracle sums every GEMM as s partial products over consecutive ranges of the
    contraction index - the same sum in another fp32 order. Comparing two oracle runs that
    differ only in this switch gives the configuration's own sensitivity to summation order."""
    lib().orc_set_ksplit(int(s))


def sgemm(transa, transb, a, b, alpha=1.0):
    """Row-major op(a) @ op(b) through the oracle's GEMM."""
    a, pa = _f32(a)
    b, pb = _f32(b)
    m = a.shape[1] if transa else a.shape[0]
    k = a.shape[0] if transa else a.shape[1]
    n = b.shape[0] if transb else b.shape[1]
    c = np.zeros((m, n), np.float32)
    lib().orc_sgemm(int(transa), int(transb), m, n, k, alpha, pa, a.shape[1], pb, b.shape[1], 0.0,
                    c.ctypes.data_as(_fp), n)
    return c


def batch_range(batch, nranks, rank):
    b, e = C.c_int(), C.c_int()
    lib().orc_batch_range(batch, nranks, rank, C.byref(b), C.byref(e))
    return b.value, e.value


def round_bf16(a):
    """Round-to-nearest-even bf16 of a float32 array, returned as float32."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return r.view(np.float32).reshape(np.shape(a))


class Oracle:
    """One MLP training job on the CPU (see mlp_oracle.h)."""

    def __init__(self, nfeatures, batch, nranks=1, mode=MODE_BASELINE, rounding=ROUND_NONE,
                 grad_bf16=False, lr=0.01):
        self.nf = list(nfeatures)
        self.L = len(self.nf) - 1
        self.batch = batch
        arr = (C.c_int * len(self.nf))(*self.nf)
        cfg = _Cfg(self.L, arr, batch, nranks, mode, rounding, int(grad_bf16), lr)
        self._h = lib().orc_create(C.byref(cfg))

    def close(self):
        if self._h:
            lib().orc_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_weights(self, l, w):
        w, p = _f32(w)
        assert w.shape == (self.nf[l + 1], self.nf[l])
        lib().orc_set_weights(self._h, l, p, w.shape[1])

    def weights(self, l):
        w = np.empty((self.nf[l + 1], self.nf[l]), np.float32)
        lib().orc_get_weights(self._h, l, w.ctypes.data_as(_fp), w.shape[1])
        return w

    def set_input(self, x):
        x, p = _f32(x)
        assert x.shape == (self.batch, self.nf[0])
        lib().orc_set_input(self._h, p, x.shape[1])

    def set_target(self, t):
        t, p = _f32(t)
        assert t.shape == (self.batch, self.nf[-1])
        lib().orc_set_target(self._h, p, t.shape[1])

    def step(self, n=1):
        lib().orc_step(self._h, n)

    def activation(self, l):
        a = np.empty((self.batch, self.nf[l]), np.float32)
        lib().orc_get_activation(self._h, l, a.ctypes.data_as(_fp), a.shape[1])
        return a

    def dz(self, l):
        g = np.empty((self.batch, self.nf[l + 1]), np.float32)
        lib().orc_get_dz(self._h, l, g.ctypes.data_as(_fp), g.shape[1])
        return g

    def input_grad(self):
        g = np.empty((self.batch, self.nf[0]), np.float32)
        lib().orc_get_input_grad(self._h, g.ctypes.data_as(_fp), g.shape[1])
        return g

    def weight_grad(self, l):
        g = np.empty((self.nf[l + 1], self.nf[l]), np.float32)
        lib().orc_get_weight_grad(self._h, l, g.ctypes.data_as(_fp), g.shape[1])
        return g

    def loss(self):
        return lib().orc_loss(self._h)


def fill_uniform(nrows, ncols, seed, lo, hi, start=0):
    a = np.empty((nrows, ncols), np.float32)
    lib().orc_fill_uniform(a.ctypes.data_as(_fp), nrows, ncols, ncols, seed, start, lo, hi)
    return a


def fill_normal(nrows, ncols, seed, stddev=1.0, start=0):
    a = np.empty((nrows, ncols), np.float32)
    lib().orc_fill_normal(a.ctypes.data_as(_fp), nrows, ncols, ncols, seed, start, stddev)
    return a


def fill_sign(nrows, ncols, seed, start=0):
    a = np.empty((nrows, ncols), np.float32)
    lib().orc_fill_sign(a.ctypes.data_as(_fp), nrows, ncols, ncols, seed, start)
    return a


def kat(nsockets, nrows, ncols):
    """(weights, grads) stacked over sockets and the expected updated replica."""
    w = np.zeros((nsockets, nrows, ncols), np.float32)
    g = np.zeros((nsockets, nrows, ncols), np.float32)
    for s in range(nsockets):
        lib().orc_kat_fill(nsockets, nrows, ncols, s, w[s].ctypes.data_as(_fp),
                           g[s].ctypes.data_as(_fp), ncols)
    e = np.zeros((nrows, ncols), np.float32)
    lib().orc_kat_expected(nsockets, nrows, ncols, e.ctypes.data_as(_fp), ncols)
    return w, g, e


def ring_update(w, g, alpha, pad=16):
    """orc_ring_update on (nsockets, nrows, ncols) arrays, laid out like the reference's
    Matrix (ld = ncols + pad, because the chunk boundaries depend on ld); returns the
    new weights."""
    n, nrows, ncols = w.shape
    ld = ncols + pad
    wp = np.zeros((n, nrows, ld), np.float32)
    gp = np.zeros((n, nrows, ld), np.float32)
    wp[:, :, :ncols] = w
    gp[:, :, :ncols] = g
    push = np.zeros_like(wp)
    lib().orc_ring_update(n, nrows, ncols, ld, wp.ctypes.data_as(_fp), gp.ctypes.data_as(_fp),
                          push.ctypes.data_as(_fp), alpha)
    return np.ascontiguousarray(wp[:, :, :ncols])


def checksum(w):
    w, p = _f32(w)
    out = (C.c_double * 3)()
    lib().orc_checksum(p, w.shape[0], w.shape[1], w.shape[1], out)
    return tuple(out)


class RefLib:
    """The unmodified reference, through ref_harness.cc (needs oracle/_ref)."""

    def __init__(self):
        if not os.path.exists(REF_SO):
            raise FileNotFoundError(REF_SO)
        L = C.CDLL(REF_SO)
        L.ref_blas_name.restype = C.c_char_p
        L.ref_get_weights.argtypes = [C.c_int, C.c_int, _fp, C.c_size_t]
        L.ref_get_weight_grad.argtypes = [C.c_int, C.c_int, _fp, C.c_size_t]
        L.ref_get_activation.argtypes = [C.c_int, _fp, C.c_size_t]
        L.ref_update_weight.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, _fp, _fp, C.c_double]
        L.ref_time_update_weight.restype = C.c_double
        L.ref_time_update_weight.argtypes = [C.c_int] * 5
        L.ref_get_partition.argtypes = [C.c_int] * 5 + [_ip]
        L.ref_intra_socket_2d.argtypes = [C.c_int, C.c_int, C.c_double, C.c_int, C.c_int, C.c_int, _ip]
        L.ref_2dpartition.argtypes = [C.c_int, C.c_int, C.c_int, C.c_double, C.c_int, C.c_int, C.c_int,
                                      C.c_int, _ip]
        L.ref_hypercube.argtypes = [C.c_int] * 5 + [_ip]
        L.ref_ring_info.argtypes = [C.c_int, C.c_int, C.c_int, _ip]
        self.L = L

    def nfeatures(self):
        return [self.L.ref_nfeatures(i) for i in range(self.L.ref_nlayers() + 1)]

    def run_main(self, nsockets, nthreads_per_socket):
        return self.L.ref_run_main(nsockets, nthreads_per_socket)

    def reinit(self):
        self.L.ref_reinit()

    def weights(self, l, replica=0):
        nf = self.nfeatures()
        w = np.empty((nf[l + 1], nf[l]), np.float32)
        self.L.ref_get_weights(l, replica, w.ctypes.data_as(_fp), nf[l])
        return w

    def weight_grad(self, l, replica=0):
        nf = self.nfeatures()
        w = np.empty((nf[l + 1], nf[l]), np.float32)
        self.L.ref_get_weight_grad(l, replica, w.ctypes.data_as(_fp), nf[l])
        return w

    def activation(self, l):
        nf = self.nfeatures()
        cols = nf[l] if l < len(nf) else nf[0]  # the spare buffer has the input's width
        a = np.empty((self.L.ref_batch(), cols), np.float32)
        self.L.ref_get_activation(l, a.ctypes.data_as(_fp), cols)
        return a

    def update_weight(self, w, g, alpha, nthreads_per_socket=1):
        n, nrows, ncols = w.shape
        w = np.array(w, np.float32, order="C")
        g = np.ascontiguousarray(g, np.float32)
        self.L.ref_update_weight(n, nthreads_per_socket, nrows, ncols, w.ctypes.data_as(_fp),
                                 g.ctypes.data_as(_fp), alpha)
        return w

    def time_update_weight(self, nsock, nthr, nrows, ncols, iters):
        """Seconds per call of the reference's allreduce + SGD on (nsock*nrows) x ncols buffers."""
        return self.L.ref_time_update_weight(nsock, nthr, nrows, ncols, iters)

    def _ints(self, fn, n, *args):
        out = (C.c_int * n)()
        fn(*args, out)
        return list(out)

    def get_partition(self, nsock, work, sid, nthr, tid):
        return self._ints(self.L.ref_get_partition, 2, nsock, work, sid, nthr, tid)

    def intra_socket_2d(self, m, n, ar, m_align, nthr, tid):
        return self._ints(self.L.ref_intra_socket_2d, 4, m, n, ar, int(m_align), nthr, tid)

    def partition_2d(self, nsock, m, n, ar, m_align, sid, nthr, tid):
        return self._ints(self.L.ref_2dpartition, 4, nsock, m, n, ar, int(m_align), sid, nthr, tid)

    def hypercube(self, twisted, n, shift, node, dim):
        return self._ints(self.L.ref_hypercube, 3, int(twisted), n, shift, node, dim)

    def ring_info(self, nsock, sid, task):
        return self._ints(self.L.ref_ring_info, 3, nsock, sid, task)
