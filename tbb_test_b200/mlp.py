"""Python view of one b200mlp handle (one GPU of a data-parallel MLP training job).

Thin object wrapper over the C ABI (include/b200mlp.h) used by the tests, the
smoke check and the benchmark; host matrices are numpy float32 arrays.  The
names follow the reference's driver: weights / weight_grads / activations
(mlp_bench_common.h:53-55), update_weight (mlp_omp.cc:297).
"""
import ctypes as C

import numpy as np

from . import _capi as K

_fp = C.POINTER(C.c_float)


def _mat(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_fp), a.shape[1]


def nccl_unique_id():
    buf = (C.c_char * K.NCCL_ID_BYTES)()
    rc = K.lib().b2_nccl_unique_id(buf)
    if rc != K.OK:
        raise K.B2Error(rc, K.lib().b2_last_error(None).decode())
    return bytes(buf)


def p2p_emulate(bufs, device=0, wait_ms=1000, lagging_rank=-1):
    """Sum of the equally long float32 arrays `bufs` (one per emulated rank) into each of them,
    by the peer-memory allreduce kernel with all ranks on one GPU."""
    arrs = [np.ascontiguousarray(b, dtype=np.float32) for b in bufs]
    ptrs = (_fp * len(arrs))(*[a.ctypes.data_as(_fp) for a in arrs])
    rc = K.lib().b2_p2p_emulate_opts(device, len(arrs), ptrs, arrs[0].size, wait_ms, lagging_rank)
    if rc != K.OK:
        raise K.B2Error(rc, K.lib().b2_last_error(None).decode())
    return arrs


class MLP:
    def __init__(self, nfeatures, batch, *, rank=0, world_size=1, device=0, mode=K.MODE_BASELINE,
                 precision=K.PREC_FP32, grad_bf16=False, allreduce=True, overlap=True, input_grad=True,
                 collect_timing=False, use_graph=False, force_simt=False, lr=0.01, nccl_id=None, comm_sms=-1,
                 ar_bucket_mb=-1, shard_update=-1):
        self.lib = K.lib()
        self.nf = [int(f) for f in nfeatures]
        self.L = len(self.nf) - 1
        self.batch = int(batch)
        cfg = K.Config()
        self.lib.b2_config_default(C.byref(cfg))
        self._nf_arr = (C.c_int * len(self.nf))(*self.nf)
        cfg.nlayers = self.L
        cfg.nfeatures = self._nf_arr
        cfg.batch = self.batch
        cfg.rank, cfg.world_size, cfg.device = rank, world_size, device
        cfg.mode, cfg.precision = mode, precision
        cfg.grad_bf16 = int(grad_bf16)
        cfg.allreduce, cfg.overlap, cfg.input_grad = int(allreduce), int(overlap), int(input_grad)
        cfg.collect_timing, cfg.use_graph, cfg.force_simt = int(collect_timing), int(use_graph), int(force_simt)
        cfg.lr = lr
        cfg.comm_sms = comm_sms
        cfg.ar_bucket_mb = ar_bucket_mb
        cfg.shard_update = shard_update
        self._id = None
        if nccl_id is not None:
            self._id = C.create_string_buffer(bytes(nccl_id), K.NCCL_ID_BYTES)
            cfg.nccl_unique_id = C.cast(self._id, C.c_void_p)
        h = C.c_void_p()
        rc = self.lib.b2_create(C.byref(cfg), C.byref(h))
        if rc != K.OK:
            raise K.B2Error(rc, self.lib.b2_last_error(None).decode())
        self._h = h
        b, e = C.c_int(), C.c_int()
        self.lib.b2_batch_range(self._h, C.byref(b), C.byref(e))
        self.rows = (b.value, e.value)

    # -- lifetime ---------------------------------------------------------
    def close(self):
        if getattr(self, "_h", None):
            self.lib.b2_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def _ck(self, rc):
        if rc != K.OK:
            raise K.B2Error(rc, self.lib.b2_last_error(self._h).decode())

    # -- state ------------------------------------------------------------
    def upload_weights(self, l, w):
        w, p, ld = _mat(w)
        assert w.shape == (self.nf[l + 1], self.nf[l])
        self._ck(self.lib.b2_upload_weights(self._h, l, p, ld))

    def weights(self, l):
        w = np.empty((self.nf[l + 1], self.nf[l]), np.float32)
        self._ck(self.lib.b2_download_weights(self._h, l, w.ctypes.data_as(_fp), w.shape[1]))
        return w

    def upload_input(self, x):
        x, p, ld = _mat(x)
        assert x.shape == (self.batch, self.nf[0])
        self._ck(self.lib.b2_upload_input(self._h, p, ld))

    def upload_target(self, t):
        t, p, ld = _mat(t)
        assert t.shape == (self.batch, self.nf[-1])
        self._ck(self.lib.b2_upload_target(self._h, p, ld))

    def _rows_only(self, full):
        return full[self.rows[0]:self.rows[1]]

    def activation(self, l):
        """This rank's rows of activation l (l = L is the network output)."""
        a = np.zeros((self.batch, self.nf[l]), np.float32)
        self._ck(self.lib.b2_download_activation(self._h, l, a.ctypes.data_as(_fp), a.shape[1]))
        return self._rows_only(a)

    def dz(self, l):
        g = np.zeros((self.batch, self.nf[l + 1]), np.float32)
        self._ck(self.lib.b2_download_dz(self._h, l, g.ctypes.data_as(_fp), g.shape[1]))
        return self._rows_only(g)

    def input_grad(self):
        g = np.zeros((self.batch, self.nf[0]), np.float32)
        self._ck(self.lib.b2_download_input_grad(self._h, g.ctypes.data_as(_fp), g.shape[1]))
        return self._rows_only(g)

    def weight_grad(self, l):
        g = np.empty((self.nf[l + 1], self.nf[l]), np.float32)
        self._ck(self.lib.b2_download_weight_grad(self._h, l, g.ctypes.data_as(_fp), g.shape[1]))
        return g

    def upload_weight_grad(self, l, g):
        g, p, ld = _mat(g)
        assert g.shape == (self.nf[l + 1], self.nf[l])
        self._ck(self.lib.b2_upload_weight_grad(self._h, l, p, ld))

    def set_lr(self, lr):
        self._ck(self.lib.b2_set_lr(self._h, lr))

    # -- compute ----------------------------------------------------------
    def step(self, iters=1):
        self._ck(self.lib.b2_step(self._h, iters))

    def loss(self):
        v = C.c_double()
        self._ck(self.lib.b2_loss(self._h, C.byref(v)))
        return v.value

    def train_step_host(self, x_ptr, ldx, t_ptr, ldt):
        """One step fed from host pointers (ctypes float pointers); returns the loss share."""
        v = C.c_double()
        self._ck(self.lib.b2_train_step_host(self._h, x_ptr, ldx, t_ptr, ldt, C.byref(v)))
        return v.value

    def train_step_host_async(self, x_ptr, ldx, t_ptr, ldt):
        """Enqueue copy + step without waiting (at most two in flight)."""
        self._ck(self.lib.b2_train_step_host_async(self._h, x_ptr, ldx, t_ptr, ldt))

    def wait_loss(self):
        v = C.c_double()
        self._ck(self.lib.b2_wait_loss(self._h, C.byref(v)))
        return v.value

    def update_weight(self, l):
        """allreduce + SGD of layer l (the reference's update_weight)."""
        self._ck(self.lib.b2_allreduce_sgd(self._h, l))

    def sgemm_host(self, precision, transa, transb, a, b, epilogue=K.EPI_NONE, aux=None):
        a, pa, lda = _mat(a)
        b, pb, ldb = _mat(b)
        m = a.shape[1] if transa else a.shape[0]
        k = a.shape[0] if transa else a.shape[1]
        n = b.shape[0] if transb else b.shape[1]
        assert (b.shape[1] if transb else b.shape[0]) == k
        c = np.zeros((m, n), np.float32)
        px, ldx = None, 0
        if aux is not None:
            aux, px, ldx = _mat(aux)
            assert aux.shape == (m, n)
        self._ck(self.lib.b2_sgemm_host(self._h, precision, int(transa), int(transb), m, n, k, pa, lda, pb, ldb,
                                        c.ctypes.data_as(_fp), n, epilogue, px, ldx))
        return c

    def allreduce(self, dev_ptr, count, dtype=K.DTYPE_F32):
        """In-place sum over all ranks of `count` elements at a device pointer of this GPU."""
        self._ck(self.lib.b2_allreduce(self._h, dev_ptr, count, dtype))

    def allreduce_bench(self, count, dtype=K.DTYPE_F32, warmup=3, iters=10):
        ms, cs = C.c_double(), C.c_double()
        self._ck(self.lib.b2_allreduce_bench(self._h, count, dtype, warmup, iters, C.byref(ms), C.byref(cs)))
        return ms.value, cs.value

    def collective_bench(self, kind, count, dtype=K.DTYPE_F32, warmup=3, iters=10):
        """kind 0 allreduce, 1 reduce-scatter, 2 allgather; device ms per call."""
        ms, cs = C.c_double(), C.c_double()
        self._ck(self.lib.b2_collective_bench(self._h, kind, count, dtype, warmup, iters, C.byref(ms), C.byref(cs)))
        return ms.value

    def sgd_bench(self, nparams, grad_dtype=K.DTYPE_F32, with_bf16_copy=False, warmup=3, iters=20):
        """(device ms per launch, algorithmic bytes per launch) of the SGD kernel on cold data."""
        ms, by = C.c_double(), C.c_double()
        self._ck(self.lib.b2_sgd_bench(self._h, nparams, grad_dtype, int(with_bf16_copy), warmup, iters, C.byref(ms),
                                       C.byref(by)))
        return ms.value, by.value

    def set_timing(self, on):
        self._ck(self.lib.b2_set_timing(self._h, int(on)))

    def weights_fingerprint(self, l):
        v = C.c_ulonglong()
        self._ck(self.lib.b2_weights_fingerprint(self._h, l, C.byref(v)))
        return v.value

    def gemm_bench(self, form, m, n, k, precision, epilogue=K.EPI_NONE, out_dtype=K.DTYPE_F32, sms=0, warmup=3,
                   iters=20):
        """Device milliseconds per launch of one GEMM of the step alone (see b2_gemm_bench)."""
        ms = C.c_double()
        self._ck(self.lib.b2_gemm_bench(self._h, form, m, n, k, precision, epilogue, out_dtype, sms, warmup, iters,
                                        C.byref(ms)))
        return ms.value

    # -- peer-memory path for small gradient messages ------------------------
    def p2p_describe(self):
        buf = (C.c_char * K.P2P_DESC_BYTES)()
        self._ck(self.lib.b2_p2p_describe(self._h, buf))
        return bytes(buf)

    def p2p_connect(self, descs, max_bytes, wait_ms=None):
        """descs: every rank's p2p_describe() bytes, in rank order."""
        blob = b"".join(descs)
        buf = C.create_string_buffer(blob, len(blob))
        self._ck(self.lib.b2_p2p_connect(self._h, buf, max_bytes))
        if wait_ms is not None:
            self._ck(self.lib.b2_p2p_set_wait_ms(self._h, wait_ms))

    # -- metrics ----------------------------------------------------------
    def timing(self):
        ph = (C.c_double * (self.L * K.T_NUM))()
        ms, n = C.c_double(), C.c_longlong()
        self._ck(self.lib.b2_get_timing(self._h, ph, C.byref(ms), C.byref(n)))
        return np.array(ph[:]).reshape(self.L, K.T_NUM), ms.value, n.value

    def gemm_busy_ms(self):
        v = C.c_double()
        self._ck(self.lib.b2_get_gemm_busy_ms(self._h, C.byref(v)))
        return v.value

    def write_trace(self, path):
        self._ck(self.lib.b2_write_trace(self._h, str(path).encode()))

    def reset_timing(self):
        self._ck(self.lib.b2_reset_timing(self._h))

    def site_report(self):
        """(GEMM sites on the tensor-core kernel, sites on the CUDA-core kernel, reason of the first refusal)."""
        a, b = C.c_int(), C.c_int()
        buf = C.create_string_buffer(256)
        self._ck(self.lib.b2_site_report(self._h, C.byref(a), C.byref(b), buf, 256))
        return a.value, b.value, buf.value.decode()

    def launch_counts(self):
        a, b = C.c_longlong(), C.c_longlong()
        self._ck(self.lib.b2_launch_counts(self._h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def sync(self):
        self._ck(self.lib.b2_sync(self._h))


def pinned_array(shape, device=None, node_out=None):
    """A float32 numpy array over pinned host memory from b2_host_alloc (never freed
    explicitly: it lives as long as the process, which is how the benchmark uses it).
    With `device`, the pages come from the NUMA node of that GPU (b2_host_alloc_near);
    `node_out`, a list, then receives the node (-1: the system does not tell)."""
    n = int(np.prod(shape))
    p = C.c_void_p()
    if device is None:
        rc = K.lib().b2_host_alloc(C.byref(p), n * 4)
    else:
        node = C.c_int(-1)
        rc = K.lib().b2_host_alloc_near(C.byref(p), n * 4, int(device), C.byref(node))
        if node_out is not None:
            node_out.append(node.value)
    if rc != K.OK:
        raise K.B2Error(rc, K.lib().b2_last_error(None).decode())
    buf = (C.c_float * n).from_address(p.value)
    return np.frombuffer(buf, dtype=np.float32).reshape(shape)
