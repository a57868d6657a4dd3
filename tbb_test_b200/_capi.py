"""ctypes binding of include/b200mlp.h (the C ABI of csrc/libb200mlp.so).

This is the binding a Python embedder writes against the header; the tests and
the benchmark call the library only through it.  There is no fallback: if the
shared library has not been built the import of `lib()` raises.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "csrc", "libb200mlp.so")

OK, ERR_INVALID, ERR_CUDA, ERR_NCCL, ERR_UNSUPPORTED, ERR_TIMEOUT, ERR_STATE = 0, -1, -2, -3, -4, -5, -6
MODE_REF, MODE_BASELINE = 0, 1
PREC_FP32, PREC_TF32, PREC_BF16, PREC_FP32_TC = 0, 1, 2, 3
DTYPE_F32, DTYPE_BF16 = 0, 1
EPI_NONE, EPI_RELU, EPI_MASK = 0, 1, 2
T_FWD, T_WGT_GRAD, T_BWD, T_WGT_UPDATE, T_ALLREDUCE, T_ALLGATHER, T_NUM = 0, 1, 2, 3, 4, 5, 6
NCCL_ID_BYTES = 128
P2P_DESC_BYTES = 128
NOALLOC_MAX_OPERAND_ELEMS = 4 * 1024 * 1024

_fp = C.POINTER(C.c_float)
_dp = C.POINTER(C.c_double)


class Config(C.Structure):
    _fields_ = [
        ("nlayers", C.c_int), ("nfeatures", C.POINTER(C.c_int)), ("batch", C.c_int), ("rank", C.c_int),
        ("world_size", C.c_int), ("device", C.c_int), ("mode", C.c_int), ("precision", C.c_int),
        ("grad_bf16", C.c_int), ("allreduce", C.c_int), ("overlap", C.c_int), ("input_grad", C.c_int),
        ("collect_timing", C.c_int), ("use_graph", C.c_int), ("force_simt", C.c_int), ("comm_sms", C.c_int), ("ar_bucket_mb", C.c_int), ("shard_update", C.c_int), ("lr", C.c_float),
        ("nccl_unique_id", C.c_void_p),
    ]


# every symbol include/b200mlp.h declares: name -> (restype, argtypes)
_H = C.c_void_p
SYMBOLS = {
    "b2_config_default": (C.c_int, [C.POINTER(Config)]),
    "b2_version": (C.c_char_p, []),
    "b2_nccl_unique_id": (C.c_int, [C.c_void_p]),
    "b2_create": (C.c_int, [C.POINTER(Config), C.POINTER(_H)]),
    "b2_destroy": (C.c_int, [_H]),
    "b2_last_error": (C.c_char_p, [_H]),
    "b2_batch_range": (C.c_int, [_H, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "b2_upload_weights": (C.c_int, [_H, C.c_int, _fp, C.c_size_t]),
    "b2_download_weights": (C.c_int, [_H, C.c_int, _fp, C.c_size_t]),
    "b2_upload_input": (C.c_int, [_H, _fp, C.c_size_t]),
    "b2_upload_target": (C.c_int, [_H, _fp, C.c_size_t]),
    "b2_download_activation": (C.c_int, [_H, C.c_int, _fp, C.c_size_t]),
    "b2_download_dz": (C.c_int, [_H, C.c_int, _fp, C.c_size_t]),
    "b2_download_input_grad": (C.c_int, [_H, _fp, C.c_size_t]),
    "b2_download_weight_grad": (C.c_int, [_H, C.c_int, _fp, C.c_size_t]),
    "b2_upload_weight_grad": (C.c_int, [_H, C.c_int, _fp, C.c_size_t]),
    "b2_set_lr": (C.c_int, [_H, C.c_float]),
    "b2_step": (C.c_int, [_H, C.c_int]),
    "b2_train_step_host": (C.c_int, [_H, _fp, C.c_size_t, _fp, C.c_size_t, _dp]),
    "b2_train_step_host_async": (C.c_int, [_H, _fp, C.c_size_t, _fp, C.c_size_t]),
    "b2_wait_loss": (C.c_int, [_H, _dp]),
    "b2_loss": (C.c_int, [_H, _dp]),
    "b2_host_alloc": (C.c_int, [C.POINTER(C.c_void_p), C.c_size_t]),
    "b2_host_alloc_near": (C.c_int, [C.POINTER(C.c_void_p), C.c_size_t, C.c_int, C.POINTER(C.c_int)]),
    "b2_host_free": (C.c_int, [C.c_void_p]),
    "b2_sgemm_host": (C.c_int, [_H, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _fp, C.c_size_t, _fp,
                                C.c_size_t, _fp, C.c_size_t, C.c_int, _fp, C.c_size_t]),
    "b2_sgemm": (C.c_int, [_H, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p,
                           C.c_size_t, C.c_void_p, C.c_size_t, C.c_float, C.c_void_p, C.c_size_t]),
    "b2_sync": (C.c_int, [_H]),
    "b2_gemm_bf16_noalloc": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_size_t,
                                       C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p]),
    "b2_noalloc_last_error": (C.c_char_p, []),
    "b2_allreduce_sgd": (C.c_int, [_H, C.c_int]),
    "b2_allreduce": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_int]),
    "b2_allreduce_bench": (C.c_int, [_H, C.c_size_t, C.c_int, C.c_int, C.c_int, _dp, _dp]),
    "b2_collective_bench": (C.c_int, [_H, C.c_int, C.c_size_t, C.c_int, C.c_int, C.c_int, _dp, _dp]),
    "b2_sgd_bench": (C.c_int, [_H, C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_int, _dp, _dp]),
    "b2_set_timing": (C.c_int, [_H, C.c_int]),
    "b2_weights_fingerprint": (C.c_int, [_H, C.c_int, C.POINTER(C.c_ulonglong)]),
    "b2_gemm_bench": (C.c_int, [_H, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                C.c_int, _dp]),
    "b2_p2p_describe": (C.c_int, [_H, C.c_void_p]),
    "b2_p2p_connect": (C.c_int, [_H, C.c_void_p, C.c_size_t]),
    "b2_p2p_emulate": (C.c_int, [C.c_int, C.c_int, C.POINTER(_fp), C.c_size_t]),
    "b2_p2p_emulate_opts": (C.c_int, [C.c_int, C.c_int, C.POINTER(_fp), C.c_size_t, C.c_int, C.c_int]),
    "b2_p2p_set_wait_ms": (C.c_int, [_H, C.c_int]),
    "b2_get_timing": (C.c_int, [_H, _dp, _dp, C.POINTER(C.c_longlong)]),
    "b2_get_gemm_busy_ms": (C.c_int, [_H, _dp]),
    "b2_reset_timing": (C.c_int, [_H]),
    "b2_write_trace": (C.c_int, [_H, C.c_char_p]),
    "b2_site_report": (C.c_int, [_H, C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_char_p, C.c_size_t]),
    "b2_launch_counts": (C.c_int, [_H, C.POINTER(C.c_longlong), C.POINTER(C.c_longlong)]),
}

_lib = None


def lib():
    """The loaded shared library with argument types set; raises if it is missing."""
    global _lib
    if _lib is None:
        path = os.environ.get("B2_LIB_PATH", LIB_PATH)  # override: A/B runs of two builds
        if not os.path.exists(path):
            raise ImportError(
                f"{path} is missing: build it with `python -m tbb_test_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        if "B2_NCCL_PATH" not in os.environ:
            # prefer the NCCL wheel of this interpreter (the one PyTorch itself loads) over a
            # system copy; the library falls back to the loader's search path without it
            import importlib.util
            spec = importlib.util.find_spec("nvidia")
            for base in (spec.submodule_search_locations if spec else []):
                cand = os.path.join(base, "nccl", "lib", "libnccl.so.2")
                if os.path.exists(cand):
                    os.environ["B2_NCCL_PATH"] = cand
                    break
        L = C.CDLL(path, mode=C.RTLD_GLOBAL)
        for name, (res, args) in SYMBOLS.items():
            if path != LIB_PATH and not hasattr(L, name):
                continue
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


class B2Error(RuntimeError):
    def __init__(self, code, text):
        super().__init__(f"b200mlp error {code}: {text}")
        self.code = code
