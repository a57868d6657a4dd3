"""The C-ABI library loads without a GPU and exports exactly what the header declares."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    with open(os.path.join(ROOT, "include", "b200mlp.h")) as f:
        text = re.sub(r"/\*.*?\*/", "", f.read(), flags=re.S)
    return sorted(set(re.findall(r"\b(b2_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(native):
    from tbb_test_b200 import _capi
    lib = _capi.lib()
    declared = header_functions()
    assert declared, "no declarations found in include/b200mlp.h"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert sorted(_capi.SYMBOLS) == declared, "ctypes binding and header disagree"


def test_config_defaults_and_struct_size(native):
    import ctypes as C
    from tbb_test_b200 import _capi as K
    cfg = K.Config()
    assert K.lib().b2_config_default(C.byref(cfg)) == K.OK
    assert (cfg.world_size, cfg.mode, cfg.precision) == (1, K.MODE_BASELINE, K.PREC_FP32)
    assert (cfg.allreduce, cfg.overlap, cfg.input_grad, cfg.comm_sms) == (1, 1, 1, -1)
    assert (cfg.ar_bucket_mb, cfg.shard_update) == (-1, -1)
    assert abs(cfg.lr - 0.01) < 1e-9
    assert K.lib().b2_version().startswith(b"b200mlp")


def test_create_fails_loudly_without_a_device(native):
    """No CPU fallback: on a machine without a GPU creating a handle is an error with
    a message, not a silent slow path."""
    from conftest import HAS_GPU
    if HAS_GPU:
        pytest.skip("a GPU is present")
    from tbb_test_b200 import _capi as K
    from tbb_test_b200.mlp import MLP
    with pytest.raises(K.B2Error) as e:
        MLP([16, 16], 8)
    assert e.value.code == K.ERR_CUDA
    assert "no CPU path" in str(e.value)


def test_argument_errors_come_before_any_device_work(native, monkeypatch):
    """Bad configurations are refused with their own codes (no GPU needed to see them),
    among them graph replay together with the gradient allreduce."""
    from tbb_test_b200 import _capi as K
    from tbb_test_b200.mlp import MLP
    monkeypatch.delenv("B2_GRAPH_WITH_ALLREDUCE", raising=False)
    with pytest.raises(K.B2Error) as e:
        MLP([16, 16], 8, world_size=2, rank=0, nccl_id=b"\0" * K.NCCL_ID_BYTES, use_graph=True)
    assert e.value.code == K.ERR_UNSUPPORTED and "use_graph" in str(e.value)
    for kw in (dict(world_size=2, rank=2, nccl_id=b"\0" * K.NCCL_ID_BYTES), dict(world_size=2, rank=0),
               dict(grad_bf16=True, precision=K.PREC_FP32)):
        with pytest.raises(K.B2Error) as e:
            MLP([16, 16], 8, **kw)
        assert e.value.code == K.ERR_INVALID, kw
    with pytest.raises(K.B2Error) as e:
        MLP([16, 0], 8)
    assert e.value.code == K.ERR_INVALID


def test_product_does_not_import_the_oracle():
    """The oracle is test infrastructure: nothing in the package may reach for it."""
    pkg = os.path.join(ROOT, "tbb_test_b200")
    for dirpath, _, files in os.walk(pkg):
        for fn in files:
            if fn.endswith((".py", ".cc", ".cu", ".h", ".cuh")):
                with open(os.path.join(dirpath, fn)) as f:
                    src = f.read()
                assert "oracle" not in src.lower().replace("# oracle", ""), os.path.join(dirpath, fn)
