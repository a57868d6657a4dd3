"""b2_gemm_bf16_noalloc: the GEMM entry point for callers that may not allocate.

Some embedders cannot let a library call cudaMalloc: they have given all device
memory to their own pool, or they sit on a path where the device-wide
synchronisation of cudaMalloc/cudaFree is not acceptable. This test plays such a
caller - the device buffers come from PyTorch's caching allocator, the library is
only handed pointers - and checks the entry point, called through the C ABI twice
in a row on different data (the fixed scratch array is reused and keeps the first
call's contents), against the allocating entry point b2_sgemm_host on the same
inputs. Collected last on purpose: a failure here must not hide other tests.
"""
import ctypes as C

import numpy as np
import pytest

from helpers import rel_fro

pytestmark = pytest.mark.gpu

TOL = 5e-5  # same as the bf16 / fp32-output GEMM tests: only the fp32 add order may differ


def test_noalloc_gemm_matches_allocating_entry_point_twice(native, oracle):
    import torch
    from tbb_test_b200 import _capi as K
    from tbb_test_b200.mlp import MLP
    lib = K.lib()
    dev = MLP([16, 16], 16)
    cases = [((False, True), (384, 320, 200), 7), ((True, False), (256, 512, 1024), 9)]
    for (ta, tb), (m, n, k), seed in cases:
        a = oracle.fill_uniform(k if ta else m, m if ta else k, seed, -1.0, 1.0)
        b = oracle.fill_uniform(n if tb else k, k if tb else n, seed + 1, -1.0, 1.0)
        want = dev.sgemm_host(K.PREC_BF16, ta, tb, a, b)
        ta_d = torch.from_numpy(a).cuda()
        tb_d = torch.from_numpy(b).cuda()
        tc_d = torch.full((m, n), float("nan"), device="cuda", dtype=torch.float32)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        rc = lib.b2_gemm_bf16_noalloc(int(ta), int(tb), m, n, k, ta_d.data_ptr(), a.shape[1], tb_d.data_ptr(),
                                      b.shape[1], tc_d.data_ptr(), n, None)
        assert rc == K.OK, lib.b2_noalloc_last_error()
        if seed != cases[0][2]:  # the first call on a device may load the kernels' module; later ones hold nothing new
            assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
        got = tc_d.cpu().numpy()
        assert rel_fro(got, want) <= TOL
        ref = oracle.sgemm(ta, tb, oracle.round_bf16(a), oracle.round_bf16(b))
        assert rel_fro(got, ref) <= TOL
    dev.close()


def test_noalloc_gemm_rejects_operands_beyond_the_fixed_scratch(native):
    import torch
    from tbb_test_b200 import _capi as K
    lib = K.lib()
    m, n, k = 4096, 256, 2048  # op(A) has 8 Mi elements: twice the limit
    assert m * k > K.NOALLOC_MAX_OPERAND_ELEMS
    a = torch.zeros((m, k), device="cuda")
    b = torch.zeros((k, n), device="cuda")
    c = torch.zeros((m, n), device="cuda")
    rc = lib.b2_gemm_bf16_noalloc(0, 0, m, n, k, a.data_ptr(), k, b.data_ptr(), n, c.data_ptr(), n, None)
    assert rc == K.ERR_UNSUPPORTED
    assert b"at most" in lib.b2_noalloc_last_error()
    assert lib.b2_gemm_bf16_noalloc(0, 0, 0, n, k, a.data_ptr(), k, b.data_ptr(), n, c.data_ptr(), n, None) == K.ERR_INVALID
    # a stored row length that is not a multiple of 8 elements cannot be repacked for TMA
    assert lib.b2_gemm_bf16_noalloc(0, 0, 64, 64, 100, a.data_ptr(), 100, b.data_ptr(), 64, c.data_ptr(), 64,
                                    None) == K.ERR_UNSUPPORTED
    assert b"not served" in lib.b2_noalloc_last_error()
