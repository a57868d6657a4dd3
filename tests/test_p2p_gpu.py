"""Peer-memory allreduce for small gradient messages, with all ranks emulated on one GPU
(one cooperative launch; the multi-GPU form of the same kernel is covered by
tests/test_multigpu_gpu.py)."""
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("count", [1, 3, 4, 31, 4096, 262144 + 5])
def test_emulated_ranks_sum_exactly_on_integers(native, world, count):
    """Small integers sum exactly in any order: every rank must end with the exact total,
    for lengths that do not divide by the rank count or by the vector width."""
    from tbb_test_b200.mlp import p2p_emulate
    rng = np.random.default_rng(world * 1000 + count)
    bufs = [rng.integers(-64, 64, count).astype(np.float32) for _ in range(world)]
    want = np.sum(bufs, axis=0, dtype=np.float64).astype(np.float32)
    got = p2p_emulate([b.copy() for b in bufs])
    for r in range(world):
        assert np.array_equal(got[r], want), (world, count, r)


def test_emulated_ranks_agree_bit_for_bit_on_reals(native, oracle):
    """Each element is summed once, in rank order, by its owner: all ranks hold the same bits,
    equal to a float32 running sum over the ranks in rank order."""
    from tbb_test_b200.mlp import p2p_emulate
    world, count = 8, 1 << 18  # the 1 MiB gradient of a 512 x 512 layer
    bufs = [oracle.fill_uniform(1, count, r, -1.0, 1.0).ravel() for r in range(world)]
    want = bufs[0].copy()
    for r in range(1, world):
        want += bufs[r]
    got = p2p_emulate([b.copy() for b in bufs])
    for r in range(world):
        assert np.array_equal(got[r], want), r


@pytest.mark.parametrize("world,lagging", [(2, 1), (4, 0), (8, 5)])
def test_a_rank_that_never_arrives_makes_every_wait_run_out(native, world, lagging):
    """The reference's flag waits spin without a limit (mlp_omp.cc:120-121,267-268). Here a
    rank that is one call behind never satisfies the others' waits: each wait gives up after
    the limit, the kernel returns, and the host gets B2_ERR_TIMEOUT instead of a hang. The
    failure is made on the host (a call counter one behind); the GPU stays usable."""
    from tbb_test_b200 import _capi as K
    from tbb_test_b200.mlp import p2p_emulate
    count = 4096
    bufs = [np.full(count, float(r + 1), np.float32) for r in range(world)]
    t0 = time.time()
    with pytest.raises(K.B2Error) as e:
        p2p_emulate([b.copy() for b in bufs], wait_ms=50, lagging_rank=lagging)
    assert e.value.code == K.ERR_TIMEOUT
    assert time.time() - t0 < 5.0
    # the device and the kernel are still good for the next call
    got = p2p_emulate([b.copy() for b in bufs], wait_ms=50)
    want = np.full(count, float(world * (world + 1) // 2), np.float32)
    for r in range(world):
        assert np.array_equal(got[r], want)
