"""The C++ host mirror (Partition, TwistedHyperCube, ring tables, Matrix layout,
init_matrices) against golden tables produced by the reference's own functions."""
import ctypes as C
import json
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def host(native):
    from tbb_test_b200 import build
    L = C.CDLL(build.HOST_LIB)
    ip = C.POINTER(C.c_int)
    L.b2h_get_partition.argtypes = [C.c_int] * 5 + [ip]
    L.b2h_intra_socket_2d.argtypes = [C.c_int, C.c_int, C.c_double, C.c_int, C.c_int, C.c_int, ip]
    L.b2h_2dpartition.argtypes = [C.c_int, C.c_int, C.c_int, C.c_double, C.c_int, C.c_int, C.c_int, C.c_int, ip]
    L.b2h_hypercube.argtypes = [C.c_int] * 5 + [ip]
    L.b2h_ring_info.argtypes = [C.c_int] * 3 + [ip]
    L.b2h_matrix_layout.argtypes = [C.c_int, C.c_int, ip, ip, C.POINTER(C.c_longlong)]
    return L


@pytest.fixture(scope="module")
def gold():
    with open(os.path.join(GOLD, "partition_topology.json")) as f:
        return json.load(f)


def _call(fn, n, *args):
    out = (C.c_int * n)()
    fn(*args, out)
    return list(out)


def test_get_partition(host, gold):
    for nsock, work, sid, nthr, tid, b, e in gold["get_partition"]:
        assert _call(host.b2h_get_partition, 2, nsock, work, sid, nthr, tid) == [b, e]


def test_intra_socket_2d_partition(host, gold):
    for m, n, ar, m_align, nthr, tid, *exp in gold["intra_socket_2d"]:
        got = _call(host.b2h_intra_socket_2d, 4, m, n, ar, m_align, nthr, tid)
        assert got == exp, (m, n, ar, m_align, nthr, tid)


def test_2d_partition(host, gold):
    for nsock, m, n, ar, m_align, sid, nthr, tid, *exp in gold["partition_2d"]:
        got = _call(host.b2h_2dpartition, 4, nsock, m, n, ar, m_align, sid, nthr, tid)
        assert got == exp, (nsock, m, n, ar, m_align, sid, nthr, tid)


def test_hypercube_tables(host, gold):
    for twisted, n, shift, node, dim, *exp in gold["hypercube"]:
        assert _call(host.b2h_hypercube, 3, twisted, n, shift, node, dim) == exp, (twisted, n, shift, node, dim)


def test_hypercube_is_a_valid_halving_schedule(host):
    """Every dimension pairs the nodes up, and after all halving steps each node owns
    a distinct chunk - the property an allreduce schedule needs (shift 2 of the
    8-node twisted cube is the reference's known-inconsistent case and is left out)."""
    for twisted in (0, 1):
        for n, dims in ((2, 1), (4, 2), (8, 3)):
            for shift in range(dims):
                if twisted and n == 8 and shift == 2:
                    continue
                for dim in range(dims):
                    peers = [_call(host.b2h_hypercube, 3, twisted, n, shift, i, dim)[0] for i in range(n)]
                    assert sorted(peers) == list(range(n))
                    assert all(peers[peers[i]] == i and peers[i] != i for i in range(n))
                owned = [_call(host.b2h_hypercube, 3, twisted, n, shift, i, 0)[1] for i in range(n)]
                assert sorted(owned) == list(range(n))


def _cube_allreduce(host, twisted, n, shift, bufs, threaded):
    fp = C.POINTER(C.c_float)
    arr = (fp * n)(*[b.ctypes.data_as(fp) for b in bufs])
    host.b2h_hypercube_allreduce.restype = C.c_int
    host.b2h_hypercube_allreduce.argtypes = [C.c_int, C.c_int, C.c_int, C.POINTER(fp), C.c_size_t, C.c_int]
    return host.b2h_hypercube_allreduce(twisted, n, shift, arr, bufs[0].size, int(threaded))


@pytest.mark.parametrize("threaded", [False, True])
def test_hypercube_allreduce_data_path(host, threaded):
    """Recursive halving + doubling driven by Peer / RecvLocation / SendLocation sums the
    buffers of all nodes into every node: exact on small integers (any summation order),
    for lengths that do and do not divide by the node count, the empty buffer included."""
    rng = np.random.default_rng(5)
    for twisted in (0, 1):
        for n, dims in ((2, 1), (4, 2), (8, 3)):
            for shift in range(dims):
                if twisted and n == 8 and shift == 2:
                    continue
                for count in (0, 1, n - 1, n, 1000, 4099):
                    bufs = [rng.integers(-50, 50, count).astype(np.float32) for _ in range(n)]
                    want = np.sum(bufs, axis=0, dtype=np.float64).astype(np.float32)
                    assert _cube_allreduce(host, twisted, n, shift, bufs, threaded) == 1
                    for b in bufs:
                        assert np.array_equal(b, want), (twisted, n, shift, count)


def test_hypercube_allreduce_is_deterministic_and_close_on_reals(host):
    """On real data every node ends with bit-identical values (each chunk is summed once,
    by its owner, and copied), within float rounding of the exact sum."""
    rng = np.random.default_rng(6)
    n, count = 8, 6000
    src = [rng.uniform(-1, 1, count).astype(np.float32) for _ in range(n)]
    runs = []
    for threaded in (False, True):
        bufs = [b.copy() for b in src]
        assert _cube_allreduce(host, 1, n, 1, bufs, threaded) == 1
        assert all(np.array_equal(bufs[0], b) for b in bufs[1:])
        runs.append(bufs[0])
    assert np.array_equal(runs[0], runs[1])
    assert np.abs(runs[0] - np.sum(src, axis=0, dtype=np.float64)).max() <= 1e-5  # mlp_omp.cc:360 bound


def test_hypercube_allreduce_refuses_the_inconsistent_schedule(host):
    """Shift 2 of the 8-node twisted cube sends and receives the same location in
    dimensions 1 and 2; the data path refuses it and leaves the buffers alone."""
    bufs = [np.full(64, i, np.float32) for i in range(8)]
    assert _cube_allreduce(host, 1, 8, 2, bufs, False) == 0
    assert all(np.array_equal(b, np.full(64, i, np.float32)) for i, b in enumerate(bufs))


def test_hypercube_steps_follow_the_golden_tables(host, gold):
    """The step list a device implementation would execute: halving from the highest
    dimension down (reading the range the node keeps), doubling upwards (reading the
    range the peer finished), peers and locations as in the reference's tables."""
    table = {(t, n, s, i, d): exp for t, n, s, i, d, *exp in gold["hypercube"]}
    host.b2h_hypercube_steps.restype = C.c_int
    for (t, n, s) in sorted({k[:3] for k in table}):
        if t and n == 8 and s == 2:
            continue
        dims = n.bit_length() - 1
        for i in range(n):
            out = (C.c_int * (5 * 2 * dims))()
            assert host.b2h_hypercube_steps(t, n, s, i, out, 2 * dims) == 2 * dims
            steps = [tuple(out[5 * k:5 * k + 5]) for k in range(2 * dims)]
            for k, d in enumerate(range(dims - 1, -1, -1)):
                peer, recv, _send = table[(t, n, s, i, d)]
                assert steps[k] == (d, peer, recv, 1 << d, 1)
            for k, d in enumerate(range(dims)):
                peer = table[(t, n, s, i, d)][0]
                assert steps[dims + k] == (d, peer, table[(t, n, s, peer, d)][1], 1 << d, 0)


def test_ring_info(host, gold):
    for nsock, sid, task, *exp in gold["ring_info"]:
        assert _call(host.b2h_ring_info, 3, nsock, sid, task) == exp


def test_matrix_layout(host):
    ld, al, off = C.c_int(), C.c_int(), C.c_longlong()
    host.b2h_matrix_layout(1024, 1024, C.byref(ld), C.byref(al), C.byref(off))
    assert ld.value == 1040 and al.value == 1 and off.value == 1023 * 1040 + 1023
    host.b2h_matrix_layout(7, 1, C.byref(ld), C.byref(al), C.byref(off))
    assert ld.value == 17 and al.value == 1 and off.value == 6 * 17


def test_init_matrices_draws_the_pinned_stream(host, oracle):
    """init_matrices() (inputs U(0,1), weights U(-0.1,0.1), replicas copied) consumes
    the counter-based stream exactly like the stand-in used to build the reference."""
    nf, batch, nsock = [24, 16, 8], 10, 2
    x = np.zeros((batch, nf[0]), np.float32)
    ws = [np.zeros((nsock * nf[l + 1], nf[l]), np.float32) for l in range(2)]
    arr = (C.POINTER(C.c_float) * 2)(*[w.ctypes.data_as(C.POINTER(C.c_float)) for w in ws])
    host.b2h_init_matrices(2, (C.c_int * 3)(*nf), batch, nsock, x.ctypes.data_as(C.POINTER(C.c_float)), arr)
    pos = 0
    assert np.array_equal(x, oracle.fill_uniform(batch, nf[0], 3, 0.0, 1.0, start=pos))
    pos += batch * nf[0]
    for l in range(2):
        exp = oracle.fill_uniform(nf[l + 1], nf[l], 3, -0.1, 0.1, start=pos)
        pos += nf[l + 1] * nf[l]
        assert np.array_equal(ws[l][:nf[l + 1]], exp)
        assert np.array_equal(ws[l][nf[l + 1]:], exp)


def _plan(host, layer_bytes, world, bucket_mb, growth=0.0, allreduce=1):
    n = len(layer_bytes)
    low, high = (C.c_int * n)(), (C.c_int * n)()
    host.b2h_plan_buckets.argtypes = [C.POINTER(C.c_size_t), C.c_int, C.c_int, C.c_int, C.c_int, C.c_double,
                                      C.POINTER(C.c_int), C.POINTER(C.c_int)]
    host.b2h_plan_buckets((C.c_size_t * n)(*layer_bytes), n, world, allreduce, bucket_mb, growth, low, high)
    return list(low), list(high)


def test_gradient_bucket_rule(host):
    """The rule the library applies to group layers into one collective: equal quarter-size
    buckets on 2 GPUs, growing ones on 4 or more, one layer per bucket on request or when there
    is nothing to sum; every layer belongs to exactly one bucket of consecutive layers."""
    mib = 1 << 20
    c4 = [64 * mib] * 8
    assert _plan(host, c4, 2, -1) == ([0, 0, 2, 2, 4, 4, 6, 6], [1, 1, 3, 3, 5, 5, 7, 7])
    assert _plan(host, c4, 4, -1) == ([0, 0, 0, 3, 3, 3, 6, 6], [2, 2, 2, 5, 5, 5, 7, 7])
    assert _plan(host, c4, 8, -1) == _plan(host, c4, 4, -1)
    assert _plan(host, c4, 8, -1, growth=1.0) == _plan(host, c4, 2, -1)
    assert _plan(host, c4, 8, 0) == (list(range(8)), list(range(8)))
    assert _plan(host, c4, 1, -1) == (list(range(8)), list(range(8)))
    assert _plan(host, c4, 8, -1, allreduce=0) == (list(range(8)), list(range(8)))
    assert _plan(host, c4, 8, 256) == ([0, 0, 0, 0, 4, 4, 4, 4], [3, 3, 3, 3, 7, 7, 7, 7])
    # the deep narrow model: 20 one-MiB layers, a quarter is 5 MiB
    low, high = _plan(host, [mib] * 20, 2, -1)
    assert sorted(set(zip(low, high))) == [(0, 4), (5, 9), (10, 14), (15, 19)]
    # the 4 MiB floor: 8 layers of 256 KiB make one bucket
    low, high = _plan(host, [mib // 4] * 8, 2, -1)
    assert set(zip(low, high)) == {(0, 7)}
    # ragged widths: consecutive, covering, ordered
    rag = [3 * mib, 70 * mib, mib, 9 * mib, 40 * mib]
    for world in (2, 4, 8):
        low, high = _plan(host, rag, world, -1)
        for l in range(len(rag)):
            assert low[l] <= l <= high[l]
            assert all(low[k] == low[l] and high[k] == high[l] for k in range(low[l], high[l] + 1))


def test_bench_reads_the_same_bucket_rule(host):
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench", os.path.join(os.path.dirname(__file__), "..", "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    mib = 1 << 20
    assert bench.gradient_buckets([64 * mib] * 8, 2, -1) == [128 * mib] * 4
    assert bench.gradient_buckets([64 * mib] * 8, 4, -1) == [128 * mib, 192 * mib, 192 * mib]
    assert bench.gradient_buckets([64 * mib] * 8, 8, 0) == [64 * mib] * 8
