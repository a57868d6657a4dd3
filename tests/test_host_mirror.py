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
