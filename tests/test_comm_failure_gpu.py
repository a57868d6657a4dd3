"""A communicator that fails under the job: reported, aborted, not waited on.

The reference has no failure handling (its flag waits spin for ever, mlp_omp.cc:120-121). Here a
step polls the communicator for asynchronous errors after it has drained; a reported error comes
back as B2_ERR_NCCL and the communicator is aborted so that no later call can block on it. The
failure is made on the host: a stand-in libnccl (tests/fake/fake_nccl.c) whose collectives do
nothing and whose error query starts reporting a lost peer after a given number of polls. One
GPU, nothing faults or hangs on the device."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_async_error_of_the_communicator_is_reported_and_the_communicator_aborted(native, tmp_path):
    so = tmp_path / "libfake_nccl.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-o", str(so), os.path.join(ROOT, "tests", "fake", "fake_nccl.c")],
                   check=True)
    flag = tmp_path / "aborted"
    child = textwrap.dedent(f"""
        import sys
        sys.path.insert(0, {ROOT!r})
        from tbb_test_b200 import _capi as K
        from tbb_test_b200.mlp import MLP, nccl_unique_id
        m = MLP([64, 64, 64], 32, rank=0, world_size=2, nccl_id=nccl_unique_id())
        m.step(1)                      # poll 1: healthy
        try:
            m.step(1)                  # poll 2: the stand-in reports a lost peer
        except K.B2Error as e:
            assert e.code == K.ERR_NCCL and "asynchronous error" in str(e), str(e)
        else:
            raise SystemExit("no error reported")
        try:
            m.step(1)                  # the communicator is gone: an error, not a hang
        except K.B2Error as e:
            assert e.code in (K.ERR_NCCL, K.ERR_STATE), str(e)
        else:
            raise SystemExit("a step on an aborted communicator succeeded")
        m.close()
        print("child ok")
    """)
    env = dict(os.environ, B2_NCCL_PATH=str(so), FAKE_NCCL_FAIL_AFTER="1", FAKE_NCCL_ABORT_FILE=str(flag))
    r = subprocess.run([sys.executable, "-c", child], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                       text=True, timeout=120)
    assert r.returncode == 0 and "child ok" in r.stdout, r.stdout[-2000:]
    assert flag.exists(), "ncclCommAbort was not called"
