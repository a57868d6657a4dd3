"""Data-parallel ranks on real GPUs (needs at least two; skipped otherwise): the
reference's known-answer test through NCCL and step parity against the oracle."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ngpus():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


@pytest.mark.parametrize("world", [2, 4, 8])
def test_data_parallel_ranks_match_the_oracle(native, oracle, world):
    if _ngpus() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29800 + world),
           os.path.join(ROOT, "tests", "_nccl_worker.py")]
    r = subprocess.run(cmd, env=env, cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                       timeout=600)
    if r.returncode != 0:  # show each rank's own traceback, not only the launcher's summary
        per_rank = [ln for ln in r.stdout.splitlines() if ln.startswith("[rank")]
        raise AssertionError("\n".join(per_rank[-60:]) or r.stdout[-3000:])
    assert r.stdout.count(": ok") == world
