"""mlp_cuda, the GPU counterpart of the reference's mlp_omp main: runs the self-check,
the training loop and prints timing and checksums in the reference's formats."""
import os
import re
import subprocess

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_mlp_cuda_reference_model_checksums(native, oracle):
    """Scaled copy of the reference run (widths ..., 1; REF mode; lr 1e-10): the printed
    l1 / l2 / trace of the final weights equal those of the oracle run from the same
    init_matrices() stream."""
    from tbb_test_b200 import build
    widths, batch, warm, iters = [256, 256, 256, 1], 256, 2, 6
    r = subprocess.run([build.DRIVER, "1", "8", "--widths", ",".join(map(str, widths)), "--batch", str(batch),
                        "--warmup", str(warm), "--iters", str(iters), "--precision", "fp32"],
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:]
    assert "wall clock time" in r.stdout and "[layer 0] fwd" in r.stdout
    sums = re.findall(r"layer (\d+) l1 (\S+) l2 (\S+) trace (\S+)", r.stdout)
    assert len(sums) == len(widths) - 1
    # the same job on the oracle: inputs U(0,1), weights U(-0.1,0.1) drawn row by row from stream 3
    pos = 0
    x = oracle.fill_uniform(batch, widths[0], 3, 0.0, 1.0, start=pos)
    pos += batch * widths[0]
    o = oracle.Oracle(widths, batch, mode=oracle.MODE_REF, lr=1e-10)
    for l in range(len(widths) - 1):
        w = oracle.fill_uniform(widths[l + 1], widths[l], 3, -0.1, 0.1, start=pos)
        pos += widths[l + 1] * widths[l]
        o.set_weights(l, w)
    o.set_input(x)
    o.step(warm + iters)
    for l, (idx, l1, l2, tr) in enumerate(sums):
        exp = oracle.checksum(o.weights(l))
        got = (float(l1), float(l2), float(tr))
        assert int(idx) == l
        assert np.allclose(got, exp, rtol=2e-5, atol=1e-6), (l, got, exp)  # %g prints 6 digits
    o.close()


def test_mlp_cuda_baseline_bf16_runs(native):
    from tbb_test_b200 import build
    r = subprocess.run([build.DRIVER, "1", "--widths", "512,512,512,512", "--batch", "512", "--warmup", "2",
                        "--iters", "5", "--precision", "bf16", "--mode", "baseline"],
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:]
    assert re.search(r"samples/s [0-9.e+]+", r.stdout)
    assert "nan" not in r.stdout.lower()


def _checksums(args):
    from tbb_test_b200 import build
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([build.DRIVER] + args, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                       timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-2000:]
    sums = re.findall(r"layer (\d+) l1 (\S+) l2 (\S+) trace (\S+)", r.stdout)
    return np.array([[float(v) for v in s[1:]] for s in sums]), r.stdout


@pytest.mark.parametrize("precision,rtol", [("fp32", 5e-5), ("bf16", 2e-3)])
def test_mlp_cuda_two_gpus_match_one(native, precision, rtol):
    """The same job on one GPU and split over two (one host thread per GPU, NCCL between them, the
    reference's allreduce self-check first): the gradient sum over the batch is the same, so the
    final weights of replica 0 agree up to summation order. The final download is a collective in
    BF16 precision (the fp32 master weights are gathered from the ranks that own them)."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    common = ["--widths", "384,512,256,128", "--batch", "512", "--warmup", "1", "--iters", "4",
              "--precision", precision, "--lr", "1e-5"]
    one, _ = _checksums(["1"] + common)
    two, out = _checksums(["2"] + common)
    assert one.shape == two.shape == (3, 3)
    assert "nan" not in out.lower()
    assert np.allclose(one, two, rtol=rtol, atol=40 * rtol), (one, two)
