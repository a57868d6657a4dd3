"""Times the GEMMs of one layer alone, per call form, at a given shape (one GPU).

    python -m tbb_test_b200.gemm_bench --batch 8192 --width 4096 [--precision bf16|tf32|fp32tc|fp32]
                                       [--forms fwd,wgrad,dgrad] [--iters 20] [--sms 0]
                                       [--grad-bf16]

Prints one JSON line per form: milliseconds per launch (CUDA events around back-to-back
launches on rotating operand sets larger than the L2), TFLOP/s (2*m*n*k) and the fraction
of the measured cuBLAS bf16 peak where that file is present.  The forms are those of the
training step: forward with the fused ReLU (operand-type output), weight gradient (fp32
or bf16 output), input gradient with the fused ReLU mask.  Also the command the ncu
summaries under profiles/ were captured with.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8192)
    ap.add_argument("--width", type=int, default=4096)
    ap.add_argument("--precision", default="bf16", choices=["bf16", "tf32", "fp32", "fp32tc"])
    ap.add_argument("--forms", default="fwd,wgrad,dgrad")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--sms", type=int, default=0)
    ap.add_argument("--grad-bf16", action="store_true")
    args = ap.parse_args()
    from tbb_test_b200 import _capi as K
    from tbb_test_b200.mlp import MLP
    prec = {"bf16": K.PREC_BF16, "tf32": K.PREC_TF32, "fp32": K.PREC_FP32, "fp32tc": K.PREC_FP32_TC}[args.precision]
    op = K.DTYPE_BF16 if args.precision == "bf16" else K.DTYPE_F32
    b, f = args.batch, args.width
    peak = None
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            peak = json.load(fh).get("bf16_tflops")
    except Exception:
        pass
    dev = MLP([16, 16], 16)
    for form in args.forms.split(","):
        if form == "fwd":
            fid, (m, n, k), epi, out = 0, (b, f, f), K.EPI_RELU, op
        elif form == "wgrad":
            fid, (m, n, k), epi, out = 1, (f, f, b), K.EPI_NONE, (K.DTYPE_BF16 if args.grad_bf16 else K.DTYPE_F32)
        elif form == "dgrad":
            fid, (m, n, k), epi, out = 2, (b, f, f), K.EPI_MASK, op
        else:
            raise SystemExit(f"unknown form {form}")
        ms = dev.gemm_bench(fid, m, n, k, prec, epi, out, args.sms, args.warmup, args.iters)
        tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        print(json.dumps({"form": form, "m": m, "n": n, "k": k, "precision": args.precision, "ms": round(ms, 5),
                          "tflops": round(tf, 1), "frac_of_measured_bf16_peak": round(tf / peak, 3) if peak else None,
                          "sms": args.sms or "all", "iters": args.iters}))
    dev.close()


if __name__ == "__main__":
    main()
