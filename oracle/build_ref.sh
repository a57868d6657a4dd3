#!/usr/bin/env bash
# Builds the checker-side binaries of the oracle directory.
#
#   oracle/liboracle.so            the C restatement (mlp_oracle.c)
#   oracle/_ref/mlp_omp            the UNMODIFIED reference benchmark
#   oracle/_ref/libref_mlp_omp.so  the same sources with main renamed + ref_harness.cc
#   oracle/_ref/mlp_omp_<cfg>      the reference with only its compile-time workload
#                                  literals replaced (layer widths, batch; the iteration
#                                  counts NWARMUP/NITER become run-time values read from
#                                  B2_REF_NWARMUP / B2_REF_NITER), used to time the
#                                  reference's CPU path on the benchmark configurations
#
# The reference sources are compiled from where they lie (the directory named by
# $REF, default: a directory "reference" next to the repository); nothing of them
# is written into the repository.  The patched
# variants are produced in a temporary directory that is removed afterwards.
# Without $REF only liboracle.so is built (the _ref binaries then have to be the
# prebuilt ones).
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REF="${REF:-$here/../../reference}"
out="$here/_ref"
CC="${B2_CC:-/usr/bin/gcc}"   # the environment's $CC may point at a toolchain without libgomp
CXX="${B2_CXX:-/usr/bin/g++}"

$CC -O3 -mavx2 -mfma -fopenmp -fPIC -shared -std=gnu99 -Wall -o "$here/liboracle.so" \
  "$here/mlp_oracle.c" -lm
echo "built $here/liboracle.so"

if [ ! -f "$REF/mlp_omp.cc" ]; then
  echo "reference sources not found at $REF: skipping oracle/_ref"
  exit 0
fi
mkdir -p "$out"
# OpenBLAS as shipped inside the scipy wheel of the interpreter on PATH ($B2_OPENBLAS_PATH overrides)
blas_default="${B2_OPENBLAS_PATH:-$(python3 - <<'PY' 2>/dev/null || true
import glob, importlib.util, os
spec = importlib.util.find_spec("scipy")
hits = sorted(glob.glob(os.path.join(os.path.dirname(os.path.dirname(spec.origin)), "scipy.libs",
                                     "libscipy_openblas-*.so"))) if spec else []
print(hits[0] if hits else "")
PY
)}"
flags=(-std=c++11 -O3 -DNDEBUG -mavx2 -mfma -mavx512f -fopenmp -fPIC -w
       -I "$here/ref_shim" -I "$REF" "-DB2_OPENBLAS_DEFAULT=\"$blas_default\"")
common=("$REF/Partition.cc" "$REF/Rand.cc" "$REF/TwistedHyperCube.cc" "$here/ref_shim/mkl_shim.cc")

$CXX "${flags[@]}" -o "$out/mlp_omp" "$REF/mlp_omp.cc" "$REF/mlp_bench_common.cc" "${common[@]}" -ldl
echo "built $out/mlp_omp"
$CXX "${flags[@]}" -Dmain=mlp_omp_main -shared -o "$out/libref_mlp_omp.so" "$REF/mlp_omp.cc" \
  "$REF/mlp_bench_common.cc" "${common[@]}" "$here/ref_harness.cc" -ldl
echo "built $out/libref_mlp_omp.so"

# name | layer widths | global batch | default warm-up | default timed iterations
variants=(
  "c1|1024, 1024, 1024, 1024, 1024, 1024|1024|2|8"
  "c3|$(python3 -c 'print(", ".join(["512"]*21))')|2048|2|8"
  "c4|$(python3 -c 'print(", ".join(["4096"]*9))')|8192|1|2"
)
for v in "${variants[@]}"; do
  IFS='|' read -r name widths batch nwarm niter <<<"$v"
  tmp="$(mktemp -d)"
  sed -e "s/^constexpr int nfeatures\[\] = .*/constexpr int nfeatures[] = {$widths};/" \
      -e "s/constexpr int NWARMUP = 16, NITER = 256;/static const int NWARMUP = getenv(\"B2_REF_NWARMUP\") ? atoi(getenv(\"B2_REF_NWARMUP\")) : $nwarm, NITER = getenv(\"B2_REF_NITER\") ? atoi(getenv(\"B2_REF_NITER\")) : $niter;/" \
      "$REF/mlp_bench_common.h" >"$tmp/mlp_bench_common.h"
  sed -e "s/int batch_size = 1024 \* nsockets;.*/int batch_size = $batch;/" \
      "$REF/mlp_omp.cc" >"$tmp/mlp_omp.cc"
  cp "$REF/mlp_bench_common.cc" "$tmp/mlp_bench_common.cc"
  if cmp -s "$REF/mlp_bench_common.h" "$tmp/mlp_bench_common.h" || cmp -s "$REF/mlp_omp.cc" "$tmp/mlp_omp.cc"; then
    echo "workload literals not found in the reference sources" >&2
    rm -rf "$tmp"
    exit 1
  fi
  $CXX "${flags[@]}" -include cstdlib -I "$tmp" -o "$out/mlp_omp_$name" "$tmp/mlp_omp.cc" "$tmp/mlp_bench_common.cc" \
    "${common[@]}" -ldl
  rm -rf "$tmp"
  echo "built $out/mlp_omp_$name (widths {$widths}, batch $batch, default $nwarm+$niter iterations)"
done
