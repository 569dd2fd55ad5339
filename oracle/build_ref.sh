#!/usr/bin/env bash
# Builds the UNMODIFIED-ALGORITHM reference (ThunderGBM) for sm_100a into oracle/_ref/.
#
# This is test infrastructure: the resulting library and harness are only ever
# executed by tests, by the golden-vector generator and as a timing baseline.
# Nothing under oracle/_ref/ is tracked by git; reference sources are never
# copied into the repository -- a scratch copy under $TMPDIR receives the two
# mechanical build fixes below and only binaries are written to oracle/_ref/.
#
# Build fixes (no algorithmic change):
#   1. src/thundergbm/syncmem.cpp: the vendored allocator calls mutex.Lock()/
#      Unlock(), the toolkit's CUB allocator uses std::mutex (lock()/unlock()).
#   2. src/thundergbm/builder/*.cu: bare `cuda::par` is ambiguous with libcu++'s
#      ::cuda namespace under CUDA 12.x -> `thrust::cuda::par`.
#
# Usage: oracle/build_ref.sh [reference_dir]     (default: $TGBM_REFERENCE_DIR, else a checkout named `reference`
#                                                 beside this repository)
set -euo pipefail
HERE=$(cd "$(dirname "$0")" && pwd)
REF=${1:-${TGBM_REFERENCE_DIR:-$HERE/../../reference}}
OUT=$HERE/_ref
if [ ! -d "$REF/src/thundergbm" ]; then
  echo "reference tree not found at $REF; keeping prebuilt $OUT if any" >&2
  exit 0
fi
WORK=$(mktemp -d "${TMPDIR:-/tmp}/tgbm_ref_build.XXXXXX")
trap 'rm -rf "$WORK"' EXIT
mkdir -p "$OUT/lib" "$OUT/bin" "$WORK/obj" "$WORK/inc"
cp -r "$REF/src" "$REF/include" "$WORK/"
chmod -R u+w "$WORK"
sed -i 's/mutex\.Lock()/mutex.lock()/g; s/mutex\.Unlock()/mutex.unlock()/g' "$WORK/src/thundergbm/syncmem.cpp"
grep -rl 'cuda::par' "$WORK/src" | xargs sed -i 's/\([^:A-Za-z_]\)cuda::par/\1thrust::cuda::par/g'
echo '/* #undef DATASET_DIR */' > "$WORK/inc/config.h"

NVCC=${NVCC:-/usr/local/cuda/bin/nvcc}
FLAGS="-std=c++17 -O2 -gencode arch=compute_100a,code=sm_100a --expt-extended-lambda --default-stream per-thread \
 -Xcompiler -fopenmp,-fPIC -DELPP_FEATURE_PERFORMANCE_TRACKING -DELPP_THREAD_SAFE -DELPP_STL_LOGGING \
 -DELPP_NO_LOG_TO_FILE -I$WORK/include -I$WORK/inc -w"

cd "$WORK"
SRCS=$(find src/thundergbm -name '*.cu' -o -name '*.cpp' | grep -v -e thundergbm_train.cpp -e thundergbm_predict.cpp | sort)
printf '%s\n' $SRCS | xargs -P "$(nproc)" -I{} sh -c \
  "$NVCC $FLAGS -x cu -c {} -o obj/\$(echo {} | tr '/' '_').o"
$NVCC -shared -gencode arch=compute_100a,code=sm_100a -Xcompiler -fopenmp obj/*.o -lcusparse -lgomp -o "$OUT/lib/libthundergbm.so"
$NVCC $FLAGS -x cu src/thundergbm/thundergbm_train.cpp -L"$OUT/lib" -lthundergbm -lgomp \
  -Xlinker -rpath -Xlinker '$ORIGIN/../lib' -o "$OUT/bin/thundergbm-train"
$NVCC $FLAGS -x cu src/thundergbm/thundergbm_predict.cpp -L"$OUT/lib" -lthundergbm -lgomp \
  -Xlinker -rpath -Xlinker '$ORIGIN/../lib' -o "$OUT/bin/thundergbm-predict"
# The golden-vector harness is our own code; it only includes the reference's public headers.
if [ -f "$HERE/ref_harness.cu" ]; then
  $NVCC $FLAGS "$HERE/ref_harness.cu" -L"$OUT/lib" -lthundergbm -lgomp \
    -Xlinker -rpath -Xlinker '$ORIGIN/../lib' -o "$OUT/bin/ref_harness"
fi
echo "reference built into $OUT"
