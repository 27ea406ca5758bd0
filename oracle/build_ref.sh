#!/usr/bin/env bash
# TEST INFRASTRUCTURE -- not part of the shipped library.
#
# Builds the UNMODIFIED microsoft/RepDL reference into oracle/_ref/ so that the
# C restatement in this folder (and the CUDA kernels) can be checked against the
# reference's own CPU backend.  Nothing is copied into the repository: the
# sources are compiled from where they lie (the directory named by
# $REPDL_REFERENCE) through a scratch copy in the temp directory, because the
# reference's setup.py writes build/ next to itself and the tree may be read-only.
#
# Outputs (all git-ignored, all under oracle/_ref/):
#   site/repdl/...                    the reference Python package
#   site/repdl/backend/cpu*.so        reference CPU backend (backend/cpu/*.cpp)
#   site/repdl/backend/cuda*.so       reference CUDA backend compiled for sm_100a
#   refmath.so, refmath_cuda.so       12-line pybind shims exposing the reference's
#                                     exp2d/log1d (backend/cpu/math.cpp:19-47), which
#                                     backend/cpu/bind.cpp:6-19 does not export
set -euo pipefail
HERE="$(cd "$(dirname "$0")" && pwd)"
REF="${REPDL_REFERENCE:-}"
OUT="$HERE/_ref"
[ -n "$REF" ] && [ -d "$REF" ] || { echo "REPDL_REFERENCE does not name a reference tree; nothing to build"; exit 0; }
export CXX=/usr/bin/g++ CC=/usr/bin/gcc TORCH_CUDA_ARCH_LIST=10.0a MAX_JOBS="${MAX_JOBS:-8}"
mkdir -p "$OUT"
SCRATCH="$(mktemp -d /tmp/repdl_ref_build.XXXXXX)"
trap 'rm -rf "$SCRATCH"' EXIT
cp -r "$REF" "$SCRATCH/src"
if [ "${REF_SKIP_CUDA:-0}" = "1" ]; then
  # CPU backend only (30 s instead of 4 min): drop the CUDAExtension from the scratch copy.
  python - "$SCRATCH/src/setup.py" <<'PY'
import re, sys
p = sys.argv[1]; s = open(p).read()
s = re.sub(r"cpp_extension\.CUDAExtension\(.*?\),\n    \],", "],", s, flags=re.S)
open(p, "w").write(s)
PY
fi
python -m pip install --no-index --no-build-isolation --no-deps --upgrade \
    --target "$OUT/site" "$SCRATCH/src" 2>&1 | tail -3
python "$HERE/build_refmath.py"
echo "reference built into $OUT"
