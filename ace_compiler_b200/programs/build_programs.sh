#!/usr/bin/env bash
# Builds compiled-program binaries for the B200 runtime: run_program.c plus one
# file emitted by the ANT-ACE compiler.
#
# usage: build_programs.sh <generated.c|.inc> <output name>
#        build_programs.sh                    (the programs committed in the
#                                              reference checkout, when present)
# Binaries go to programs/_ref/ (not tracked).  A generated file is compiled as
# it is; nothing is copied out of the reference tree.
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
PKG="$(dirname "$HERE")"
REPO="$(dirname "$PKG")"
LIB="$PKG/libFHErt_b200.so"
OUT="$HERE/_ref"
[ -f "$LIB" ] || { echo "build the CUDA library first" >&2; exit 1; }
mkdir -p "$OUT"

build_one() {  # $1 generated file, $2 name
  # the host code of a generated file is only glue: no optimisation needed
  gcc -O0 -w -Werror=implicit-function-declaration -I"$REPO/include" \
      -include "$REPO/include/common/rtlib.h" -x c -c "$1" -o "$OUT/$2.o"
  gcc -O2 -I"$REPO/include" "$HERE/run_program.c" "$OUT/$2.o" -o "$OUT/$2" "$LIB" -lm \
      -Wl,-rpath,'$ORIGIN/../..'
  # the same program as a shared object, for hosts that drive it in-process
  gcc -O0 -w -fPIC -shared -I"$REPO/include" -include "$REPO/include/common/rtlib.h" \
      -x c "$1" -x none -o "$OUT/$2.so" "$LIB" -lm -Wl,-rpath,'$ORIGIN/../..'
  rm -f "$OUT/$2.o"
  echo "built $OUT/$2 and $OUT/$2.so"
}

if [ $# -ge 2 ]; then
  build_one "$1" "$2"
  exit 0
fi
DATASET="${REFERENCE_ROOT:-}/fhe-cmplr/rtlib/ant/dataset"
if [ -z "${REFERENCE_ROOT:-}" ] || [ ! -d "$DATASET" ]; then
  echo "REFERENCE_ROOT names no reference checkout; keeping any prebuilt programs in $OUT" >&2
  exit 0
fi
for name in resnet20_cifar10 resnet32_cifar10 resnet32_cifar100 resnet44_cifar10 resnet110_cifar10; do
  src="$DATASET/${name}_pre.onnx.inc"
  [ -f "$src" ] && build_one "$src" "$name" || true
done
