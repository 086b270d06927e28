#!/usr/bin/env bash
# TEST INFRASTRUCTURE ONLY.
#
# Compiles the reference's example programs (fhe-cmplr/rtlib/ant/example:
# a hand-written driver plus the body the compiler emitted for one operator)
# from the read-only reference checkout, unchanged, against this repository's
# headers, and links them with the B200 library.  The binaries land in
# oracle/_ref/examples/ and are run by the GPU tests: each one encrypts its
# input, runs its Main_graph through the C-ABI, decrypts and compares with the
# values its author expected.  Nothing is copied out of the reference tree.
#
# usage: oracle/build_examples.sh [reference-root]   (default /root/reference)
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REPO="$(dirname "$HERE")"
REF="${1:-/root/reference}"
EG="$REF/fhe-cmplr/rtlib/ant/example"
OUT="$HERE/_ref/examples"
if [ ! -d "$EG" ]; then
  echo "reference checkout not found at $REF; keeping any prebuilt $OUT" >&2
  exit 0
fi
LIB="$REPO/ace_compiler_b200/libFHErt_b200.so"
[ -f "$LIB" ] || { echo "build the CUDA library first" >&2; exit 1; }
mkdir -p "$OUT"
built=0; skipped=()
for src in "$EG"/eg_fhertlib_*.c; do
  name="$(basename "$src" .c)"
  if gcc -O1 -w -Werror=implicit-function-declaration -I"$REPO/include" -I"$EG" \
       "$src" -o "$OUT/$name" "$LIB" -lm \
       -Wl,-rpath,'$ORIGIN/../../../ace_compiler_b200' 2> "$OUT/$name.log"; then
    built=$((built + 1)); rm -f "$OUT/$name.log"
  else
    skipped+=("$name"); rm -f "$OUT/$name"
  fi
done
echo "built $built example programs in $OUT; not built: ${skipped[*]:-none}"
