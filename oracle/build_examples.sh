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
# usage: oracle/build_examples.sh [reference-root]   (or REFERENCE_ROOT in the environment)
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REPO="$(dirname "$HERE")"
REF="${1:-${REFERENCE_ROOT:-}}"
EG="$REF/fhe-cmplr/rtlib/ant/example"
OUT="$HERE/_ref/examples"
if [ -z "$REF" ] || [ ! -d "$EG" ]; then
  echo "no reference checkout given (argument or REFERENCE_ROOT); keeping any prebuilt $OUT" >&2
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

# Twin builds of single-layer programs of the newer emit generation
# (fhe-cmplr/rtlib/ant/dataset/conv_*): once against the B200 library, once
# against the reference library, both with the driver
# ace_compiler_b200/programs/run_program.c.  The GPU tests run both with the
# same pinned randomness, input and weight file and compare the outputs.
DATASET="$REF/fhe-cmplr/rtlib/ant/dataset"
RT="$REF/fhe-cmplr/rtlib"
REFLIB="$HERE/_ref/libFHErt_ant_prog.so"
DRIVER="$REPO/ace_compiler_b200/programs/run_program.c"
TW="$HERE/_ref/twins"
mkdir -p "$TW"
RINC=(-I"$HERE/shims" -I"$RT/include" -I"$RT/ant/include" -I"$RT/ant/util/include"
      -I"$RT/ant/hal/include" -I"$RT/ant/poly/include" -I"$RT/ant/ckks/include"
      -I"$REF/fhe-cmplr/include" -I"$REF/air-infra/include" -I"$REF/nn-addon/include")
for name in conv_3x16x32x3 conv_16x16x32x3; do
  src="$DATASET/${name}_pre.onnx.inc"
  [ -f "$src" ] && [ -f "$REFLIB" ] || continue
  gcc -O0 -w -Werror=implicit-function-declaration -I"$REPO/include" \
      -include "$REPO/include/common/rtlib.h" -x c -c "$src" -o "$TW/$name.b200.o"
  gcc -O2 -I"$REPO/include" "$DRIVER" "$TW/$name.b200.o" -o "$TW/$name.b200" "$LIB" -lm \
      -Wl,-rpath,'$ORIGIN/../../../ace_compiler_b200'
  gcc -O0 -w -std=gnu11 -DRTLIB_SUPPORT_LINUX -DOPENFHE_COMPAT -DNDEBUG "${RINC[@]}" \
      -DGet_rt_data_info=Program_rt_data_info -include "$RT/include/common/rtlib.h" \
      -x c -c "$src" -o "$TW/$name.ref.o"
  gcc -O2 -std=gnu11 -DREFERENCE_RUNTIME -DRTLIB_SUPPORT_LINUX -DOPENFHE_COMPAT -DNDEBUG "${RINC[@]}" \
      "$DRIVER" "$TW/$name.ref.o" -o "$TW/$name.ref" "$REFLIB" -lm -Wl,-rpath,'$ORIGIN/..'
  rm -f "$TW/$name.b200.o" "$TW/$name.ref.o"
  echo "built twins $TW/$name.{b200,ref}"
done

# bootstrap_full (N = 16384, depth 23, two inputs): a program of the EDSL front
# end, emitted as C++ (extern "C" hooks), so both twins go through g++.
name=bootstrap_full
src="$DATASET/$name.inc"
if [ -f "$src" ] && [ -f "$REFLIB" ]; then
  g++ -O0 -w -I"$REPO/include" -include "$REPO/include/common/rtlib.h" -x c++ -c "$src" \
      -o "$TW/$name.b200.o"
  gcc -O2 -I"$REPO/include" -c "$DRIVER" -o "$TW/$name.drv.o"
  g++ "$TW/$name.drv.o" "$TW/$name.b200.o" -o "$TW/$name.b200" "$LIB" -lm \
      -Wl,-rpath,'$ORIGIN/../../../ace_compiler_b200'
  g++ -O0 -w -fpermissive -DRTLIB_SUPPORT_LINUX -DOPENFHE_COMPAT -DNDEBUG "${RINC[@]}" \
      -DGet_rt_data_info=Program_rt_data_info -include "$RT/include/common/rtlib.h" \
      -x c++ -c "$src" -o "$TW/$name.ref.o"
  gcc -O2 -std=gnu11 -DREFERENCE_RUNTIME -DRTLIB_SUPPORT_LINUX -DOPENFHE_COMPAT -DNDEBUG \
      "${RINC[@]}" -c "$DRIVER" -o "$TW/$name.drv.ref.o"
  g++ "$TW/$name.drv.ref.o" "$TW/$name.ref.o" -o "$TW/$name.ref" "$REFLIB" -lm -Wl,-rpath,'$ORIGIN/..'
  rm -f "$TW/$name.b200.o" "$TW/$name.ref.o" "$TW/$name.drv.o" "$TW/$name.drv.ref.o"
  echo "built twins $TW/$name.{b200,ref}"
fi
