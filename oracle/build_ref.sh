#!/usr/bin/env bash
# TEST INFRASTRUCTURE ONLY.
#
# Builds the unmodified ANT-ACE CPU runtime (fhe-cmplr/rtlib/ant + rtlib/common)
# from the read-only reference checkout into oracle/_ref/libFHErt_ant_ref.so.
# The reference's own build fetches GMP headers, uthash and BLAKE2 from the
# network; here they are replaced by the stand-ins in oracle/shims/.  Nothing
# is copied out of the reference tree: sources are compiled where they lie.
#
# usage: oracle/build_ref.sh [reference-root]      (or REFERENCE_ROOT in the environment)
#   env OMP=1 additionally builds libFHErt_ant_ref_omp.so (-fopenmp, the
#   reference's BUILD_WITH_OPENMP variant).
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REF="${1:-${REFERENCE_ROOT:-}}"
RT="$REF/fhe-cmplr/rtlib"
OUT="$HERE/_ref"
if [ -z "$REF" ] || [ ! -d "$RT/ant" ]; then
  echo "no reference checkout given (argument or REFERENCE_ROOT); keeping any prebuilt $OUT" >&2
  exit 0
fi
mkdir -p "$OUT/obj"

INC=(-I"$HERE/shims" -I"$RT/include" -I"$RT/ant/include" -I"$RT/ant/util/include"
     -I"$RT/ant/hal/include" -I"$RT/ant/poly/include" -I"$RT/ant/ckks/include"
     -I"$REF/fhe-cmplr/include" -I"$REF/air-infra/include" -I"$REF/nn-addon/include")
DEF=(-DRTLIB_SUPPORT_LINUX -DOPENFHE_COMPAT -DUSE_PRNG_SEED -DNDEBUG)
# CMake "Release" defaults of the reference: -O3 -DNDEBUG, no -march
CFLAGS=(-O3 -fPIC -std=gnu11 -w -Werror=implicit-function-declaration)

SRCS=()
for d in context ckks poly lpoly hal util; do
  for f in "$RT/ant/$d/src/"*.c; do SRCS+=("$f"); done
done
SRCS+=("$RT/ant/porting/pt_mgr.c")
for f in "$RT/common/src/"*.c "$RT/common/linux/"*.c; do SRCS+=("$f"); done
SRCS+=("$HERE/shims/minigmp.c" "$HERE/shims/blake2xb.c" "$HERE/ref_hooks.c" "$HERE/ref_harness.c")

build_variant() {  # $1 = suffix, rest = extra flags
  local suf="$1"; shift
  local objs=()
  for f in "${SRCS[@]}"; do
    local o="$OUT/obj/$(echo "${f#$REF/}" | tr "/" "_")$suf.o"
    gcc "${CFLAGS[@]}" "$@" "${DEF[@]}" "${INC[@]}" -c "$f" -o "$o" &
    objs+=("$o")
    # bound the number of parallel compiles
    while [ "$(jobs -r | wc -l)" -ge 8 ]; do wait -n; done
  done
  wait
  gcc -shared "$@" -o "$OUT/libFHErt_ant_ref$suf.so" "${objs[@]}" -lm \
      -Wl,--allow-shlib-undefined -Wl,-z,defs -Wl,-Bsymbolic
  echo "built $OUT/libFHErt_ant_ref$suf.so"
  if [ -z "$suf" ]; then
    # the same objects without the Python-facing harness (which answers the
    # program hooks itself): compiled programs link against this one and keep
    # their own Get_context_params, Main_graph ...
    local prog=()
    for o in "${objs[@]}"; do case "$o" in *ref_harness*) ;; *) prog+=("$o");; esac; done
    gcc -shared -o "$OUT/libFHErt_ant_prog.so" "${prog[@]}" -lm -Wl,--allow-shlib-undefined
    echo "built $OUT/libFHErt_ant_prog.so"
  fi
}

build_variant ""
if [ "${OMP:-0}" = "1" ]; then build_variant "_omp" -fopenmp; fi
