#!/usr/bin/env bash
# TEST INFRASTRUCTURE ONLY.
#
# Writes tests/golden/resnet20_reference_logits.json: the logits the unmodified
# reference CPU runtime computes for the committed resnet20_cifar10 program with
# pinned randomness (--pin 9), the seeded input image (--seed 5) and the seeded
# synthetic weight file tests/test_gpu_resnet20_program.py also uses.  The GPU
# test requires the B200 runtime to reproduce them bit for bit.
#
# The run needs the reference checkout, about 45 GB of host memory and about
# half an hour on one core.  The program is compiled where it lies (nothing is
# copied out of the reference tree) against oracle/_ref/libFHErt_ant_prog.so
# with the adapter for its older Alloc_poly call (oracle/shims/old_program_adapter.h).
#
# usage: tests/golden/make_resnet20_reference.sh <reference-root>
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REPO="$(dirname "$(dirname "$HERE")")"
REF="${1:-${REFERENCE_ROOT:-}}"
[ -n "$REF" ] || { echo "usage: $0 <reference-root>" >&2; exit 1; }
RT="$REF/fhe-cmplr/rtlib"
ORACLE="$REPO/oracle"
WORK="$(mktemp -d)"
RINC=(-I"$ORACLE/shims" -I"$RT/include" -I"$RT/ant/include" -I"$RT/ant/util/include"
      -I"$RT/ant/hal/include" -I"$RT/ant/poly/include" -I"$RT/ant/ckks/include"
      -I"$REF/fhe-cmplr/include" -I"$REF/air-infra/include" -I"$REF/nn-addon/include")
DEF=(-std=gnu11 -DRTLIB_SUPPORT_LINUX -DOPENFHE_COMPAT -DNDEBUG)
gcc -O0 -w "${DEF[@]}" "${RINC[@]}" -DGet_rt_data_info=Program_rt_data_info \
    -include "$RT/include/common/rtlib.h" -include "$ORACLE/shims/old_program_adapter.h" \
    -x c -c "$RT/ant/dataset/resnet20_cifar10_pre.onnx.inc" -o "$WORK/program.o"
gcc -O2 "${DEF[@]}" -DREFERENCE_RUNTIME "${RINC[@]}" \
    "$REPO/ace_compiler_b200/programs/run_program.c" "$WORK/program.o" -o "$WORK/resnet20.ref" \
    "$ORACLE/_ref/libFHErt_ant_prog.so" -lm -Wl,-rpath,"$ORACLE/_ref"
ARGS=(--pin 9 --seed 5 --images 1 --values 10)
PYTHONPATH="$REPO" python - "$WORK/weights.msg" <<'PY'
import sys
from ace_compiler_b200.msgfile import write_synthetic_msg_file
write_synthetic_msg_file(sys.argv[1], 6044 + 56, sigma=0.02, seed=7)
PY
FHERT_DATA_FILE="$WORK/weights.msg" "$WORK/resnet20.ref" "${ARGS[@]}" > "$WORK/run.out"
python - "$WORK/run.out" "$HERE/resnet20_reference_logits.json" <<'PY'
import json, sys
lines = open(sys.argv[1]).read().splitlines()
image = json.loads([ln for ln in lines if ln.startswith('{"image"')][0])
tail = json.loads([ln for ln in lines if ln.startswith('{"setup_s"')][0])
json.dump({"program": "resnet20_cifar10", "args": ["--pin", "9", "--seed", "5", "--images", "1", "--values", "10"],
           "weights": {"entry_count": 6044 + 56, "sigma": 0.02, "seed": 7},
           "logits": image["logits"],
           "reference_cpu_seconds": {"setup": tail["setup_s"], "encrypt": image["encrypt_s"],
                                     "inference": image["infer_s"], "decrypt": image["decrypt_s"]}},
          open(sys.argv[2], "w"), indent=1)
PY
rm -rf "$WORK"
echo "wrote $HERE/resnet20_reference_logits.json"
