"""The compiled ResNet-20 program as a whole (N = 2^16, 34 limbs, 19
bootstraps), the workload the benchmark times.

* recorded against eager: the per-limb calls of the program are normally
  recorded and replayed in batches (hw_queue.cu); with FHERT_EAGER_HW=1 every
  call launches at once.  Both runs must give identical logits and identical
  checksums of every ciphertext that passes Copy_ciph and the bootstrap stages
  (FHERT_TRACE_SUMS=1).
* against the reference CPU runtime: tests/golden/resnet20_reference_logits.json
  holds the logits the unmodified reference runtime computed for the same
  program, pinned randomness, input and weight file
  (tests/golden/make_resnet20_reference.sh wrote it); the GPU run must
  reproduce them bit for bit.
* replayed against direct: with FHERT_REPLAY=1 the second image's Main_graph is
  captured as one CUDA graph and the following images are served by launching
  it; every image must give the logits of the directly launched run.
"""
import json
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
EXE = os.path.join(ROOT, "ace_compiler_b200", "programs", "_ref", "resnet20_cifar10")
GOLDEN = os.path.join(HERE, "golden", "resnet20_reference_logits.json")
# must match tests/golden/make_resnet20_reference.sh
WEIGHTS = dict(entry_count=6044 + 56, sigma=0.02, seed=7)
ARGS = ["--pin", "9", "--seed", "5", "--images", "1", "--values", "10"]


@pytest.fixture(scope="module")
def weights(tmp_path_factory):
    from ace_compiler_b200.msgfile import write_synthetic_msg_file
    path = str(tmp_path_factory.mktemp("r20") / "weights.msg")
    write_synthetic_msg_file(path, WEIGHTS["entry_count"], sigma=WEIGHTS["sigma"], seed=WEIGHTS["seed"])
    return path


def run(weights, **env):
    e = dict(os.environ, FHERT_DATA_FILE=weights, FHERT_RT_STAT="0", FHERT_TRACE_SUMS="1")
    e.update(env)
    out = subprocess.run([EXE] + ARGS, capture_output=True, text=True, timeout=1500, env=e)
    assert out.returncode == 0, (out.stdout + out.stderr)[-2000:]
    line = [ln for ln in out.stdout.splitlines() if ln.startswith('{"image"')][0]
    trace = [ln for ln in out.stderr.splitlines() if ln.startswith("[FHERT_SUM]")]
    return json.loads(line)["logits"], trace


@pytest.fixture(scope="module")
def recorded(weights):
    if not os.path.exists(EXE):
        pytest.skip("compiled program not built (ace_compiler_b200/programs/build_programs.sh)")
    return run(weights)


def test_recorded_run_equals_eager_run(recorded, weights):
    logits, trace = recorded
    e_logits, e_trace = run(weights, FHERT_EAGER_HW="1")
    assert len(trace) > 100          # every layer and every bootstrap stage left checksums
    assert trace == e_trace
    assert logits == e_logits


def test_logits_equal_the_reference_runtime(recorded):
    if not os.path.exists(GOLDEN):
        pytest.skip("no golden logits committed")
    with open(GOLDEN) as f:
        golden = json.load(f)
    assert golden["args"] == ARGS and golden["weights"] == WEIGHTS
    assert recorded[0] == golden["logits"]


def run_images(weights, images, **env):
    e = dict(os.environ, FHERT_DATA_FILE=weights, FHERT_RT_STAT="0")
    e.update(env)
    args = ["--pin", "9", "--seed", "5", "--images", str(images), "--values", "10"]
    out = subprocess.run([EXE] + args, capture_output=True, text=True, timeout=1500, env=e)
    assert out.returncode == 0, (out.stdout + out.stderr)[-2000:]
    lines = [json.loads(ln) for ln in out.stdout.splitlines() if ln.startswith("{")]
    return [ln["logits"] for ln in lines if "image" in ln], lines[-1]


def test_replayed_runs_equal_direct_runs(recorded, weights):
    direct, _ = run_images(weights, 4, FHERT_PT_CACHE_MB="20000")
    replayed, summary = run_images(weights, 4, FHERT_PT_CACHE_MB="20000", FHERT_REPLAY="1")
    assert summary["replay_state"] == 2, summary
    assert summary["replayed_runs"] == 2      # image 0 direct, image 1 captured, 2 and 3 replayed
    assert direct[0] == recorded[0]
    assert replayed == direct
