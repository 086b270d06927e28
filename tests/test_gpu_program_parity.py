"""Whole compiled programs on both runtimes.  Single-layer programs of the
newer emit generation (stack POLYNOMIALs, Init_poly_by_size, Set_pk0/1,
Pt_from_msg_ofst, Zero_ciph, compiler event timers) are built twice by
oracle/build_examples.sh, against the B200 library and against the reference
library, with the same driver.  With the same pinned randomness, the same
seeded input tensor and the same synthetic weight file the decrypted outputs
must be identical doubles: every ciphertext residue on the way was identical.

Replay: with FHERT_REPLAY=1 the second run of a program is captured as one
CUDA graph and later runs are served by launching it; every image must come
out as from the directly launched runs."""
import json
import os
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
TWINS = os.path.join(os.path.dirname(HERE), "oracle", "_ref", "twins")
PROGRAMS = {"conv_3x16x32x3": "1,3,32,32", "conv_16x16x32x3": "1,16,32,32"}


@pytest.fixture(scope="module")
def weights(tmp_path_factory):
    from ace_compiler_b200.msgfile import write_synthetic_msg_file
    path = str(tmp_path_factory.mktemp("w") / "conv.msg")
    write_synthetic_msg_file(path, 8, entry_floats=1 << 22, distinct=2, sigma=0.05, seed=11)
    return path


def run(exe, shape, weights, extra_env=None):
    env = dict(os.environ, FHERT_DATA_FILE=weights, FHERT_RT_STAT="0")
    env.update(extra_env or {})
    out = subprocess.run([exe, "--shape", shape, "--pin", "9", "--seed", "5", "--values", "16384"],
                         capture_output=True, text=True, timeout=900, env=env)
    assert out.returncode == 0, (out.stdout + out.stderr)[-2000:]
    line = [ln for ln in out.stdout.splitlines() if ln.startswith('{"image"')][0]
    return json.loads(line)["logits"]


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(PROGRAMS))
def test_program_outputs_identical_to_reference(name, weights):
    ours, ref = os.path.join(TWINS, name + ".b200"), os.path.join(TWINS, name + ".ref")
    if not (os.path.exists(ours) and os.path.exists(ref)):
        pytest.skip("twin binaries not built (oracle/build_examples.sh)")
    want = run(ref, PROGRAMS[name], weights)
    got = run(ours, PROGRAMS[name], weights)
    assert len(got) == len(want) == 16384
    assert max(abs(v) for v in want) > 1e-3          # a real convolution came out
    assert got == want
    # and the same with the per-limb calls launched one by one
    assert run(ours, PROGRAMS[name], weights, {"FHERT_EAGER_HW": "1"}) == want


def splitmix_uniform(seed, count, amp):
    """The driver's input stream (run_program.c): splitmix64, top 53 bits, [-amp, amp)."""
    out, state, mask = [], seed, (1 << 64) - 1
    for _ in range(count):
        state = (state + 0x9E3779B97F4A7C15) & mask
        z = state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
        z ^= z >> 31
        out.append(amp * ((z >> 11) / 4503599627370496.0 - 1.0))
    return out


@pytest.mark.gpu
def test_bootstrap_full_program_identical_to_reference(tmp_path):
    """dataset/bootstrap_full (N = 16384, depth 23, two inputs, written out in
    polynomial-level calls): the outputs equal the reference runtime's bit for
    bit and approximate sin(8x) of the first input within the tolerance of the
    program's own driver (bootstrap_full.main.inc:17-35, 1e-2)."""
    import math
    from ace_compiler_b200.msgfile import write_synthetic_msg_file
    ours, ref = os.path.join(TWINS, "bootstrap_full.b200"), os.path.join(TWINS, "bootstrap_full.ref")
    if not (os.path.exists(ours) and os.path.exists(ref)):
        pytest.skip("twin binaries not built (oracle/build_examples.sh)")
    weights = str(tmp_path / "unused.msg")  # the program reads no weights; the file must exist
    write_synthetic_msg_file(weights, 2, entry_floats=64, distinct=2, sigma=0.05, seed=1)
    args = ["--pin", "9", "--seed", "5", "--shape", "1,1,1,8", "--input", "p0", "--input", "p1=0",
            "--amp", "0.8", "--values", "8"]

    def go(exe, extra=None):
        env = dict(os.environ, FHERT_DATA_FILE=weights, FHERT_RT_STAT="0")
        env.update(extra or {})
        out = subprocess.run([exe] + args, capture_output=True, text=True, timeout=900, env=env)
        assert out.returncode == 0, (out.stdout + out.stderr)[-2000:]
        return json.loads([ln for ln in out.stdout.splitlines() if ln.startswith('{"image"')][0])["logits"]

    want = go(ref)
    got = go(ours)
    assert got == want
    assert go(ours, {"FHERT_EAGER_HW": "1"}) == want
    x = splitmix_uniform(5, 8, 0.8)
    for v, xi in zip(got, x):
        assert abs(v - math.sin(8 * xi)) < 1e-2


def run_images(exe, args, weights, images, **extra):
    env = dict(os.environ, FHERT_DATA_FILE=weights, FHERT_RT_STAT="0")
    env.update(extra)
    out = subprocess.run([exe] + args + ["--images", str(images)], capture_output=True, text=True,
                         timeout=900, env=env)
    assert out.returncode == 0, (out.stdout + out.stderr)[-2000:]
    lines = [json.loads(ln) for ln in out.stdout.splitlines() if ln.startswith("{")]
    return [ln["logits"] for ln in lines if "image" in ln], lines[-1]


@pytest.mark.gpu
@pytest.mark.parametrize("cache_mb", ["4000", "0"])   # "0": every weight is encoded inside the run
def test_replayed_convolution_equals_direct_runs(weights, cache_mb):
    exe = os.path.join(TWINS, "conv_16x16x32x3.b200")
    if not os.path.exists(exe):
        pytest.skip("twin binaries not built (oracle/build_examples.sh)")
    args = ["--shape", PROGRAMS["conv_16x16x32x3"], "--pin", "9", "--seed", "5", "--values", "16384"]
    direct, _ = run_images(exe, args, weights, 5, FHERT_PT_CACHE_MB=cache_mb)
    replayed, summary = run_images(exe, args, weights, 5, FHERT_PT_CACHE_MB=cache_mb, FHERT_REPLAY="1")
    assert summary["replay_state"] == 2 and summary["replayed_runs"] == 3, summary
    assert len({tuple(v) for v in direct}) == 5      # five different images
    assert replayed == direct


@pytest.mark.gpu
def test_replayed_two_input_bootstrap_program_equals_direct_runs(tmp_path):
    from ace_compiler_b200.msgfile import write_synthetic_msg_file
    exe = os.path.join(TWINS, "bootstrap_full.b200")
    if not os.path.exists(exe):
        pytest.skip("twin binaries not built (oracle/build_examples.sh)")
    weights = str(tmp_path / "unused.msg")
    write_synthetic_msg_file(weights, 2, entry_floats=64, distinct=2, sigma=0.05, seed=1)
    args = ["--pin", "9", "--seed", "5", "--shape", "1,1,1,8", "--input", "p0", "--input", "p1=0",
            "--amp", "0.8", "--values", "8"]
    direct, _ = run_images(exe, args, weights, 4)
    replayed, summary = run_images(exe, args, weights, 4, FHERT_REPLAY="1")
    assert summary["replay_state"] == 2 and summary["replayed_runs"] == 2, summary
    assert replayed == direct


@pytest.mark.gpu
def test_a_run_that_cannot_be_captured_is_launched_directly(weights):
    # without the plaintext cache every weight is encoded from host data inside
    # the run, and with no room for snapshots of that data the capture ends at the
    # first one: what was captured is launched, the rest of the run and all later
    # runs are launched directly
    exe = os.path.join(TWINS, "conv_16x16x32x3.b200")
    if not os.path.exists(exe):
        pytest.skip("twin binaries not built (oracle/build_examples.sh)")
    args = ["--shape", PROGRAMS["conv_16x16x32x3"], "--pin", "9", "--seed", "5", "--values", "16384"]
    direct, _ = run_images(exe, args, weights, 3)
    broken, summary = run_images(exe, args, weights, 3, FHERT_REPLAY="1", FHERT_REPLAY_STAGE_MB="0")
    assert summary["replay_state"] == 0 and summary["replayed_runs"] == 0, summary
    assert "cannot be captured" in summary["replay_off_because"]
    assert broken == direct
