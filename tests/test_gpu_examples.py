"""The reference's own example programs, compiled unchanged against this
repository's headers and linked with the B200 library.

Each program (fhe-cmplr/rtlib/ant/example/eg_fhertlib_*.c plus the .inc body
the compiler emitted) builds a context from its CKKS_PARAMS, encrypts a small
tensor with Prepare_input, runs its Main_graph limb by limb through the C-ABI
(Coeffs, Hw_modadd, Hw_modmul, Hw_rotate, Decomp, Mod_up, Mod_down, Rescale,
Init_ciph_*, Encode_float ...), decrypts with Handle_output and compares with
the values its author wrote down, printing "SUCESS!" (sic) when they agree to
1e-3.  oracle/build_examples.sh makes the binaries where the reference
checkout is present; here they are only executed.
"""
import os
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
EXAMPLES = os.path.join(os.path.dirname(HERE), "oracle", "_ref", "examples")

# programs that need entry points outside the built scope do not link and are
# absent from the directory; every one that was built must pass
NAMES = sorted(f for f in (os.listdir(EXAMPLES) if os.path.isdir(EXAMPLES) else [])
               if f.startswith("eg_fhertlib_") and "." not in f)


@pytest.mark.gpu
def test_examples_were_built():
    assert len(NAMES) >= 15, f"expected the example programs under {EXAMPLES}, found {NAMES}"


@pytest.mark.gpu
@pytest.mark.parametrize("name", NAMES)
def test_example_program(name):
    exe = os.path.join(EXAMPLES, name)
    run = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    tail = (run.stdout + run.stderr)[-2000:]
    assert run.returncode == 0, tail
    if name == "eg_fhertlib_mul_const_rtv":
        # this one feeds a message that is too large for its modulus and expects
        # the run-time validation to notice
        assert "EXPECTED FAILED!" in run.stdout, tail
        assert "internal validation fail" in run.stdout, tail
        return
    assert "SUCESS!" in run.stdout, tail
    assert "FAILED" not in run.stdout, tail


@pytest.mark.gpu
@pytest.mark.parametrize("name", [n for n in NAMES if n.split("_")[-1] in
                                  ("conv2d", "gemm", "relu", "rotate", "relin", "bootstrap")])
def test_recording_is_transparent(name):
    """With pinned randomness, the checksums of every ciphertext the program
    copies are the same whether the per-limb calls are recorded and merged or
    launched one by one."""
    exe = os.path.join(EXAMPLES, name)
    traces = []
    for eager in ("0", "1"):
        env = dict(os.environ, FHERT_PIN="3", FHERT_TRACE_SUMS="1", FHERT_EAGER_HW=eager)
        run = subprocess.run([exe], capture_output=True, text=True, timeout=600, env=env)
        assert run.returncode == 0, run.stderr[-2000:]
        traces.append([ln for ln in run.stderr.splitlines() if ln.startswith("[FHERT_SUM]")])
    assert len(traces[0]) > 0
    assert traces[0] == traces[1]
