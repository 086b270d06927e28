"""The bookkeeping behind the data-flow dependences of a captured program run
(ace_compiler_b200/csrc/access_map.h) against a per-byte record, on the CPU."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(HERE), "ace_compiler_b200", "csrc")


def test_dependences_match_a_per_byte_record(tmp_path):
    exe = str(tmp_path / "access_map_check")
    subprocess.run(["g++", "-O2", "-std=c++17", "-I", CSRC, os.path.join(HERE, "access_map_check.cpp"),
                    "-o", exe], check=True)
    out = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout
    assert out.stdout.startswith("ok ")
