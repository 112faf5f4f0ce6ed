"""Builds and runs the C++ host mirror of the reference interface on the GPU and checks
it against the oracle (tests/host/mirror_check.cpp)."""
import os
import subprocess
import tempfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _compile(exe):
    import oracle_lib

    oracle_lib.build()
    lib_dir = os.path.join(ROOT, "project_b200")
    ora_dir = os.path.join(ROOT, "oracle")
    subprocess.run(["g++", "-O2", "-std=c++17", "-o", exe, os.path.join(ROOT, "tests", "host", "mirror_check.cpp"),
                    f"-L{lib_dir}", f"-L{ora_dir}", "-l:libgatzk_b200.so", "-l:liboracle.so",
                    f"-Wl,-rpath,{lib_dir}", f"-Wl,-rpath,{ora_dir}", "-pthread"], check=True)


def test_host_mirror_compiles():
    with tempfile.TemporaryDirectory() as tmp:
        _compile(os.path.join(tmp, "mirror_check"))


@pytest.mark.gpu
def test_host_mirror_matches_oracle_on_gpu():
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "mirror_check")
        _compile(exe)
        out = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout + out.stderr
    assert out.stdout.strip().endswith("OK")
