"""Carry-chain field arithmetic of the CUDA kernels, compiled for the host (emulated
carry flag) and compared with the oracle's 64-bit implementation.  No GPU needed."""
import os
import subprocess
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_point_formulas_match_oracle_on_host():
    _run(os.path.join(ROOT, "tests", "host", "g1_host_check.cpp"))


def test_device_arithmetic_matches_oracle_on_host():
    _run(os.path.join(ROOT, "tests", "host", "mp_host_check.cpp"))


def test_proof_byte_codec_on_host():
    """Size formula of the reference's proof_size_bytes, byte round trip and reader errors (pure host code)."""
    _run(os.path.join(ROOT, "tests", "host", "proof_codec_check.cpp"))


def test_exchange_wait_gives_up_when_a_peer_never_posts():
    """The host-side wait behind gzk_comm_wait with a fake stream query: times out, aborts once, keeps going."""
    _run(os.path.join(ROOT, "tests", "host", "bounded_wait_check.cpp"))


def _run(src):
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "mp_host_check")
        subprocess.run(["g++", "-O2", "-std=c++17", "-pthread", "-o", exe, src], check=True)
        out = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout + out.stderr
    assert out.stdout.strip().endswith("OK")
