"""The shared library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


LIBRARY_OF_HEADER = {"gatzk_b200.h": "libgatzk_b200.so", "gatzk_b200_tuning.h": "libgatzk_b200_tuning.so",
                     "gatzk_b200_flow.h": "libgatzk_b200_flow.so"}


def declared_symbols(header=None):
    names = []
    for fname in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if not fname.endswith(".h") or (header is not None and fname != header):
            continue
        text = open(os.path.join(ROOT, "include", fname)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"\b(gzk_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    import __graft_entry__ as entry

    entry.build()
    headers = [f for f in sorted(os.listdir(os.path.join(ROOT, "include"))) if f.endswith(".h")]
    assert set(headers) == set(LIBRARY_OF_HEADER), "every header of include/ must name the library that exports it"
    for header in headers:
        lib = ctypes.CDLL(os.path.join(ROOT, "project_b200", LIBRARY_OF_HEADER[header]))
        names = declared_symbols(header)
        assert len(names) >= (15 if header == "gatzk_b200.h" else 1)
        missing = [n for n in names if not hasattr(lib, n)]
        assert not missing, f"declared in include/{header} but not exported: {missing}"


def test_no_cpu_fallback_without_gpu():
    import torch

    if torch.cuda.is_available():
        return
    import pytest

    from project_b200 import Backend, GzkError

    with pytest.raises(GzkError):
        Backend(0)


def test_msm_window_choice_is_host_arithmetic():
    """gzk_msm_window_bits / gzk_msm_table_points run on the host: the window avoids widths whose top
    window is only a few bits wide for 255-bit scalars, and the table holds one copy of the points per window."""
    import ctypes

    from project_b200 import load_library

    lib = load_library()
    lib.gzk_msm_window_bits.restype = ctypes.c_uint
    lib.gzk_msm_table_points.restype = ctypes.c_size_t
    for log2n in range(10, 27):
        n = 1 << log2n
        c = lib.gzk_msm_window_bits(ctypes.c_size_t(n))
        assert 15 <= c <= 24
        full = -(-255 // c)
        top_bits = 255 - c * (full - 1)
        assert top_bits >= 12, (log2n, c)
        points = lib.gzk_msm_table_points(ctypes.c_size_t(n), ctypes.c_uint(c))
        assert points in (n * full, n * (full + 1))
    # 17-bit windows need a 16th window: the top digit of a scalar just below the group order exceeds 2^16
    assert lib.gzk_msm_table_points(ctypes.c_size_t(1), ctypes.c_uint(17)) == 16
    assert lib.gzk_msm_table_points(ctypes.c_size_t(1), ctypes.c_uint(16)) == 16
    assert lib.gzk_msm_table_points(ctypes.c_size_t(1), ctypes.c_uint(20)) == 13


def test_host_scalar_arithmetic_matches_integers():
    """gzk_fr_op (the 64-bit-limb host product, sum, difference, inverse) against Python integers."""
    import random

    from project_b200 import load_library

    lib = load_library()
    r = 0x73EDA753299D7D483339D80809A1D80553BDA402FFFE5BFEFFFFFFFF00000001
    word = ctypes.c_uint8 * 32

    def op(code, a, b=0):
        out = word()
        rc = lib.gzk_fr_op(code, word.from_buffer_copy(a.to_bytes(32, "little")), word.from_buffer_copy(b.to_bytes(32, "little")), out)
        return rc, int.from_bytes(bytes(out), "little")

    rng = random.Random(7)
    edge = [0, 1, 2, r - 1, r - 2, (1 << 64) - 1, 1 << 64, (1 << 128) - 1, (1 << 192) + 1, (1 << 255) % r, r >> 1]
    cases = [(a, b) for a in edge for b in edge] + [(rng.randrange(r), rng.randrange(r)) for _ in range(3000)]
    for a, b in cases:
        assert op(0, a, b) == (0, (a + b) % r)
        assert op(1, a, b) == (0, (a - b) % r)
        assert op(2, a, b) == (0, a * b % r)
    for a, _ in cases[-200:] + [(1, 0), (r - 1, 0)]:
        rc, inv = op(3, a)
        assert rc == 0 and inv * a % r == 1
    assert op(3, 0)[0] != 0          # FieldElement::inv throws on zero
    assert op(2, r, 1)[0] != 0       # not canonical


def test_header_is_plain_c(tmp_path):
    """The boundary is a C ABI: the header must compile as C99 (and as C++) with nothing but its own declarations."""
    import os
    import subprocess

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = tmp_path / "include_only.c"
    src.write_text('#include "gatzk_b200.h"\nint main(void) { return GZK_OK; }\n')
    inc = os.path.join(root, "include")
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only", f"-I{inc}", str(src)], check=True)
    subprocess.run(["g++", "-std=c++17", "-Wall", "-Wextra", "-Werror", "-fsyntax-only", "-x", "c++", f"-I{inc}", str(src)], check=True)
