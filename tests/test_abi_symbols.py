"""The shared library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = []
    for fname in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if not fname.endswith(".h"):
            continue
        text = open(os.path.join(ROOT, "include", fname)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"\b(gzk_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    import __graft_entry__ as entry

    entry.build()
    lib = ctypes.CDLL(os.path.join(ROOT, "project_b200", "libgatzk_b200.so"))
    names = declared_symbols()
    assert len(names) >= 15
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"


def test_no_cpu_fallback_without_gpu():
    import torch

    if torch.cuda.is_available():
        return
    import pytest

    from project_b200 import Backend, GzkError

    with pytest.raises(GzkError):
        Backend(0)
