"""B200 (sm_100a) compute backend for the data-parallel core of the GAT-ZKML prover.

The product is the C-ABI shared library `libgatzk_b200.so` (declared in
include/gatzk_b200.h) plus the C++ host-side mirror of the reference's
operator interface under project_b200/host/.  This Python package only loads
the library through ctypes for tests and benchmarks; it holds no compute path
of its own and raises if the CUDA library is missing.
"""
from .lib import fr_sum, g1_sum, incoming_lists, shard_rows  # noqa: F401
from .lib import Backend, Buffer, GzkError, load_library, KIND_FR, KIND_FR_MONT, KIND_I64, KIND_U32, KIND_F64, KIND_G1  # noqa: F401
