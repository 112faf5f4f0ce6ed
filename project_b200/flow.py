"""ctypes view of the prover flow (include/gatzk_b200_flow.h).  The same C entry points exist
twice: in libgatzk_b200_flow.so over the GPU library (prefix gzk_flow_) and, as test
infrastructure, in oracle/liboracle.so over the CPU restatement (prefix ora_flow_)."""
import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
FLOW_LIB_PATH = os.path.join(HERE, "libgatzk_b200_flow.so")
DOMAINS = ("FH", "edge", "in", "d", "cat", "C", "N")


class FlowConfig(ctypes.Structure):
    _fields_ = [("node_count", ctypes.c_uint64), ("feature_count", ctypes.c_uint64), ("class_count", ctypes.c_uint64), ("edge_count", ctypes.c_uint64),
                ("hidden_layer_count", ctypes.c_uint64), ("hidden_heads", ctypes.c_void_p), ("hidden_head_dim", ctypes.c_void_p),
                ("output_heads", ctypes.c_uint64), ("range_bits", ctypes.c_uint32), ("seed", ctypes.c_uint64), ("features", ctypes.c_void_p),
                ("edge_src", ctypes.c_void_p), ("edge_dst", ctypes.c_void_p), ("params", ctypes.c_void_p), ("param_count", ctypes.c_uint64),
                ("generator", ctypes.c_void_p), ("compact_columns", ctypes.c_uint32)]


class FlowError(RuntimeError):
    pass


class Flow:
    """One prepared proof context (model, graph, features, key) on one backend."""

    def __init__(self, lib, prefix, target, inputs, generator, seed=11, range_bits=12, compact_columns=False):
        self.lib, self.prefix = lib, prefix
        self._fn = lambda name: getattr(lib, prefix + name)
        self._fn("error").restype = ctypes.c_char_p
        for name in ("dump", "proof_bytes", "domain_labels"):
            self._fn(name).restype = ctypes.c_size_t
        self._keep = {
            "heads": np.ascontiguousarray([h for h, _ in inputs["hidden"]], dtype=np.uint64),
            "dims": np.ascontiguousarray([d for _, d in inputs["hidden"]], dtype=np.uint64),
            "features": np.ascontiguousarray(inputs["features"], dtype=np.float64),
            "src": np.ascontiguousarray(inputs["edge_src"], dtype=np.uint32),
            "dst": np.ascontiguousarray(inputs["edge_dst"], dtype=np.uint32),
            "params": np.ascontiguousarray(inputs["params"], dtype=np.float64),
            "generator": np.ascontiguousarray(generator, dtype=np.uint8).reshape(-1),
        }
        k = self._keep
        cfg = FlowConfig(inputs["nodes"], inputs["feature_count"], inputs["class_count"], k["src"].size, len(inputs["hidden"]),
                         k["heads"].ctypes.data, k["dims"].ctypes.data, inputs["output_heads"], range_bits, seed, k["features"].ctypes.data,
                         k["src"].ctypes.data, k["dst"].ctypes.data, k["params"].ctypes.data, k["params"].size, k["generator"].ctypes.data,
                         int(bool(compact_columns)))
        handle = ctypes.c_void_p()
        self._check(self._fn("create")(int(target), ctypes.byref(cfg), ctypes.byref(handle)))
        self.handle = handle

    def _check(self, rc):
        if rc != 0:
            raise FlowError(self._fn("error")().decode())

    def prove(self, inputs_resident=False):
        self._check(self._fn("prove_resident" if inputs_resident else "prove")(self.handle))

    def set_msm_commit(self, on):
        """Switch the MSM commitment path of a GPU flow; returns (commitments checked so far, mismatches)."""
        counts = (ctypes.c_uint64 * 2)()
        self._check(self._fn("set_msm_commit")(self.handle, int(bool(on)), counts))
        return int(counts[0]), int(counts[1])

    def dump(self):
        fn = self._fn("dump")
        size = fn(self.handle, None, ctypes.c_size_t(0))
        buf = ctypes.create_string_buffer(size)
        fn(self.handle, buf, ctypes.c_size_t(size))
        return buf.raw.decode()

    def proof_bytes(self):
        fn = self._fn("proof_bytes")
        size = fn(self.handle, None, ctypes.c_size_t(0))
        buf = np.zeros(size, dtype=np.uint8)
        fn(self.handle, buf.ctypes.data_as(ctypes.c_void_p), ctypes.c_size_t(size))
        return buf

    def stats(self):
        out = (ctypes.c_uint64 * 14)()
        self._check(self._fn("stats")(self.handle, out))
        v = list(out)
        return {"commit_barriers": v[0], "challenges": v[1], "dynamic_commitments": v[2], "opened_columns": v[3],
                "domains": dict(zip(DOMAINS, v[4:11])), "h2d_bytes": v[11], "d2h_bytes": v[12], "guard_flags": v[13]}

    def constraint_violations(self):
        """(rows with a non-zero quotient numerator per domain, [(domain index, constraint index, rows it failed on), ...])."""
        out = (ctypes.c_uint64 * 7)()
        cap = 4096
        failures = (ctypes.c_uint64 * (3 * cap))()
        count = ctypes.c_size_t(0)
        self._check(self._fn("constraint_violations")(self.handle, out, failures, ctypes.c_size_t(cap), ctypes.byref(count)))
        n = min(int(count.value), cap)
        return list(out), [(int(failures[3 * i]), int(failures[3 * i + 1]), int(failures[3 * i + 2])) for i in range(n)]

    def honest_quotient(self, domain, log2_blowup=2, classes=1):
        """N = t (X^n - 1) + R of one domain's quotient numerator, restricted to the constraint classes in `classes`
        (bit 0 exact, bit 1 wrapping, bit 2 loose), through the backend's transforms."""
        out = (ctypes.c_uint64 * 6)()
        self._check(self._fn("honest_quotient")(self.handle, domain.encode(), ctypes.c_uint(log2_blowup), ctypes.c_uint(classes), out))
        keys = ("n", "points", "numerator_degree", "remainder_rows", "identity_holds", "quotient_degree")
        return dict(zip(keys, (int(v) for v in out)))

    def domain_labels(self, domain):
        fn = self._fn("domain_labels")
        size = fn(self.handle, domain.encode(), None, ctypes.c_size_t(0))
        buf = ctypes.create_string_buffer(size + 1)
        fn(self.handle, domain.encode(), buf, ctypes.c_size_t(size))
        return [s for s in buf.raw[:size].decode().split("\n") if s]

    def column(self, label, limit=None):
        """(kind, values) of a committed column of the last proof: int arrays for the small-integer
        kinds, [n, 32] uint8 canonical field elements otherwise."""
        kind, length = ctypes.c_int(), ctypes.c_uint64()
        fn = self._fn("column")
        self._check(fn(self.handle, label.encode(), ctypes.byref(kind), ctypes.byref(length), None, ctypes.c_size_t(0)))
        n = int(length.value) if limit is None else min(int(length.value), limit)
        dtype, width = {0: (np.uint8, 32), 1: (np.uint8, 32), 2: (np.int64, 1), 3: (np.uint32, 1), 4: (np.float64, 1)}[kind.value]
        out = np.zeros((n, width) if width > 1 else (n,), dtype=dtype)
        self._check(fn(self.handle, label.encode(), None, None, out.ctypes.data_as(ctypes.c_void_p), ctypes.c_size_t(n)))
        return kind.value, out

    def context(self):
        """The gzk_ctx of a GPU flow (for timing queries); None for the CPU flow."""
        if self.prefix != "gzk_flow_":
            return None
        self.lib.gzk_flow_context.restype = ctypes.c_void_p
        return ctypes.c_void_p(self.lib.gzk_flow_context(self.handle))

    def side_contexts(self):
        """The further gzk_ctx handles a GPU flow deals independent call chains over (they exist once a proof has run)."""
        if self.prefix != "gzk_flow_":
            return []
        self.lib.gzk_flow_side_context.restype = ctypes.c_void_p
        out = []
        while True:
            side = self.lib.gzk_flow_side_context(self.handle, ctypes.c_size_t(len(out)))
            if not side:
                return out
            out.append(ctypes.c_void_p(side))

    def close(self):
        if self.handle:
            fn = self._fn("destroy")
            fn.restype = None
            fn(self.handle)
            self.handle = None


def gpu_flow(device, inputs, generator, **kw):
    from .lib import load_library

    load_library()  # the flow library links against libgatzk_b200.so
    if not os.path.exists(FLOW_LIB_PATH):
        raise RuntimeError(f"{FLOW_LIB_PATH} is missing: build it with `python -m project_b200.build`")
    return Flow(ctypes.CDLL(FLOW_LIB_PATH), "gzk_flow_", device, inputs, generator, **kw)
