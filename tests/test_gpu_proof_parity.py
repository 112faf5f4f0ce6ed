"""Commit + prove flow on the GPU backend against the same flow on the CPU restatement, field by
field: every Fiat-Shamir challenge, tau-evaluation, commitment point, quotient scalar, opened value,
opening witness, external evaluation and witness scalar, and the serialised proof bytes.

Both runs execute project_b200/host/prover_flow.hpp (the host orchestration the reference keeps
in src/protocol/trace.cpp and prover.cpp); what differs is the compute backend underneath:
libgatzk_b200.so through its C ABI versus oracle/.  A single differing field value anywhere in
the chain changes every later challenge, so equality of the listings is equality of the proofs."""
import numpy as np
import pytest

import oracle_lib as ora
import pyref
from project_b200 import synthetic
from project_b200.flow import Flow, gpu_flow

pytestmark = pytest.mark.gpu

G = np.frombuffer(pyref.g1_bytes((pyref.GX, pyref.GY)), dtype=np.uint8).copy()


def first_difference(a, b):
    la, lb = a.splitlines(), b.splitlines()
    for i, (x, y) in enumerate(zip(la, lb)):
        if x != y:
            return f"line {i}: gpu `{x[:120]}` vs cpu `{y[:120]}`"
    return None if len(la) == len(lb) else f"{len(la)} vs {len(lb)} lines"


@pytest.mark.parametrize("shape", [
    dict(seed=1, nodes=40, directed_edges=120, feature_count=12, hidden=[(2, 4)], output_heads=2, class_count=3),
    dict(seed=2, nodes=64, directed_edges=300, feature_count=20, hidden=[(1, 8)], output_heads=1, class_count=7),
    dict(seed=3, nodes=50, directed_edges=200, feature_count=9, hidden=[(2, 3), (2, 2)], output_heads=1, class_count=4),
])
def test_gpu_proof_equals_cpu_proof_field_by_field(shape):
    inputs = synthetic.make_inputs(**shape)
    cpu = Flow(ora.lib(), "ora_flow_", 4, inputs, G)
    gpu = gpu_flow(0, inputs, G)
    cpu.prove()
    gpu.prove()
    assert first_difference(gpu.dump(), cpu.dump()) is None
    assert np.array_equal(gpu.proof_bytes(), cpu.proof_bytes())
    counters = ("commit_barriers", "challenges", "dynamic_commitments", "opened_columns", "domains")
    assert {k: gpu.stats()[k] for k in counters} == {k: cpu.stats()[k] for k in counters}
    # a second proof on the same context recomputes everything and gives the same bytes
    gpu.prove()
    assert np.array_equal(gpu.proof_bytes(), cpu.proof_bytes())
    # a few committed columns themselves (not only their evaluations)
    for label in ("P_h0_R_L", "P_h0_PSQ", "P_h0_Query_dst", "P_h0_m_exp", "P_h0_S"):
        kind_g, col_g = gpu.column(label)
        kind_c, col_c = cpu.column(label)
        assert kind_g == kind_c and np.array_equal(col_g, col_c), label
    cpu.close()
    gpu.close()


def test_values_on_a_rounding_boundary_take_the_host_recheck():
    """Inputs on a 1/32 grid put many forward-pass values exactly on a rounding boundary of the
    quantisation (16 v = k + 1/2).  The GPU flow must notice (guard_flags > 0), repeat the forward pass
    with the host loop, and still produce the CPU proof byte for byte."""
    shape = dict(seed=9, nodes=48, directed_edges=160, feature_count=8, hidden=[(2, 4)], output_heads=1, class_count=3)
    inputs = synthetic.make_inputs(**shape)
    rng = np.random.default_rng(4)
    inputs["features"] = rng.integers(0, 9, size=inputs["features"].shape) / 4.0
    inputs["params"] = np.round(inputs["params"] * 8.0) / 8.0
    cpu = Flow(ora.lib(), "ora_flow_", 2, inputs, G)
    gpu = gpu_flow(0, inputs, G)
    cpu.prove()
    gpu.prove()
    assert gpu.stats()["guard_flags"] > 0
    assert first_difference(gpu.dump(), cpu.dump()) is None
    assert np.array_equal(gpu.proof_bytes(), cpu.proof_bytes())
    cpu.close()
    gpu.close()


def test_msm_commitments_equal_the_trapdoor_commitments():
    """Every commitment of a proof, computed once more as an MSM of the column against the resident SRS
    (Lagrange basis of its domain, monomial basis for the matrices), is the same point as [p(tau)] G."""
    shape = dict(seed=12, nodes=40, directed_edges=120, feature_count=10, hidden=[(2, 4)], output_heads=2, class_count=3)
    gpu = gpu_flow(0, synthetic.make_inputs(**shape), G)
    gpu.set_msm_commit(True)
    gpu.prove()
    checked, mismatches = gpu.set_msm_commit(False)
    assert checked == gpu.stats()["dynamic_commitments"] - 4  # the four lazy feature-lookup commitments are scalar combinations
    assert mismatches == 0
    gpu.close()


@pytest.mark.parametrize("shape", [
    dict(seed=1, nodes=40, directed_edges=120, feature_count=12, hidden=[(2, 4)], output_heads=2, class_count=3),
    dict(seed=8, nodes=200, directed_edges=500, feature_count=6, hidden=[(1, 128)], output_heads=1, class_count=3),
    # more than 2^20 rows in the edge columns: the running sums take the single-column entry points
    dict(seed=4, nodes=9000, directed_edges=30000, feature_count=6, hidden=[(1, 128)], output_heads=1, class_count=3),
])
def test_prefix_stored_gpu_proof_equals_whole_domain_cpu_proof(shape):
    """compact_columns on the GPU (edge-domain columns stored as prefixes, running sums with their constant
    tail) against the whole-domain CPU run: the same proof."""
    inputs = synthetic.make_inputs(**shape)
    big = shape["nodes"] > 1000
    cpu = Flow(ora.lib(), "ora_flow_", 8, inputs, G, compact_columns=big)  # the large shape: both compact (CPU time)
    gpu = gpu_flow(0, inputs, G, compact_columns=True)
    cpu.prove()
    gpu.prove()
    assert first_difference(gpu.dump(), cpu.dump()) is None
    assert np.array_equal(gpu.proof_bytes(), cpu.proof_bytes())
    if big:
        # and the whole-domain GPU run agrees with the compact one
        full = gpu_flow(0, inputs, G)
        full.prove()
        assert np.array_equal(full.proof_bytes(), gpu.proof_bytes())
        full.close()
    cpu.close()
    gpu.close()


def test_no_builder_reads_a_row_nobody_wrote():
    """With every fresh device buffer of the flow filled with a byte pattern, the GPU proof is still the CPU
    proof: no kernel of the flow depends on the previous contents of its output or scratch buffers."""
    import ctypes

    from project_b200.flow import FLOW_LIB_PATH
    from project_b200.lib import load_library

    load_library()
    hook = ctypes.CDLL(FLOW_LIB_PATH).gzk_flow_debug_poison_allocations
    for shape, compact in ((dict(seed=3, nodes=50, directed_edges=200, feature_count=9, hidden=[(2, 3), (2, 2)], output_heads=1, class_count=4), False),
                           (dict(seed=1, nodes=40, directed_edges=120, feature_count=12, hidden=[(2, 4)], output_heads=2, class_count=3), True)):
        inputs = synthetic.make_inputs(**shape)
        cpu = Flow(ora.lib(), "ora_flow_", 4, inputs, G)
        cpu.prove()
        hook(1)
        try:
            gpu = gpu_flow(0, inputs, G, compact_columns=compact)
            gpu.prove()
            gpu.prove()
        finally:
            hook(0)
        assert first_difference(gpu.dump(), cpu.dump()) is None
        cpu.close()
        gpu.close()


@pytest.mark.parametrize("compact", [False, True])
def test_quotient_constraints_vanish_on_the_rows_of_the_gpu_columns(compact):
    """The row check of the restated quotient numerators (every constraint the reference's own witness satisfies
    vanishes on every row; ProverFlow::constraint_violations) over the columns the GPU backend built, two hidden
    layers and two output heads."""
    inputs = synthetic.make_inputs(seed=5, nodes=30, directed_edges=90, feature_count=7, hidden=[(2, 3), (1, 4)], output_heads=2, class_count=3)
    gpu = gpu_flow(0, inputs, G, compact_columns=compact)
    gpu.prove()
    bad, failures = gpu.constraint_violations()
    gpu.close()
    assert bad == [0] * 7, failures


def test_honest_quotients_through_the_gpu_transforms():
    """The honest quotient of every domain with the columns built, interpolated and extended on the GPU (gzk_ntt on
    the trace columns of a proof): the same report as over the CPU backend for every class of constraints, no
    remainder for the constraints that vanish on every row, and the division identity at a point outside the
    domains."""
    inputs = synthetic.make_inputs(seed=3, nodes=24, directed_edges=60, feature_count=6, hidden=[(2, 4)], output_heads=1, class_count=3)
    cpu = Flow(ora.lib(), "ora_flow_", 2, inputs, G)
    gpu = gpu_flow(0, inputs, G)
    cpu.prove()
    gpu.prove()
    for domain in ("FH", "in", "d", "cat", "C", "N", "edge"):
        for classes in (1, 3, 7):
            report = gpu.honest_quotient(domain, 2, classes)
            assert report["identity_holds"] == 1, (domain, classes, report)
            if classes == 1:
                assert report["remainder_rows"] == 0, (domain, report)
            if domain != "edge" or classes == 1:
                assert report == cpu.honest_quotient(domain, 2, classes), (domain, classes)
    assert gpu.honest_quotient("in", 1, 1)["identity_holds"] == 0
    cpu.close()
    gpu.close()
