"""The prover flow over the CPU restatement: structure of the proof it produces.  (The comparison
with the GPU backend is tests/test_gpu_proof_parity.py.)"""
import pytest
import numpy as np

import oracle_lib as ora
import pyref
from project_b200 import synthetic
from project_b200.flow import Flow

G = np.frombuffer(pyref.g1_bytes((pyref.GX, pyref.GY)), dtype=np.uint8).copy()


def run(shape):
    flow = Flow(ora.lib(), "ora_flow_", 2, synthetic.make_inputs(**shape), G)
    flow.prove()
    return flow


def test_label_counts_follow_the_protocol_order():
    """#dynamic commitments = 5 + 82 H + 5 L + 68 K + 2 [K > 1] (src/protocol/challenges.cpp:396-507); the
    opened labels per domain: edge 43 H + 36 K, in 3 H, d 15 H, cat 3 L + 3 K, C 9 K, N 18 H + 17 K + L."""
    # the head layout of the small citation configuration (8 hidden heads of width 8, one output head):
    # 734 dynamic commitments
    flow = run(dict(seed=5, nodes=24, directed_edges=60, feature_count=6, hidden=[(8, 8)], output_heads=1, class_count=7))
    stats = flow.stats()
    assert stats["dynamic_commitments"] == 734
    h, k, layers = 8, 1, 1
    expect = {"edge": 43 * h + 36 * k, "in": 3 * h, "d": 15 * h, "cat": 3 * layers + 3 * k, "C": 9 * k, "N": 18 * h + 17 * k + layers}
    for domain, count in expect.items():
        assert len(flow.domain_labels(domain)) == count, domain
    # proof_size_bytes (src/protocol/prover.cpp:3831-3905) of the serialised proof: 48-byte points, 32-byte
    # values, (#labels + 1) rows of two values per bundle
    listing = flow.dump()
    rows = sum(1 for line in listing.splitlines() if line.startswith("opened "))
    assert rows == sum(expect.values()) + 5 + 7  # + the five feature-domain labels + one quotient row per bundle
    size = len(flow.proof_bytes())
    commitments = 734
    ext = sum(1 for line in listing.splitlines() if line.startswith("external "))
    scalars = sum(1 for line in listing.splitlines() if line.startswith("witness_scalar "))
    meta = sum(1 for _ in range(24)) * 8
    fixed = 8 + 8 + 8 + 48 * commitments + 8 + 48 * 7 + 8 + 7 * (8 + 48) + rows * (8 + 64) + 8 + 32 * ext + 8 + 32 * scalars + 48
    blocks = sum(8 + len(b) for b in ["M_pub", "Com_dyn", "S_route", "Eval_ext", "Eval_dom", "Com_quot", "Open_dom", "W_ext", "Pi_bind"])
    # what is left are the metadata strings themselves
    assert size - fixed - blocks - meta > 0
    flow.close()


def test_two_proofs_of_one_context_are_identical_and_inputs_matter():
    shape = dict(seed=6, nodes=30, directed_edges=80, feature_count=8, hidden=[(2, 4)], output_heads=2, class_count=3)
    flow = run(shape)
    first = flow.proof_bytes().copy()
    flow.prove()
    assert np.array_equal(first, flow.proof_bytes())
    other = run(dict(shape, seed=7))
    assert not np.array_equal(first[-4000:], other.proof_bytes()[-4000:])
    flow.close()
    other.close()


def test_prefix_stored_columns_give_the_same_proof():
    """compact_columns stores the edge-domain columns as prefixes (running sums up to their final value,
    which the remaining rows repeat); every challenge, evaluation, commitment and opened value must equal
    the whole-domain run's.  The second shape has node_count x head_dim above the largest lookup table, so
    the ELU lookup columns are longer than the other edge columns."""
    for shape in (dict(seed=6, nodes=30, directed_edges=80, feature_count=8, hidden=[(2, 4)], output_heads=2, class_count=3),
                  dict(seed=8, nodes=200, directed_edges=500, feature_count=6, hidden=[(1, 128)], output_heads=1, class_count=3)):
        inputs = synthetic.make_inputs(**shape)
        full = Flow(ora.lib(), "ora_flow_", 2, inputs, G)
        compact = Flow(ora.lib(), "ora_flow_", 2, inputs, G, compact_columns=True)
        full.prove()
        compact.prove()
        a, b = full.dump().splitlines(), compact.dump().splitlines()
        assert len(a) == len(b)
        differing = [(x, y) for x, y in zip(a, b) if x != y]
        assert not differing, differing[:3]
        assert np.array_equal(full.proof_bytes(), compact.proof_bytes())
        full.close()
        compact.close()


@pytest.mark.parametrize("output_heads,compact", [(1, False), (2, False), (1, True)])
def test_quotient_constraints_vanish_on_the_rows(output_heads, compact):
    """The constraint numerators of the seven quotients, restated from src/protocol/quotients.cpp, read at the points
    of a domain: every constraint that the witness of the reference's own builders satisfies must vanish on every row
    (the running-sum steps on every row but the last).  Which constraints are left out, and why, is stated where the
    numerators are written (ProverFlow::quotient_numerator)."""
    inputs = synthetic.make_inputs(seed=3, nodes=24, directed_edges=60, feature_count=6, hidden=[(2, 4)], output_heads=output_heads, class_count=3)
    flow = Flow(ora.lib(), "ora_flow_", 2, inputs, G, compact_columns=compact)
    flow.prove()
    bad, failures = flow.constraint_violations()
    flow.close()
    assert bad == [0] * 7, failures
    assert failures == []


def test_honest_quotients_divide():
    """The honest quotient of every domain (no counterpart in the reference, which commits t_D = N(tau)/Z(tau) by the
    trapdoor, src/protocol/prover.cpp:3076-3160): the numerator of the constraints that vanish on every row, extended
    through the transforms to four times the domain, divides by X^n - 1 without remainder; with the wrapping
    running-sum steps the remainder lives on the last row alone; the division identity N = t (X^n - 1) + R holds at a
    point outside the domains for every class of constraints; a blow-up too small for the numerator's degree is
    reported."""
    inputs = synthetic.make_inputs(seed=3, nodes=24, directed_edges=60, feature_count=6, hidden=[(2, 4)], output_heads=1, class_count=3)
    flow = Flow(ora.lib(), "ora_flow_", 2, inputs, G)
    flow.prove()
    bad, _ = flow.constraint_violations()
    assert bad == [0] * 7
    for domain in ("FH", "in", "d", "cat", "C", "N", "edge"):
        exact = flow.honest_quotient(domain, 2, 1)
        assert exact["remainder_rows"] == 0 and exact["identity_holds"] == 1, (domain, exact)
        assert exact["points"] == 4 * exact["n"]
        if exact["numerator_degree"] > 0:
            assert exact["quotient_degree"] == exact["numerator_degree"] - exact["n"], (domain, exact)
        if domain == "edge":
            continue  # 131072 points: the other classes of this domain are covered on the GPU
        wrapping = flow.honest_quotient(domain, 2, 3)
        assert wrapping["remainder_rows"] <= 1 and wrapping["identity_holds"] == 1, (domain, wrapping)
        everything = flow.honest_quotient(domain, 2, 7)
        assert everything["identity_holds"] == 1 and everything["remainder_rows"] >= wrapping["remainder_rows"], (domain, everything)
    # degree 3n - 3 (n = 8) does not fit 2n points
    assert flow.honest_quotient("in", 1, 1)["identity_holds"] == 0
    assert flow.honest_quotient("N", 3, 1) == dict(flow.honest_quotient("N", 2, 1), points=8 * 32)
    with pytest.raises(Exception):
        flow.honest_quotient("N", 0, 1)
    flow.close()
