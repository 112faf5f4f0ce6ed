"""Generates tests/golden/hotpath_small.json.

The reference cannot be built or imported here (its arithmetic library is
absent), so the vectors come from plain Python integer arithmetic (pyref.py),
which shares no code with the oracle or the CUDA library.  Run from the repo
root:  python tests/golden/make_golden.py
"""
import json
import os
import random
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import pyref  # noqa: E402
from pyref import R, fr_bytes  # noqa: E402


def main():
    rng = random.Random(20240611)
    out = {}
    out["omega"] = {"n": 1 << 22, "value": fr_bytes(pyref.root_of_unity(1 << 22)).hex()}

    x = rng.randrange(1 << 64)
    n = 64
    out["bary"] = {"n": n, "x": fr_bytes(x).hex(), "weights": b"".join(fr_bytes(v) for v in pyref.bary_weights(x, n)).hex()}

    k, n = 3, 32
    cols = [pyref.rand_fr(rng, n) for _ in range(k)]
    w = pyref.rand_fr(rng, n)
    rots = [0, 1, 5]
    res = []
    for rot in rots:
        for col in cols:
            res.append(sum(w[c] * col[(c + rot) % n] for c in range(n)) % R)
    out["eval"] = {
        "k": k, "n": n, "rotations": rots,
        "columns": b"".join(fr_bytes(v) for col in cols for v in col).hex(),
        "weights": b"".join(fr_bytes(v) for v in w).hex(),
        "out": b"".join(fr_bytes(v) for v in res).hex(),
    }

    G = (pyref.GX, pyref.GY)
    scalars = [0, 1, 28, R - 1] + pyref.rand_fr(rng, 4)
    out["g1_same_base"] = {
        "base": pyref.g1_bytes(G).hex(),
        "scalars": b"".join(fr_bytes(s) for s in scalars).hex(),
        "points": b"".join(pyref.g1_bytes(pyref.g1_mul(s, G)) for s in scalars).hex(),
    }

    n = 16
    table, query, mult = (pyref.rand_fr(rng, n) for _ in range(3))
    qt = [1] * 9 + [0] * 7
    qq = [1] * 13 + [0] * 3
    beta = rng.randrange(1 << 64)
    active = 13
    run, acc = 0, [0]
    for i in range(active):
        run = (run + qt[i] * mult[i] * pow(table[i] + beta, -1, R) - qq[i] * pow(query[i] + beta, -1, R)) % R
        acc.append(run)
    acc += [run] * (n - len(acc))
    enc = lambda v: b"".join(fr_bytes(a) for a in v).hex()
    out["logup"] = {"table": enc(table), "query": enc(query), "mult": enc(mult), "q_table": enc(qt), "q_query": enc(qq),
                    "beta": fr_bytes(beta).hex(), "active": active, "out": enc(acc)}

    with open(os.path.join(HERE, "hotpath_small.json"), "w") as f:
        json.dump(out, f, indent=1)


if __name__ == "__main__":
    main()
