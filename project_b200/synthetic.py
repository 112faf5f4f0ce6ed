"""Seeded synthetic inputs of the prover flow: a destination-sorted graph with one self loop per
node (the layout normalize_graph_input produces, src/data/loader.cpp:416-539), a feature matrix
and Glorot-style GAT parameters scaled so that every quantised witness value stays inside the
static lookup tables (|S|, |H_agg| <= 4096/16, M - Z < 2^range_bits/16: the guard the reference
enforces by throwing "escaped static table", src/protocol/trace.cpp:2025-2030, 2083-2088).

The real datasets and checkpoints of the reference are not available; these inputs copy their
shapes (node / edge / feature counts, head layout), not their values."""
import numpy as np


def make_graph(rng, nodes, directed_edges, power_law=False, symmetrize=False):
    """(src, dst) uint32 arrays: `directed_edges` random edges (with their reverses when `symmetrize`,
    the loader's symmetrize_edges switch), deduplicated, plus a self loop per node, stably sorted by
    destination."""
    if power_law:
        weights = (np.arange(1, nodes + 1, dtype=np.float64)) ** (-1.0 / 1.5)
        weights /= weights.sum()
        src = rng.choice(nodes, size=directed_edges, p=weights)
        dst = rng.integers(0, nodes, size=directed_edges)
    else:
        src = rng.integers(0, nodes, size=directed_edges)
        dst = rng.integers(0, nodes, size=directed_edges)
    if symmetrize:
        src, dst = np.concatenate([src, dst]), np.concatenate([dst, src])
    keep = src != dst
    keys = np.unique(src[keep].astype(np.int64) * nodes + dst[keep])  # ordered by (src, dst)
    src = np.concatenate([keys // nodes, np.arange(nodes)])
    dst = np.concatenate([keys % nodes, np.arange(nodes)])
    order = np.argsort(dst, kind="stable")
    return src[order].astype(np.uint32), dst[order].astype(np.uint32)


def make_features(rng, nodes, width, density=0.1, kind="exp"):
    """Row-normalised non-negative features (loader.cpp:18-34 normalises rows to sum 1); kind "gauss":
    dense N(0,1) values, unnormalised."""
    if kind == "gauss":
        return rng.standard_normal((nodes, width))
    mask = rng.random((nodes, width)) < density
    values = rng.exponential(1.0, size=(nodes, width)) if kind == "exp" else np.ones((nodes, width))
    feats = values * mask
    feats[np.arange(nodes), rng.integers(0, width, size=nodes)] += 1.0  # no empty rows
    feats /= feats.sum(axis=1, keepdims=True)
    # a 1/16 grid carries features through quantisation; scale rows so that entries are visible at that scale
    return feats * 8.0


def make_params(rng, feature_count, hidden, output_heads, class_count):
    """Flat float64 parameter block in the order gzk_flow_config documents.
    hidden: list of (heads, head_dim) per hidden layer."""
    blocks = []

    def head(input_dim, width):
        limit = np.sqrt(6.0 / (input_dim + width))
        blocks.append(rng.uniform(-limit, limit, size=(input_dim, width)).reshape(-1))
        blocks.append(rng.uniform(-0.5, 0.5, size=width))   # attn_src
        blocks.append(rng.uniform(-0.5, 0.5, size=width))   # attn_dst
        blocks.append(rng.uniform(-0.1, 0.1, size=2))       # the two attention biases
        blocks.append(rng.uniform(-0.25, 0.25, size=width))  # output bias

    input_dim = feature_count
    for heads, dim in hidden:
        for _ in range(heads):
            head(input_dim, dim)
        input_dim = heads * dim
    for _ in range(output_heads):
        head(input_dim, class_count)
    return np.concatenate(blocks).astype(np.float64)


def make_inputs(seed, nodes, directed_edges, feature_count, hidden, output_heads, class_count, density=0.1, power_law=False, symmetrize=False,
                feature_kind="exp"):
    rng = np.random.default_rng(seed)
    src, dst = make_graph(rng, nodes, directed_edges, power_law, symmetrize)
    return {
        "nodes": nodes, "feature_count": feature_count, "class_count": class_count, "hidden": list(hidden), "output_heads": output_heads,
        "edge_src": src, "edge_dst": dst, "features": make_features(rng, nodes, feature_count, density, feature_kind),
        "params": make_params(rng, feature_count, hidden, output_heads, class_count),
    }
