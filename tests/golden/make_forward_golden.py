"""Generates tests/golden/forward_head.npz: inputs and outputs of ONE attention head computed by the
reference's own Python forward pass, `head_forward` of scripts/gat_reference.py (dense-bias form,
lines 37-87), imported from the reference tree.  Run in a container that holds the reference:

    python tests/golden/make_forward_golden.py /path/to/reference

The fixture pins the oracle's restatement of attention_head_forward_impl (src/model/gat.cpp:474-615) to
reference-generated output.  numpy's matrix products sum in another order than the C++ loops, so the
comparison in tests/test_oracle.py is to 1e-12, not bit for bit.  Edge entries only are stored (the dense
N x N intermediates of the script are sampled at the graph's edges)."""
import os
import sys

import numpy as np


def main(reference_root):
    sys.path.insert(0, os.path.join(reference_root, "scripts"))
    import gat_reference  # the reference's script; needs numpy and scipy only

    rng = np.random.default_rng(20240611)
    nodes, inner, width, directed = 120, 17, 6, 700
    src = rng.integers(0, nodes, size=directed)
    dst = rng.integers(0, nodes, size=directed)
    keep = src != dst
    pairs = np.unique(np.stack([src[keep], dst[keep]], axis=1), axis=0)
    src = np.concatenate([pairs[:, 0], np.arange(nodes)])
    dst = np.concatenate([pairs[:, 1], np.arange(nodes)])
    order = np.argsort(dst, kind="stable")
    src, dst = src[order], dst[order]
    features = rng.normal(size=(nodes, inner))
    seq_kernel = rng.uniform(-0.4, 0.4, size=(1, inner, width))
    src_kernel = rng.uniform(-1, 1, size=(1, width, 1))
    dst_kernel = rng.uniform(-1, 1, size=(1, width, 1))
    src_bias, dst_bias = np.array([0.07]), np.array([-0.02])
    output_bias = rng.uniform(-0.3, 0.3, size=width)
    # adj_to_bias of scripts/planetoid_utils.py: 0 on edges (row = destination, column = source), -1e9 elsewhere
    bias = np.full((nodes, nodes), -1e9)
    bias[dst, src] = 0.0
    out = {}
    for tag, apply_bias, apply_activation in (("hidden", False, True), ("output", True, False)):
        trace = gat_reference.head_forward(features, bias, seq_kernel, dst_kernel, dst_bias, src_kernel, src_bias, output_bias,
                                           apply_output_bias=apply_bias, apply_activation=apply_activation)
        for name in ("H_prime", "E_src", "E_dst", "M", "Sum", "inv", "H_agg_pre_bias", "H_agg"):
            out[f"{tag}_{name}"] = np.asarray(trace[name], dtype=np.float64)
        for name in ("S", "Z", "Delta", "U", "alpha"):
            out[f"{tag}_{name}"] = np.asarray(trace[name], dtype=np.float64)[dst, src]
    here = os.path.dirname(os.path.abspath(__file__))
    np.savez_compressed(os.path.join(here, "forward_head.npz"), features=features, seq_kernel=seq_kernel[0], attn_src=src_kernel[0, :, 0],
                        attn_dst=dst_kernel[0, :, 0], attn_src_bias=src_bias, attn_dst_bias=dst_bias, output_bias=output_bias,
                        edge_src=src.astype(np.uint32), edge_dst=dst.astype(np.uint32), **out)
    print("wrote forward_head.npz:", {k: v.shape for k, v in out.items() if k.startswith("hidden")})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python make_forward_golden.py <checkout of the reference repository>")
    main(sys.argv[1])
