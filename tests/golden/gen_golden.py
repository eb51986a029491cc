"""Generates the golden vectors of the quantizer from the reference's own header.

Run in a container that holds the reference tree (the oracle Makefile compiles
python/fish_scales_ops/include/fso/activation_contract.h into oracle/_ref/libfso_ref_contract.so):

    python tests/golden/gen_golden.py

Writes tests/golden/quantize_1x32.npz:
  edge_x_bits, edge_q, edge_sf      the corner-case activation of tests/inputs.py (full bytes)
  cfg1_x_sha, cfg1_w_sha            sha256 of (codes || words) of the seed-0 [128,512] activation and [256,512] weight
  cfg1_x_q_head, cfg1_x_sf          first 8 rows of codes and all scale words of that activation
"""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

import inputs  # noqa: E402
from oracle import oracle as O  # noqa: E402


def sha(q, sf):
    return hashlib.sha256(q.tobytes() + sf.tobytes()).hexdigest()


def main():
    O.build()
    assert O.ref_lib() is not None, "the reference-header shim is not built (needs the reference tree)"
    edge = inputs.edge_activation()
    eq, es = O.ref_quantize_1x32(edge)
    x = inputs.activation(128, 512, 0)
    w = inputs.weight(256, 512, 1)
    xq, xs = O.ref_quantize_1x32(x)
    wq, ws = O.ref_quantize_1x32(w)
    np.savez_compressed(os.path.join(HERE, "quantize_1x32.npz"), edge_x_bits=O.bf16_bits(edge), edge_q=eq, edge_sf=es,
                        cfg1_x_sha=np.array(sha(xq, xs)), cfg1_w_sha=np.array(sha(wq, ws)), cfg1_x_q_head=xq[:8],
                        cfg1_x_sf=xs)
    print("wrote quantize_1x32.npz", os.path.getsize(os.path.join(HERE, "quantize_1x32.npz")), "bytes")


if __name__ == "__main__":
    main()
