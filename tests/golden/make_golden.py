"""Generates the committed fixtures of tests/golden/ from the CPU oracle.

    python tests/golden/make_golden.py

The reference (Rust) cannot be built where this runs, and its tests hold no stored vectors,
so these are the ORACLE's outputs on seeded inputs: they pin the oracle against silent
change and let a GPU box check results without recomputing them. Inputs are regenerated
from their seeds (`config1_inputs`), only outputs are stored.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))


def config1_inputs(seed: int = 1):
    """benchmark configuration 1: 4 sequences with contexts 37/128/300/511, 8 query heads, 2 KV heads,
    head_dim 64, page size 16, block tables a seeded permutation of a 128-page pool, Q/K/V
    f16 ~N(0,1), scale 1/sqrt(64)."""
    g = np.random.default_rng(seed)
    lens = np.asarray([37, 128, 300, 511], np.int32)
    B, H, G, D, P, NP, MP = 4, 8, 2, 64, 16, 128, 32
    q = g.standard_normal((B, H, D), dtype=np.float32).astype(np.float16)
    kc = g.standard_normal((NP, P, G, D), dtype=np.float32).astype(np.float16)
    vc = g.standard_normal((NP, P, G, D), dtype=np.float32).astype(np.float16)
    perm = g.permutation(NP).astype(np.int32)
    table = np.zeros((B, MP), np.int32)
    nxt = 0
    for b in range(B):
        n = -(-int(lens[b]) // P)
        table[b, :n] = perm[nxt:nxt + n]
        nxt += n
    return dict(q=q, kc=kc, vc=vc, table=table, lens=lens, scale=np.float32(0.125))


def main():
    import oracle
    c = config1_inputs()
    o = oracle.decode_attention(c["q"], c["kc"], c["vc"], c["table"], c["lens"], float(c["scale"]))
    np.savez_compressed(os.path.join(HERE, "decode_config1.npz"), o=o)
    print("decode_config1.npz", o.shape)


if __name__ == "__main__":
    main()
