"""Synthetic weights for the benchmarks: random-init f16 ~N(0, 0.02), generated on the device.

The benchmark configurations name shapes, not checkpoints (no checkpoint or tokenizer ships with
this repository), so the model is drawn from seeds: every matrix in full from a seed of its own
(layer, role), of which a tensor-parallel rank keeps its rows or columns. The model is therefore
the same model at every number of GPUs."""
from __future__ import annotations

import numpy as np


def device_weights(cfg, rank, world, torch):
    """Random-init f16 weights ~N(0, 0.02) generated on the device. Every matrix is drawn in full
    from a seed of its own (layer, role) and this rank keeps its rows or columns of it, so the
    model is the same model at every N: a rank's shard at TP N is a slice of the TP 1 weights."""
    from tessel_b200.model import Config, DevArray, Layer, Weights
    gen = torch.Generator(device="cuda")
    keep = []
    H, G, D, F, dm = cfg.heads, cfg.kv_heads, cfg.head_dim, cfg.ffn, cfg.dim
    hl, gl, fl = H // world, G // world, F // world
    local = Config(**{**cfg.__dict__, "heads": hl, "kv_heads": gl, "ffn": fl})

    def full(r, c, seed):
        gen.manual_seed(seed)
        t = torch.empty((r, c), dtype=torch.float16, device="cuda")
        t.normal_(0.0, 0.02, generator=gen)
        return t

    def dev(t):
        t = t.contiguous()
        keep.append(t)
        return DevArray(t.data_ptr(), tuple(t.shape), np.float16, t)

    def ones(n):
        return dev(torch.ones((n,), dtype=torch.float16, device="cuda"))

    layers = []
    for l in range(cfg.layers):
        w = full(cfg.qkv(), dm, 16 * l + 1)
        q = w[rank * hl * D:(rank + 1) * hl * D]
        k = w[H * D + rank * gl * D:H * D + (rank + 1) * gl * D]
        v = w[(H + G) * D + rank * gl * D:(H + G) * D + (rank + 1) * gl * D]
        wqkv = dev(torch.cat([q, k, v], 0) if world > 1 else w)
        wo = dev(full(dm, H * D, 16 * l + 2)[:, rank * hl * D:(rank + 1) * hl * D])
        wg = dev(full(F, dm, 16 * l + 3)[rank * fl:(rank + 1) * fl])
        wu = dev(full(F, dm, 16 * l + 4)[rank * fl:(rank + 1) * fl])
        wd = dev(full(dm, F, 16 * l + 5)[:, rank * fl:(rank + 1) * fl])
        layers.append(Layer(ones(dm), wqkv, wo, ones(dm), wg, wu, wd))
    return Weights(local, dev(full(cfg.vocab, dm, 900001)), layers, ones(dm), dev(full(cfg.vocab, dm, 900002)))
