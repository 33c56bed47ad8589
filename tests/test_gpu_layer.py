"""One decoder layer and a slice of the LM head at the benchmark configurations' dimensions,
through ``Engine.launch_all`` on the GPU against the same engine on the CPU oracle.

The kernel tests cover these shapes one kernel at a time; this covers the layer as the
benchmark runs it: a decode step of 256 rows (Llama-3-8B shape, configuration 5) or 64 rows
(TinyLlama shape, configuration 4), so the tile plans the benchmark's projections pick are the
ones under test, and the shard a rank holds under 8-way tensor parallelism. The KV cache is
filled with random pages (prefilling it through the oracle would take minutes); a few sequences
have benchmark-sized contexts, the rest short ones, which keeps the oracle's attention cheap
while every row of the step is real. Compared: the residual stream x, the normalised h, the
attention output O, the logits (max |got - want| / max |want| <= 2e-3), and the cache rows the
step wrote: bit for bit against the oracle's kv_write applied to the GPU's own QKV."""
import numpy as np
import pytest

import oracle
from emu import EmuGpu
from refs import rel_err
from tessel_b200.engine import Decode, Engine, Limits
from tessel_b200.model import Config, Weights

pytestmark = pytest.mark.gpu
TOL = 2e-3
P = 16

CASES = {
    # rows, long sequences, context range of the long ones
    "llama3_8b": (Config(dim=4096, layers=1, heads=32, kv_heads=8, head_dim=128, ffn=14336, vocab=128256 // 8,
                         rope_theta=500000.0, max_pos=2304, eos=-1), 256, 16, (512, 2300)),
    "tinyllama": (Config(dim=2048, layers=1, heads=32, kv_heads=4, head_dim=64, ffn=5632, vocab=32000 // 8,
                         rope_theta=10000.0, max_pos=1152, eos=-1), 64, 16, (128, 1150)),
    # What one rank of an 8-way tensor-parallel Llama-3-8B run holds: 4 query heads, 1 KV head, 1792 MLP columns.
    "llama3_8b_tp8_shard": (Config(dim=4096, layers=1, heads=4, kv_heads=1, head_dim=128, ffn=14336 // 8,
                                   vocab=128256 // 8, rope_theta=500000.0, max_pos=2304, eos=-1), 256, 16, (512, 2300)),
}


@pytest.mark.parametrize("name", list(CASES))
def test_decoder_layer_and_head_slice(gpu, name):
    cfg, rows, nlong, (lo, hi) = CASES[name]
    w = Weights.gaussian(cfg, 5)
    g = np.random.default_rng(11)
    ctx = np.concatenate([g.integers(lo, hi + 1, nlong), g.integers(1, 18, rows - nlong)])  # cached tokens before this step
    g.shuffle(ctx)
    need = [-(-(int(c) + 1) // P) for c in ctx]
    mp = max(need)
    pages = sum(need) + 3
    lim = Limits(page=P, pages=pages, max_tokens=rows, max_seq_pages=mp)
    order = g.permutation(pages)  # block tables scattered over the pool
    tables, at = [], 0
    for n in need:
        tables.append(order[at:at + n].tolist())
        at += n
    G, D = cfg.kv_heads, cfg.head_dim
    kc0 = g.standard_normal((pages * P, G, D), dtype=np.float32).astype(np.float16)
    vc0 = g.standard_normal((pages * P, G, D), dtype=np.float32).astype(np.float16)
    toks = g.integers(0, cfg.vocab, rows).tolist()
    pos = [int(c) for c in ctx]
    slots = [tables[b][p // P] * P + p % P for b, p in enumerate(pos)]
    attn = Decode(tables, [p + 1 for p in pos])
    want_rows = list(range(rows))

    got = {}
    for kind, dev in (("gpu", gpu), ("cpu", EmuGpu())):
        e = Engine(dev, w, lim)
        e.graphs = False
        dev.write(e.layers[0].kc, 0, kc0)
        dev.write(e.layers[0].vc, 0, vc0)
        logits = e.step(toks, pos, slots, attn, want_rows).copy()
        got[kind] = dict(
            logits=logits,
            x=dev.fetch(e.x, np.float32, (e.tmax, cfg.dim))[:rows],
            h=dev.fetch(e.h, np.float16, (e.tmax, cfg.dim))[:rows],
            o=dev.fetch(e.o, np.float16, (e.tmax, cfg.heads * D))[:rows],
            qkv=dev.fetch(e.qkv, np.float16, (e.tmax, cfg.qkv()))[:rows],
            kc=dev.fetch(e.layers[0].kc, np.float16, (pages * P, G, D)),
            vc=dev.fetch(e.layers[0].vc, np.float16, (pages * P, G, D)))
        if kind == "gpu":
            C, S = oracle.rope_tables(cfg.max_pos, D, cfg.rope_theta)
    a, b = got["gpu"], got["cpu"]
    for key in ("qkv", "o", "x", "h", "logits"):
        assert rel_err(a[key], b[key]) <= TOL, f"{name}: {key} differs from the oracle by {rel_err(a[key], b[key]):.2e}"
    # The cache after the step: untouched slots keep their bits, the step's slots hold exactly
    # what the reference's kv_write makes of the QKV the GPU computed.
    kc_want, vc_want, _, _ = oracle.kv_write(a["qkv"], np.asarray(pos, np.int32), np.asarray(slots, np.int32), C, S,
                                             kc0, vc0, G, D)
    assert np.array_equal(a["kc"].view(np.uint16), kc_want.view(np.uint16)), "K pages are not bit-exact"
    assert np.array_equal(a["vc"].view(np.uint16), vc_want.view(np.uint16)), "V pages are not bit-exact"
    assert not np.array_equal(a["kc"][slots].view(np.uint16), kc0[slots].view(np.uint16)), "the step wrote its slots"
