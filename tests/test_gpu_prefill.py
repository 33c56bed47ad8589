"""Causal FlashAttention (packed GQA prefill and the plain [H,S,D] layout) against the CPU
oracle and the f64 procedure of the reference's tests."""
import numpy as np
import pytest

import oracle
from refs import attention_ref, rel_err
from tessel_b200.gpu import F32

pytestmark = pytest.mark.gpu
h, f, i32 = np.float16, np.float32, np.int32
TOL = 2e-3


def prefill(gpu, q, k, v, starts, scale):
    arrays = [q, k, v, starts, np.zeros(q.shape, h)]
    bufs = [gpu.tensor(a) for a in arrays]
    kern = gpu.kernel("prefill_attention", [a.shape for a in arrays])
    gpu.launch(kern, bufs + [F32(scale)])
    gpu.sync()
    o = gpu.fetch(bufs[4], h, q.shape)
    for b in bufs:
        gpu.free(b)
    return o


def flash(gpu, q, k, v, scale):
    arrays = [q, k, v, np.zeros(q.shape, h)]
    bufs = [gpu.tensor(a) for a in arrays]
    kern = gpu.kernel("flash_attention", [a.shape for a in arrays])
    gpu.launch(kern, bufs + [F32(scale)])
    gpu.sync()
    o = gpu.fetch(bufs[3], h, q.shape)
    for b in bufs:
        gpu.free(b)
    return o


def starts_of(lengths, total):
    s = np.arange(total, dtype=i32)  # padding rows start at themselves
    at = 0
    for n in lengths:
        s[at:at + n] = at
        at += n
    return s


@pytest.mark.parametrize("H,G,D,lengths,pad", [
    (4, 2, 64, [70, 26], 0),                 # examples/metal_cases.rs:176-177
    (4, 2, 64, [10], 6),                     # one prompt, padded to 16 rows
    (8, 2, 128, [300, 5, 129, 64], 14),      # blocks that straddle prompts; a start after a whole key block
    (32, 8, 128, [257], 255),
    (4, 2, 16, [70, 20], 38),                # the tiny test model (generic path)
    (2, 2, 32, [150], 0),
])
def test_packed_prefill(gpu, H, G, D, lengths, pad):
    S = sum(lengths) + pad
    r = oracle.Rng(41)
    q, k, v = r.tensor(h, (S, H, D)), r.tensor(h, (S, G, D)), r.tensor(h, (S, G, D))
    st = starts_of(lengths, S)
    scale = float(1.0 / np.sqrt(D))
    got = prefill(gpu, q, k, v, st, scale)
    want = oracle.prefill_attention(q, k, v, st, scale)
    assert not np.isnan(got.astype(f)).any()
    assert rel_err(got, want) <= TOL


@pytest.mark.parametrize("H,S,D", [(2, 150, 32), (3, 200, 64), (2, 384, 128), (1, 1, 128)])
def test_flash_attention(gpu, H, S, D):
    """tests/interp.rs:103-124 at (2, 150, 32), and tile-multiple / ragged lengths on the tensor-core path."""
    r = oracle.Rng(4)
    q, k, v = (r.tensor(h, (H, S, D)) for _ in range(3))
    scale = float(1.0 / np.sqrt(D))
    got = flash(gpu, q, k, v, scale)
    assert rel_err(got, oracle.flash_attention(q, k, v, scale)) <= TOL
    assert rel_err(got, attention_ref(q, k, v, scale)) <= 5e-3


def test_config3_shape_sampled(gpu):
    """benchmark configuration 3 (batch 8 x 32 heads folded into H = 256, S 4096, D 128, ~N(0,1)): a
    few (head, row-block) programs against the oracle; and the first row of every head
    attends to itself only, so O[h, 0] == V[h, 0] exactly."""
    g = np.random.default_rng(3)
    H, S, D = 256, 4096, 128
    q, k, v = (g.standard_normal((H, S, D), dtype=f).astype(h) for _ in range(3))
    scale = float(1.0 / np.sqrt(D))
    got = flash(gpu, q, k, v, scale)
    assert np.array_equal(got[:, 0].view(np.uint16), v[:, 0].view(np.uint16))
    for hh, blk in [(0, 0), (17, 31), (255, 63), (100, 7)]:
        want = oracle.flash_attention(q[hh:hh + 1], k[hh:hh + 1], v[hh:hh + 1], scale, blocks=(blk, blk + 1))
        rows = slice(blk * 64, blk * 64 + 64)
        assert rel_err(got[hh, rows], want[0, rows]) <= TOL


@pytest.mark.parametrize("G", [32, 8])
def test_config3_packed_form_sampled(gpu, G):
    """benchmark configuration 3 as the engine runs it: 8 prompts of 4096 tokens packed into one
    step (S = 32768, per-row starts), 32 query heads on 32 or 8 KV heads, D 128. Sampled 64-row
    blocks (the first and last of a prompt, one that a prompt boundary cuts just before) against
    the oracle; and the first row of every prompt attends to itself only, so O == V there."""
    g = np.random.default_rng(7)
    H, D, n, L = 32, 128, 8, 4096
    S = n * L
    q = g.standard_normal((S, H, D), dtype=f).astype(h)
    k, v = g.standard_normal((S, G, D), dtype=f).astype(h), g.standard_normal((S, G, D), dtype=f).astype(h)
    st = starts_of([L] * n, S)
    scale = float(1.0 / np.sqrt(D))
    got = prefill(gpu, q, k, v, st, scale)
    first = np.arange(n) * L
    rep = H // G
    assert np.array_equal(got[first].view(np.uint16), np.repeat(v[first], rep, axis=1).view(np.uint16))
    for blk in (0, L // 64 - 1, L // 64, 3 * L // 64 + 17, S // 64 - 1):
        rows = slice(blk * 64, blk * 64 + 64)
        lo = int(st[blk * 64])
        # The block's rows see keys [lo, blk * 64 + 64) only: the oracle on that window.
        w0, w1 = lo, blk * 64 + 64
        want = oracle.prefill_attention(q[w0:w1], k[w0:w1], v[w0:w1], (st[w0:w1] - lo).astype(i32), scale)
        assert rel_err(got[rows], want[-64:]) <= TOL, blk


@pytest.mark.parametrize("H,G,D,P,T,chunks", [
    # (row0, nrows, pos0): rows of the step, tokens at positions pos0 ... of their sequence
    (32, 8, 128, 16, 512, [(3, 300, 77), (303, 5, 0), (310, 128, 512)]),   # several 256-row CTAs; a start mid-page
    (32, 4, 64, 16, 256, [(0, 256, 1000)]),                                 # TinyLlama grouping, a long cached prefix
    (8, 2, 128, 16, 64, [(10, 48, 0), (58, 1, 333)]),                       # a first chunk (no cache yet); one row
    (4, 2, 32, 8, 64, [(5, 40, 9)]),                                        # generic path: D = 32, page 8
])
def test_chunk_attention_against_decode_rows(gpu, H, G, D, P, T, chunks):
    """Rows of prompts fed in pieces, attended through the paged cache: each row must equal the
    decode attention of the same query with the cache cut off after its own position (which is how
    the CPU engine computes it). Rows outside every chunk keep their contents."""
    r = oracle.Rng(61)
    g = np.random.default_rng(61)
    need = [-(-(pos0 + n) // P) for _, n, pos0 in chunks]
    MP, NP = max(need) + 1, sum(need) + 5
    order = g.permutation(NP)
    q = r.tensor(h, (T, H, D))
    kc, vc = r.tensor(h, (NP, P, G, D)), r.tensor(h, (NP, P, G, D))
    table = np.zeros((T, MP), i32)
    meta = np.zeros((4, 4), i32)
    at = 0
    for c, ((row0, n, pos0), pages) in enumerate(zip(chunks, need)):
        table[row0:row0 + n, :pages] = order[at:at + pages]
        at += pages
        meta[c, :3] = (row0, n, pos0)
    scale = float(1.0 / np.sqrt(D))
    sentinel = np.full((T, H, D), 7.0, h)
    arrays = [q, kc, vc, table, meta, sentinel]
    bufs = [gpu.tensor(a) for a in arrays]
    kern = gpu.kernel("chunk_attention", [a.shape for a in arrays])
    gpu.launch(kern, bufs + [F32(scale)])
    gpu.sync()
    got = gpu.fetch(bufs[5], h, q.shape)
    for b in bufs:
        gpu.free(b)
    touched = np.zeros(T, bool)
    for row0, n, pos0 in chunks:
        rows = np.arange(row0, row0 + n)
        touched[rows] = True
        lens = (pos0 + 1 + np.arange(n)).astype(i32)
        want = oracle.decode_attention(q[rows], kc, vc, table[rows], lens, scale)
        assert not np.isnan(got[rows].astype(f)).any()
        assert rel_err(got[rows], want) <= TOL, (row0, n, pos0)
    assert np.array_equal(got[~touched].view(np.uint16), sentinel[~touched].view(np.uint16))
