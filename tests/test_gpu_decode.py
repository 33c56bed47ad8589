"""Paged grouped-query decode attention on the GPU against the CPU oracle and the committed
fixture: benchmark configuration 1, the reference's own test shapes (ragged lengths 37/1/64, an empty
sequence, lengths that end mid-page), both head dims of the TMA path, the generic path, and at
full Llama-3-8B decode size a linearity property that needs no oracle."""
import os

import numpy as np
import pytest

import oracle
from refs import paged_case, paged_ref, rel_err
from tessel_b200.gpu import F32

pytestmark = pytest.mark.gpu
h, f, i32 = np.float16, np.float32, np.int32
TOL = 2e-3
HERE = os.path.dirname(os.path.abspath(__file__))


def decode(gpu, q, kc, vc, table, lens, scale, name="decode_attention"):
    arrays = [q, kc, vc, table, lens, np.zeros(q.shape, h)]
    bufs = [gpu.tensor(a) for a in arrays]
    k = gpu.kernel(name, [a.shape for a in arrays])
    gpu.launch(k, bufs + [F32(scale)])
    gpu.sync()
    o = gpu.fetch(bufs[5], h, q.shape)
    for b in bufs:
        gpu.free(b)
    return o


def check(got, want, lens):
    live = np.asarray(lens) > 0
    assert np.isnan(got[~live].astype(f)).all(), "an empty sequence is 0/0 = NaN, as in the reference"
    if live.any():
        assert not np.isnan(got[live].astype(f)).any()
        assert rel_err(got[live], want[live]) <= TOL


def test_config1_matches_oracle_and_fixture(gpu):
    from golden.make_golden import config1_inputs
    c = config1_inputs()
    got = decode(gpu, c["q"], c["kc"], c["vc"], c["table"], c["lens"], float(c["scale"]))
    want = np.load(os.path.join(HERE, "golden", "decode_config1.npz"))["o"]
    assert rel_err(got, want) <= TOL
    assert rel_err(got, paged_ref(c["q"], c["kc"], c["vc"], c["table"], c["lens"], float(c["scale"]))) <= TOL


@pytest.mark.parametrize("H,G,D,P,lens", [
    (2, 2, 32, 16, [37, 1, 64]),            # tests/interp.rs:126-136 (generic path: D = 32)
    (4, 2, 64, 16, [5, 64, 0]),             # examples/metal_cases.rs:296-309
    (8, 2, 64, 16, [37, 128, 300, 511]),
    (32, 8, 128, 16, [1, 15, 16, 17, 1000, 2303, 0, 512]),
    (32, 4, 64, 16, [700, 33, 1152]),       # TinyLlama grouping: 8 query heads per KV head
    (16, 1, 128, 16, [100, 260]),           # multi-query: 16 heads on one KV head (two head groups)
    (4, 2, 16, 8, [9, 40, 64]),             # the tiny test model: page 8, D = 16 (generic path)
])
def test_against_oracle(gpu, H, G, D, P, lens):
    r = oracle.Rng(21)
    q, kc, vc, table, ln, scale = paged_case(r, len(lens), H, D, P, lens, g=G)
    got = decode(gpu, q, kc, vc, table, ln, scale)
    check(got, oracle.decode_attention(q, kc, vc, table, ln, scale), lens)


@pytest.mark.parametrize("splits,lens", [
    (1, [300, 0, 17, 1000, 64]),              # one split: the kernel writes O itself (and the NaN row)
    (5, [300, 0, 17, 1000, 64, 2]),           # five splits: partials merged by the second kernel
    (2, [1, 0, 16, 33, 2303, 512, 100]),
])
def test_forced_split_counts(gpu, monkeypatch, splits, lens):
    """Both ways of finishing (direct, or split-KV partials + merge) on the same kind of input;
    the split count is fixed when the kernel is made, so each case has its own batch size."""
    monkeypatch.setenv("TB200_DECODE_SPLITS", str(splits))
    r = oracle.Rng(31 + splits)
    q, kc, vc, table, ln, scale = paged_case(r, len(lens), 32, 128, 16, lens, g=8)
    got = decode(gpu, q, kc, vc, table, ln, scale)
    check(got, oracle.decode_attention(q, kc, vc, table, ln, scale), lens)


def test_paged_attention_name(gpu):
    """kernels/attention.tl:29-51 is the same computation with one KV head per query head."""
    r = oracle.Rng(22)
    q, kc, vc, table, ln, scale = paged_case(r, 3, 4, 64, 16, [37, 1, 64])
    got = decode(gpu, q, kc, vc, table, ln, scale, name="paged_attention")
    check(got, oracle.decode_attention(q, kc, vc, table, ln, scale), [37, 1, 64])


def test_out_of_range_pages_read_zero(gpu):
    """A block-table entry outside the pool reads K = V = 0 (masked load), it does not fault."""
    r = oracle.Rng(23)
    q, kc, vc, table, ln, scale = paged_case(r, 2, 8, 128, 16, [48, 80], g=2)
    table[0, 1] = kc.shape[0] + 5
    table[1, 2] = -3
    got = decode(gpu, q, kc, vc, table, ln, scale)
    check(got, oracle.decode_attention(q, kc, vc, table, ln, scale), [48, 80])


@pytest.mark.parametrize("splits", [1, 3])
def test_lengths_past_the_block_table_see_page_zero(gpu, monkeypatch, splits):
    """A length beyond MP * P (the device-side step advance can grow one there): the reference's
    masked table load reads 0 past the row, so those tokens attend to page 0; nothing reads past
    the table or the split scratch, with one split and with several."""
    monkeypatch.setenv("TB200_DECODE_SPLITS", str(splits))
    r = oracle.Rng(40 + splits)
    lens = [70, 200, 16 * 9 + 5, 40 + splits]  # the table below is 8 pages wide: 128 tokens
    q, kc, vc, table, ln, scale = paged_case(r, len(lens), 32, 128, 16, [min(l, 128) for l in lens], g=8)
    table = np.ascontiguousarray(table[:, :8])
    ln = np.asarray(lens, i32)
    got = decode(gpu, q, kc, vc, table, ln, scale)
    check(got, oracle.decode_attention(q, kc, vc, table, ln, scale), lens)


def test_llama8b_decode_size_properties(gpu):
    """Llama-3-8B decode shape (256 sequences, 32 heads on 8 KV heads, D 128, contexts up to
    2304) on a 2 GB cache: (1) a sampled subset of sequences matches the oracle; (2) with V set
    to a per-token constant c[t] replicated over D, every output element equals the softmax-
    weighted mean of c, so all D columns of a head agree; (3) permuting which physical page holds
    which tokens (and the table with it) changes nothing."""
    g = np.random.default_rng(5)
    B, H, G, D, P, MP = 256, 32, 8, 128, 16, 144
    lens = g.integers(512, 2305, B).astype(i32)
    lens[:4] = [2304, 513, 1, 0]
    need = int(sum(-(-int(l) // P) for l in lens))
    NP = need + 7
    kc = (g.standard_normal((NP, P, G, D), dtype=f)).astype(h)
    vc = (g.standard_normal((NP, P, G, D), dtype=f)).astype(h)
    q = g.standard_normal((B, H, D), dtype=f).astype(h)
    perm = g.permutation(NP).astype(i32)
    table = np.zeros((B, MP), i32)
    nxt = 0
    for b in range(B):
        n = -(-int(lens[b]) // P)
        table[b, :n] = perm[nxt:nxt + n]
        nxt += n
    scale = 1.0 / np.sqrt(128.0)
    got = decode(gpu, q, kc, vc, table, lens, scale)
    sub = [0, 1, 2, 3, 77, 255]
    want = oracle.decode_attention(q[sub], kc, vc, table[sub], lens[sub], scale)
    check(got[sub], want, lens[sub])
    # (3) physical page order is invisible.
    p2 = g.permutation(NP)
    inv = np.empty(NP, np.int64)
    inv[p2] = np.arange(NP)
    got2 = decode(gpu, q, kc[p2], vc[p2], inv[table].astype(i32), lens, scale)
    live = lens > 0
    assert np.array_equal(got2[live].view(np.uint16), got[live].view(np.uint16))
    # (2) constant-over-D values.
    vconst = np.repeat(vc[..., :1], D, axis=-1)
    got3 = decode(gpu, q, kc, vconst, table, lens, scale)[live].astype(f)
    assert np.abs(got3 - got3[..., :1]).max() == 0.0
