"""Parity of the memory-bound glue kernels with the CPU oracle, through the C ABI.
Bit-exact where the arithmetic is exact or rounded op by op (embed, rope_q, kv_write pages
and block-table indexing, argmax); 2e-3 of the largest value elsewhere."""
import numpy as np
import pytest

import oracle
from refs import rel_err
from tessel_b200.gpu import F32

pytestmark = pytest.mark.gpu
h, f, i32 = np.float16, np.float32, np.int32
TOL = 2e-3  # relative to the largest reference value (the target for this path)


def run(gpu, name, arrays, outs, scalars=()):
    """Uploads `arrays`, launches `name` on their shapes, returns the arrays at indices `outs`."""
    bufs = [gpu.tensor(a) for a in arrays]
    k = gpu.kernel(name, [a.shape for a in arrays])
    gpu.launch(k, bufs + [F32(s) for s in scalars])
    gpu.sync()
    res = [gpu.fetch(bufs[i], arrays[i].dtype, arrays[i].shape) for i in outs]
    for b in bufs:
        gpu.free(b)
    return res


@pytest.mark.parametrize("T,V,Dm", [(16, 300, 128), (5, 64, 24), (256, 1000, 4096), (3, 7, 6)])
def test_embed(gpu, T, V, Dm):
    r = oracle.Rng(1)
    tok = (np.arange(T) * 37 % V).astype(i32)
    if T > 4:
        tok[1], tok[3] = -1, V
    E = r.tensor(h, (V, Dm))
    (x,) = run(gpu, "embed", [tok, E, np.full((T, Dm), 7, f)], [2])
    assert np.array_equal(x, oracle.embed(tok, E))


@pytest.mark.parametrize("T,Dm", [(16, 128), (256, 4096), (64, 2048), (3, 64), (2, 8200), (17, 700)])
def test_rmsnorm(gpu, T, Dm):
    r = oracle.Rng(2)
    x, w = r.tensor(f, (T, Dm), 2.0), r.tensor(h, (Dm,))
    (y,) = run(gpu, "rmsnorm", [x, w, np.zeros((T, Dm), h)], [2], [1e-5])
    want = oracle.rmsnorm(x, w, 1e-5)
    assert rel_err(y, want) <= TOL
    # Only the f32 sum's order differs: at most one f16 step anywhere.
    assert np.abs(y.view(np.int16).astype(int) - want.view(np.int16).astype(int)).max() <= 1


def test_rmsnorm_rows(gpu):
    r = oracle.Rng(3)
    T, Dm = 64, 2048
    x, w = r.tensor(f, (T, Dm), 2.0), r.tensor(h, (Dm,))
    idx = np.asarray([15, 3, 0, 63, 9, 9, -1, 64], i32)  # out-of-range rows read zeros
    (y,) = run(gpu, "rmsnorm_rows", [x, idx, w, np.ones((8, Dm), h)], [3], [1e-5])
    want = oracle.rmsnorm_rows(x, idx, w, 1e-5)
    assert rel_err(y, want) <= TOL
    assert not y[6].any() and not y[7].any()


@pytest.mark.parametrize("T,H,G,D,NPOS", [(16, 4, 2, 64, 64), (256, 32, 8, 128, 2304), (7, 4, 2, 16, 32)])
def test_rope_q_and_kv_write_bit_exact(gpu, T, H, G, D, NPOS):
    """KV-cache pages, the dense K/V rows and the rotated queries carry exactly the oracle's bits;
    padding rows (slot == NS) and out-of-range slots leave the cache untouched."""
    r = oracle.Rng(4)
    W = (H + 2 * G) * D
    P, NPG = 16, (T + 15) // 16 + 3
    NS = P * NPG
    qkv = r.tensor(h, (T, W))
    pos = ((np.arange(T) * 3) % NPOS).astype(i32)
    pos[-1] = NPOS  # outside the tables: cos = sin = 0
    Ct, St = oracle.rope_tables(NPOS, D, 10000.0)
    perm = np.random.default_rng(0).permutation(NS)[:T].astype(i32)
    slot = perm.copy()
    slot[-2:] = NS  # padding
    slot[0] = -5
    (q,) = run(gpu, "rope_q", [qkv, pos, Ct, St, np.zeros((T, H, D), h)], [4])
    assert np.array_equal(q.view(np.uint16), oracle.rope_q(qkv, pos, Ct, St, H, D).view(np.uint16))
    kc0, vc0 = r.tensor(h, (NS, G, D)), r.tensor(h, (NS, G, D))  # a cache already in use
    kc, vc, kd, vd = run(gpu, "kv_write", [qkv, pos, slot, Ct, St, kc0, vc0, np.zeros((T, G, D), h),
                                           np.zeros((T, G, D), h)], [5, 6, 7, 8])
    wkc, wvc, wkd, wvd = oracle.kv_write(qkv, pos, slot, Ct, St, kc0, vc0, G, D)
    for got, want in ((kc, wkc), (vc, wvc), (kd, wkd), (vd, wvd)):
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    # The engine's one-launch form of the two kernels gives the same bits.
    q2, kc2, vc2, kd2, vd2 = run(gpu, "rope_kv", [qkv, pos, slot, Ct, St, np.zeros((T, H, D), h), kc0, vc0,
                                                  np.zeros((T, G, D), h), np.zeros((T, G, D), h)], [5, 6, 7, 8, 9])
    for got, want in ((q2, q), (kc2, wkc), (vc2, wvc), (kd2, wkd), (vd2, wvd)):
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


@pytest.mark.parametrize("plan,T,K,H,G,D", [
    (None, 256, 512, 32, 8, 128),            # the Llama-3-8B heads, whatever tile the library picks
    ("2,256,1", 250, 264, 4, 2, 128), ("1,128,1", 100, 136, 6, 1, 64), ("2,128,2", 256, 1032, 6, 2, 64),
    ("2,256,2", 256, 1040, 4, 2, 128), ("3,256,1", 256, 520, 8, 4, 64), ("3,128,1", 200, 272, 5, 1, 128),
    ("3,256,2", 256, 2056, 12, 2, 128), ("3,128,2", 256, 1096, 6, 1, 64), ("1,256,4", 128, 2048, 8, 4, 64),
])
def test_projection_with_rope_and_kv_write_as_its_epilogue(gpu, monkeypatch, plan, T, K, H, G, D):
    """linear_rope_kv: the product it stores is `linear`'s (within tolerance of the oracle), and
    Q, the dense K and V and the cache pages are exactly what the oracle's rope_q and kv_write make
    of THAT product - bit for bit, through every tile, the CTA-pair kernel and the split-K exchange
    (whose unit ownership goes by heads here); dropped writes and positions outside the tables
    included."""
    if plan:
        monkeypatch.setenv("TB200_GEMM_PLAN", plan)
    r = oracle.Rng(6)
    W = (H + 2 * G) * D
    NPOS, P = 96, 16
    NS = P * ((T + 15) // 16 + 3)
    x, w = r.tensor(h, (T, K)), r.tensor(h, (W, K), 0.1)
    pos = ((np.arange(T) * 7) % NPOS).astype(i32)
    pos[-1] = NPOS
    Ct, St = oracle.rope_tables(NPOS, D, 10000.0)
    slot = np.random.default_rng(1).permutation(NS)[:T].astype(i32)
    slot[-2:] = NS
    slot[0] = -5
    kc0, vc0 = r.tensor(h, (NS, G, D)), r.tensor(h, (NS, G, D))
    z = lambda *shape: np.zeros(shape, h)
    qkv, q, kc, vc, kd, vd = run(gpu, "linear_rope_kv", [x, w, pos, slot, Ct, St, z(T, W), z(T, H, D), kc0, vc0,
                                                         z(T, G, D), z(T, G, D)], [6, 7, 8, 9, 10, 11])
    assert rel_err(qkv, oracle.linear(x, w)) <= TOL
    assert np.array_equal(q.view(np.uint16), oracle.rope_q(qkv, pos, Ct, St, H, D).view(np.uint16))
    wkc, wvc, wkd, wvd = oracle.kv_write(qkv, pos, slot, Ct, St, kc0, vc0, G, D)
    for name, got, want in (("Kc", kc, wkc), ("Vc", vc, wvc), ("K", kd, wkd), ("V", vd, wvd)):
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16)), name


def test_residual_add_and_argmax(gpu):
    r = oracle.Rng(5)
    a, b = r.tensor(f, (64, 512)), r.tensor(f, (64, 512))
    (s,) = run(gpu, "residual_add", [a, b], [0])
    assert np.array_equal(s, a + b)
    x = r.tensor(f, (33, 5000))
    x[0, 17] = x[0, 4000] = 5.0   # ties: the first wins
    x[1, 4999] = 9.0
    x[2, 0] = 9.0
    x[3, :] = 1.0
    x[4, 100] = np.nan            # a NaN never wins
    x[5, 0] = np.nan              # ... unless it is first: then nothing beats it
    (pick,) = run(gpu, "argmax_rows", [x, np.zeros(33, i32)], [1])
    want = np.asarray([oracle.argmax(row) for row in x], i32)
    assert np.array_equal(pick, want)
    assert pick[0] == 17 and pick[1] == 4999 and pick[2] == 0 and pick[3] == 0 and pick[5] == 0
    # A row length that is not a multiple of four takes the scalar scan.
    y = np.ascontiguousarray(x[:, :4999])
    y[1, 4998] = 9.0
    (pick,) = run(gpu, "argmax_rows", [y, np.zeros(33, i32)], [1])
    assert np.array_equal(pick, np.asarray([oracle.argmax(row) for row in y], i32))


@pytest.mark.parametrize("R", [2, 4, 8])
def test_argmax_over_a_split_vocabulary(gpu, R):
    """argmax_partial on each of R column slices, the slots summed as the allreduce sums them,
    then argmax_merge: the token the whole-row scan picks."""
    from tessel_b200.gpu import I32
    r = oracle.Rng(6)
    M, V = 19, 4096
    vs = V // R
    x = r.tensor(f, (M, V))
    x[0, 17] = x[0, V - 3] = 5.0           # a tie across slices: the first wins
    x[1, V - 1] = 9.0
    x[2, :] = 1.0                          # all equal: index 0
    x[3, 100] = np.nan                     # a NaN inside never wins
    x[4, 0] = np.nan                       # a NaN first sticks
    x[5, vs] = np.nan                      # a later slice that begins with NaN is still searched
    x[5, vs + 5] = 7.0
    x[6, vs:2 * vs] = np.nan               # a slice with nothing to offer
    x[7, :] = -np.inf
    x[8, :vs] = -np.inf                    # the first slice offers only -inf
    total = np.zeros((R, M, 2), f)
    for rank in range(R):
        part = np.ascontiguousarray(x[:, rank * vs:(rank + 1) * vs])
        bufs = [gpu.tensor(part), gpu.tensor(np.full((R, M, 2), 3.0, f))]
        k = gpu.kernel("argmax_partial", [part.shape, (R, M, 2)])
        gpu.launch(k, bufs + [I32(rank), I32(rank * vs)])
        gpu.sync()
        pr = gpu.fetch(bufs[1], f, (R, M, 2))
        others = [q for q in range(R) if q != rank]
        assert not pr[others].any(), "the other ranks' slots must be zero"
        total += pr
        for b in bufs:
            gpu.free(b)
    (pick,) = run(gpu, "argmax_merge", [total, np.zeros(M, i32)], [1], scalars=())
    want = np.asarray([oracle.argmax(row) for row in x], i32)
    assert np.array_equal(pick, want)
    assert pick[0] == 17 and pick[4] == 0 and pick[5] == vs + 5 and pick[7] == 0


def test_argument_checks(gpu):
    from tessel_b200.gpu import GpuError
    with pytest.raises(GpuError, match="no kernel"):
        gpu.kernel("nope", [[1]])
    with pytest.raises(GpuError, match="takes 3 arrays"):
        gpu.kernel("embed", [[4], [8, 8]])
    k = gpu.kernel("embed", [[4], [8, 8], [4, 8]])
    with pytest.raises(GpuError, match="takes 3 arguments"):
        gpu.launch(k, [])
    b = gpu.alloc(64)
    with pytest.raises(GpuError, match="write of 128 bytes"):
        gpu.write(b, 0, np.zeros(128, np.uint8))
    with pytest.raises(GpuError, match="read of"):
        gpu.read(b, 32, np.zeros(64, np.uint8))
    assert not gpu.fetch(b, np.uint8, (64,)).any(), "alloc must zero-fill"
    with pytest.raises(GpuError, match="bytes requested"):
        gpu.alloc(1 << 50)
    gpu.free(b)
