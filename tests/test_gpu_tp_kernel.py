"""The tensor-parallel exchange kernels on one GPU.

The arithmetic and the data movement of ``linear_scatter`` and ``tp_reduce_norm`` with the peers
played by buffers of this GPU, and their failure detection without a second GPU: a rank whose
peers' partial rows never arrive, and finished rows that never land. In both, every pointer of
the table is valid, but nothing ever writes what the kernel waits for. The wait gives up after
its limit (one second), the kernel raises the context's status word and returns, `sync` reports
it, and the context keeps working."""
import time

import numpy as np
import pytest

from tessel_b200.gpu import F32, GpuError, I32

pytestmark = pytest.mark.gpu
f, hf = np.float32, np.float16
EMPTY = np.uint32(0xFFFFFFFF)


def group(gpu, n, T, dim, rank=0):
    """Buffers of an n-rank group, all on this GPU: inboxes and landing areas (every word empty),
    this rank's x and h."""
    def empty(nbytes):
        b = gpu.alloc(nbytes)
        gpu.fill(b, 0xFF)
        return b
    b = dict(part=[[empty((T + n) * dim * 4) for _ in range(n)] for _ in range(2)],
             stage=[empty(T * dim * 4) for _ in range(n)], x=gpu.alloc(T * dim * 4), h=gpu.alloc(T * dim * 2))
    gpu.sync()
    raw = gpu.tp_table(rank, n, b["part"][0], b["part"][1], b["stage"], b["x"], b["h"])
    b["table"] = gpu.tensor(np.frombuffer(raw, np.uint8).copy())
    return b


def inbox_image(n, T, dim, rows_of_source):
    """An inbox [n sources][ceil(T/n)][dim] f32 (as u32 words, empty beyond) holding, for every
    source, the rows it would have stored."""
    per = -(-T // n)
    words = np.full((T + n) * dim, EMPTY, np.uint32)
    box = words[:n * per * dim].reshape(n, per, dim)
    for s_, rows in enumerate(rows_of_source):
        box[s_, :len(rows)] = np.ascontiguousarray(rows, f).view(np.uint32)
    return words


def test_partials_that_never_arrive_are_reported_and_the_context_survives(gpu):
    T, dim = 16, 256
    b = group(gpu, 2, T, dim)  # rank 0's inbox holds its own partials only: rank 1's never come
    own = np.arange(T) % 2 == 0
    gpu.write(b["part"][0][0], 0, inbox_image(2, T, dim, [np.ones((int(own.sum()), dim), f)]))
    w = gpu.tensor(np.ones(dim, hf))
    k = gpu.kernel("tp_reduce_norm", [[b["table"].bytes], [dim], [T, dim]])
    t0 = time.perf_counter()
    gpu.launch(k, [b["table"], w, b["x"], F32(1e-5), I32(0), I32(1), I32(2)])
    with pytest.raises(GpuError, match="status 401"):
        gpu.sync()
    waited = time.perf_counter() - t0
    assert 0.3 < waited < 10.0, f"the wait limit is one second, the call took {waited:.2f} s"
    # The context is intact: the status was cleared by the report, and kernels run as before.
    gpu.sync()
    a, c = gpu.tensor(np.full((4, 8), 1.5, f)), gpu.tensor(np.full((4, 8), 2.0, f))
    gpu.launch(gpu.kernel("residual_add", [[4, 8], [4, 8]]), [a, c])
    gpu.sync()
    assert np.array_equal(gpu.fetch(a, f, (4, 8)), np.full((4, 8), 3.5, f))
    with pytest.raises(GpuError, match="nranks"):
        gpu.launch(k, [b["table"], w, b["x"], F32(1e-5), I32(0), I32(1), I32(1)])


def test_rows_that_never_land_are_reported(gpu):
    """Every source's partials are in the inbox, but the other owner's finished rows never arrive
    in this rank's landing area: the gather gives up in exactly that wait (status 402)."""
    T, dim = 16, 256
    b = group(gpu, 2, T, dim)
    rows = np.ones((T // 2, dim), f)
    gpu.write(b["part"][0][0], 0, inbox_image(2, T, dim, [rows, rows]))
    w = gpu.tensor(np.ones(dim, hf))
    k = gpu.kernel("tp_reduce_norm", [[b["table"].bytes], [dim], [T, dim]])
    gpu.launch(k, [b["table"], w, b["x"], F32(1e-5), I32(0), I32(1), I32(2)])
    with pytest.raises(GpuError, match="status 402"):
        gpu.sync()
    gpu.sync()


@pytest.mark.parametrize("n,T,dim", [(2, 16, 256), (3, 20, 8192), (8, 256, 4096), (4, 37, 1024)])
def test_one_rank_of_a_group_whose_peers_are_buffers(gpu, n, T, dim):
    """``tp_reduce_norm`` for rank 0 of ``n``, on one GPU and with no second kernel: the host puts
    into rank 0's inbox what the sources' projections would have stored, and into its landing
    area the rows the other owners would have sent, so it never waits. What rank 0 sends must
    appear in every peer's landing area, and everything it consumed must be empty again."""
    import oracle
    from refs import rel_err
    r = oracle.Rng(41 + n)
    b = group(gpu, n, T, dim)
    own = np.arange(T) % n == 0
    parts = [[r.tensor(f, (T, dim)) for _ in range(n)] for _ in range(2)]   # every source's whole partial product
    x0 = r.tensor(f, (T, dim))
    w = r.tensor(hf, (dim,))
    hs = [r.tensor(hf, (T, dim)) for _ in range(n)]     # what the other owners would have normalised
    xs = [r.tensor(f, (T, dim)) for _ in range(n)]      # ... and their final residual rows
    # One word that happens to hold the "empty" pattern's stand-in must travel like any other.
    parts[0][1][0, 3] = np.float32(np.nan)
    for wh in range(2):
        gpu.write(b["part"][wh][0], 0, inbox_image(n, T, dim, [parts[wh][s_][own] for s_ in range(n)]))
    gpu.write(b["x"], 0, x0)
    land = np.full((T, dim), EMPTY, np.uint32)
    for q in range(1, n):
        rows = np.arange(T) % n == q
        land.reshape(T * 2, dim // 2)[:T][rows] = hs[q][rows].view(np.uint32)   # [T][dim / 2] words of two halves
    gpu.write(b["stage"][0], 0, land)
    k = gpu.kernel("tp_reduce_norm", [[b["table"].bytes], [dim], [T, dim]])
    eps = 1e-5

    # Call 1: inbox 0, normalise, gather h.
    gpu.launch(k, [b["table"], gpu.tensor(w), b["x"], F32(eps), I32(0), I32(1), I32(n)])
    gpu.sync()
    want_x = x0.copy()
    acc = parts[0][0].copy()
    for q in range(1, n):
        acc = acc + parts[0][q]                                        # rank order, one rounded add each
    want_x[own] = (x0 + acc)[own]
    got_x = gpu.fetch(b["x"], f, (T, dim))
    fin = ~np.isnan(want_x)
    assert np.array_equal(np.isnan(got_x), ~fin) and np.array_equal(got_x[fin], want_x[fin]), \
        "own rows take the sum in rank order, the others stay"
    got_h = gpu.fetch(b["h"], hf, (T, dim))
    ok = ~np.isnan(want_x[own]).any(axis=1)
    want_h = oracle.rmsnorm(want_x, w, eps)
    assert rel_err(got_h[own][ok], want_h[own][ok]) < 2e-3
    assert np.isnan(got_h[0]).all(), "the row with a NaN partial normalises to NaN"
    for q in range(1, n):
        rows = np.arange(T) % n == q
        assert np.array_equal(got_h[rows].view(np.uint16), hs[q][rows].view(np.uint16)), "h rows taken from the landing area"
        sent = gpu.fetch(b["stage"][q], np.uint32, (T * 2, dim // 2))[:T]
        assert not (sent[own] == EMPTY).any(), "a NaN pair of halves is sent as another NaN, never as the empty word"
        sent_h = sent[own].view(hf)
        assert np.array_equal(np.isnan(sent_h), np.isnan(got_h[own])), "own h rows sent to every peer"
        m = ~np.isnan(sent_h)
        assert np.array_equal(sent_h[m], got_h[own][m])
        assert (sent[~own] == EMPTY).all()
    assert (gpu.fetch(b["stage"][0], np.uint32, (T * dim,)) == EMPTY).all(), "the landing area is empty again"
    assert (gpu.fetch(b["part"][0][0], np.uint32, ((T + n) * dim,)) == EMPTY).all(), "the inbox is empty again"

    # Call 2: inbox 1, no norm, gather x.
    land = np.full((T, dim), EMPTY, np.uint32)
    for q in range(1, n):
        rows = np.arange(T) % n == q
        land[rows] = xs[q][rows].view(np.uint32)
    gpu.write(b["stage"][0], 0, land)
    for q in range(1, n):
        gpu.fill(b["stage"][q], 0xFF)
    gpu.launch(k, [b["table"], gpu.tensor(w), b["x"], F32(eps), I32(1), I32(0), I32(n)])
    gpu.sync()
    acc = parts[1][0].copy()
    for q in range(1, n):
        acc = acc + parts[1][q]
    want2 = want_x.copy()
    want2[own] = (want_x + acc)[own]
    for q in range(1, n):
        rows = np.arange(T) % n == q
        want2[rows] = xs[q][rows]
    got2 = gpu.fetch(b["x"], f, (T, dim))
    m = ~np.isnan(want2)
    assert np.array_equal(np.isnan(got2), ~m) and np.array_equal(got2[m], want2[m])
    assert np.array_equal(gpu.fetch(b["h"], hf, (T, dim)).view(np.uint16), got_h.view(np.uint16)), "h untouched"
    for q in range(1, n):
        sent = gpu.fetch(b["stage"][q], np.uint32, (T, dim))
        assert not (sent[own] == EMPTY).any()
        sx = sent[own].view(f)
        mm = ~np.isnan(sx)
        assert np.array_equal(mm, m[own]) and np.array_equal(sx[mm], want2[own][mm]), "own x rows sent to every peer"
    assert (gpu.fetch(b["stage"][0], np.uint32, (T * dim,)) == EMPTY).all()
    assert (gpu.fetch(b["part"][1][0], np.uint32, ((T + n) * dim,)) == EMPTY).all()


@pytest.mark.parametrize("n,rank,M,N,K", [(2, 1, 16, 256, 512), (8, 3, 256, 4096, 512), (4, 0, 37, 1024, 264),
                                          (8, 7, 256, 4096, 1792)])
def test_linear_scatter_stores_rows_into_their_owners(gpu, n, rank, M, N, K):
    """The projection of rank ``rank``: row r of its product must land in inbox ``which`` of rank
    r % n at [rank][r // n], and nowhere else; the values are linear_f32's."""
    import oracle
    r = oracle.Rng(70 + n)
    b = group(gpu, n, M, N, rank=rank)
    x, w = r.tensor(hf, (M, K)), r.tensor(hf, (N, K), 0.1)
    bx, bw, by = gpu.tensor(x), gpu.tensor(w), gpu.alloc(M * N * 4)
    gpu.launch(gpu.kernel("linear_f32", [[M, K], [N, K], [M, N]]), [bx, bw, by])
    k = gpu.kernel("linear_scatter", [[M, K], [N, K], [b["table"].bytes]])
    gpu.launch(k, [bx, bw, b["table"], I32(1)])
    gpu.sync()
    want = gpu.fetch(by, f, (M, N))
    per = -(-M // n)
    for o in range(n):
        box = gpu.fetch(b["part"][1][o], np.uint32, ((M + n) * N,))[:n * per * N].reshape(n, per, N)
        rows = np.arange(M)[np.arange(M) % n == o]
        assert np.array_equal(box[rank, :len(rows)], want[rows].view(np.uint32)), f"rows of owner {o}"
        box[rank, :len(rows)] = EMPTY
        assert (box == EMPTY).all(), "nothing else of the inbox is touched"
        assert (gpu.fetch(b["part"][0][o], np.uint32, ((M + n) * N,)) == EMPTY).all(), "the other inbox is untouched"
