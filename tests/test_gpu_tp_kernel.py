"""The tensor-parallel exchange kernels on one GPU.

The arithmetic and the data movement of ``linear_scatter`` and ``tp_reduce_norm`` with the peers
played by buffers of this GPU, and their failure detection without a second GPU: a rank whose
peer never arrives, and rows that never land. In both, every pointer of the table is valid, but
nothing ever writes what the kernel waits for. The wait gives up after its limit (one second),
the kernel raises the context's status word and returns, `sync` reports it, and the context keeps
working."""
import time

import numpy as np
import pytest

from tessel_b200.gpu import F32, GpuError, I32

pytestmark = pytest.mark.gpu
f, hf = np.float32, np.float16


def group(gpu, n, T, dim, rank=0, flags_value=0):
    """Buffers of an n-rank group, all on this GPU: inboxes, x, h, landing areas, flags."""
    _, fb, eb = gpu.tp_sizes()
    z = gpu.alloc
    b = dict(part=[[z((T + n) * dim * 4) for _ in range(n)] for _ in range(2)],
             x=[z(T * dim * 4) for _ in range(n)], h=[z(T * dim * 2) for _ in range(n)],
             stage=[z(T * dim * 8) for _ in range(n)],
             flags=[gpu.tensor(np.full(fb // 4, flags_value, np.uint32)) if q == rank else z(fb) for q in range(n)],
             epoch=z(eb))
    raw = gpu.tp_table(rank, n, b["part"][0], b["part"][1], b["x"], b["h"], b["stage"], b["flags"], b["epoch"])
    b["table"] = gpu.tensor(np.frombuffer(raw, np.uint8).copy())
    return b


def test_a_peer_that_never_arrives_is_reported_and_the_context_survives(gpu):
    T, dim = 16, 256
    b = group(gpu, 2, T, dim)  # the flags rank 0 polls are never written
    w = gpu.tensor(np.ones(dim, hf))
    k = gpu.kernel("tp_reduce_norm", [[b["table"].bytes], [dim], [T, dim]])
    t0 = time.perf_counter()
    gpu.launch(k, [b["table"], w, b["x"][0], F32(1e-5), I32(0), I32(1), I32(2)])
    with pytest.raises(GpuError, match="gave up a bounded wait"):
        gpu.sync()
    waited = time.perf_counter() - t0
    assert 0.5 < waited < 10.0, f"the wait limit is one second, the call took {waited:.2f} s"
    # The context is intact: the status was cleared by the report, and kernels run as before.
    gpu.sync()
    a, c = gpu.tensor(np.full((4, 8), 1.5, f)), gpu.tensor(np.full((4, 8), 2.0, f))
    gpu.launch(gpu.kernel("residual_add", [[4, 8], [4, 8]]), [a, c])
    gpu.sync()
    assert np.array_equal(gpu.fetch(a, f, (4, 8)), np.full((4, 8), 3.5, f))
    with pytest.raises(GpuError, match="nranks"):
        gpu.launch(k, [b["table"], w, b["x"][0], F32(1e-5), I32(0), I32(1), I32(1)])


def test_rows_that_never_land_are_reported(gpu):
    """The peers' projections are announced (flags preset) but their finished rows never arrive
    in this rank's landing area: the gather gives up in exactly that wait (status 402)."""
    T, dim = 16, 256
    b = group(gpu, 2, T, dim, flags_value=1000)
    w = gpu.tensor(np.ones(dim, hf))
    k = gpu.kernel("tp_reduce_norm", [[b["table"].bytes], [dim], [T, dim]])
    gpu.launch(k, [b["table"], w, b["x"][0], F32(1e-5), I32(0), I32(1), I32(2)])
    with pytest.raises(GpuError, match="status 402"):
        gpu.sync()
    gpu.sync()


def tagged(payload_u32, epoch):
    """8-byte units {payload | epoch << 32} as the kernels store them."""
    return payload_u32.astype(np.uint64) | (np.uint64(epoch) << np.uint64(32))


@pytest.mark.parametrize("n,T,dim", [(2, 16, 256), (3, 20, 8192), (8, 256, 4096), (4, 37, 1024)])
def test_one_rank_of_a_group_whose_peers_are_buffers(gpu, n, T, dim):
    """``tp_reduce_norm`` for rank 0 of ``n``, on one GPU and with no second kernel: the host puts
    into rank 0's inbox what the peers' projections would have stored, and into its landing area
    the rows the other owners would have sent (tagged with the call's counter); the flags rank 0
    polls are preset to a later epoch, so it never waits. What rank 0 sends must appear, tagged,
    in every peer's landing area."""
    import oracle
    from refs import rel_err
    r = oracle.Rng(41 + n)
    b = group(gpu, n, T, dim, flags_value=1000)
    per = -(-T // n)
    own = np.arange(T) % n == 0
    nown = int(own.sum())
    parts = [[r.tensor(f, (T, dim)) for _ in range(n)] for _ in range(2)]   # every source's whole partial product
    x0 = r.tensor(f, (T, dim))
    w = r.tensor(hf, (dim,))
    hs = [r.tensor(hf, (T, dim)) for _ in range(n)]     # what the other owners would have normalised
    xs = [r.tensor(f, (T, dim)) for _ in range(n)]      # ... and their final residual rows
    for wh in range(2):
        inbox = np.zeros((T + n, dim), f).reshape(-1)
        box = np.zeros((n, per, dim), f)
        for s in range(n):
            box[s, :nown] = parts[wh][s][own]
        inbox[:box.size] = box.reshape(-1)
        gpu.write(b["part"][wh][0], 0, inbox)
    gpu.write(b["x"][0], 0, x0)
    land = np.zeros((T, dim), np.uint64)
    for q in range(1, n):
        rows = np.arange(T) % n == q
        land[rows, :dim // 2] = tagged(hs[q][rows].view(np.uint32), 1)
    gpu.write(b["stage"][0], 0, land)
    k = gpu.kernel("tp_reduce_norm", [[b["table"].bytes], [dim], [T, dim]])
    eps = 1e-5

    # Call 1: inbox 0, normalise, gather h.
    gpu.launch(k, [b["table"], gpu.tensor(w), b["x"][0], F32(eps), I32(0), I32(1), I32(n)])
    gpu.sync()
    want_x = x0.copy()
    acc = parts[0][0].copy()
    for q in range(1, n):
        acc = acc + parts[0][q]                                        # rank order, one rounded add each
    want_x[own] = (x0 + acc)[own]
    got_x = gpu.fetch(b["x"][0], f, (T, dim))
    assert np.array_equal(got_x, want_x), "own rows take the sum in rank order, the others stay"
    got_h = gpu.fetch(b["h"][0], hf, (T, dim))
    want_h = oracle.rmsnorm(want_x, w, eps)
    assert rel_err(got_h[own], want_h[own]) < 2e-3
    for q in range(1, n):
        rows = np.arange(T) % n == q
        assert np.array_equal(got_h[rows].view(np.uint16), hs[q][rows].view(np.uint16)), "h rows taken from the landing area"
        sent = gpu.fetch(b["stage"][q], np.uint64, (T, dim))
        assert np.array_equal(sent[own, :dim // 2], tagged(got_h[own].view(np.uint32), 1)), "own h rows sent to every peer"
        assert not sent[~own].any()

    # Call 2 (epoch 2): inbox 1, no norm, gather x.
    land = np.zeros((T, dim), np.uint64)
    for q in range(1, n):
        rows = np.arange(T) % n == q
        land[rows] = tagged(xs[q][rows].view(np.uint32), 2)
    gpu.write(b["stage"][0], 0, land)
    gpu.launch(k, [b["table"], gpu.tensor(w), b["x"][0], F32(eps), I32(1), I32(0), I32(n)])
    gpu.sync()
    acc = parts[1][0].copy()
    for q in range(1, n):
        acc = acc + parts[1][q]
    want2 = want_x.copy()
    want2[own] = (want_x + acc)[own]
    for q in range(1, n):
        rows = np.arange(T) % n == q
        want2[rows] = xs[q][rows]
    assert np.array_equal(gpu.fetch(b["x"][0], f, (T, dim)), want2)
    assert np.array_equal(gpu.fetch(b["h"][0], hf, (T, dim)).view(np.uint16), got_h.view(np.uint16)), "h untouched"
    for q in range(1, n):
        sent = gpu.fetch(b["stage"][q], np.uint64, (T, dim))
        assert np.array_equal(sent[own], tagged(want2[own].view(np.uint32), 2)), "own x rows sent to every peer"


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
        box = gpu.fetch(b["part"][1][o], f, ((M + n) * N,))[:n * per * N].reshape(n, per, N)
        rows = np.arange(M)[np.arange(M) % n == o]
        assert np.array_equal(box[rank, :len(rows)], want[rows]), f"rows of owner {o}"
        box[rank, :len(rows)] = 0
        assert not box.any(), "nothing else of the inbox is touched"
        assert not gpu.fetch(b["part"][0][o], f, ((M + n) * N,)).any(), "the other inbox is untouched"
