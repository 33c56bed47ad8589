"""The fused tensor-parallel exchange kernel on one GPU.

Its arithmetic and data movement, with the peers played by buffers (second test), and its failure
detection without a second GPU: a rank whose peer never arrives. The table names this GPU's own buffers as "rank 1" as well, so every pointer
is valid, but nothing ever writes the flags rank 0 waits for. The wait gives up after its limit
(one second), the kernel raises the context's status word and returns, `sync` reports it, and
the context keeps working."""
import time

import numpy as np
import pytest

from tessel_b200.gpu import F32, GpuError, I32

pytestmark = pytest.mark.gpu


def test_a_peer_that_never_arrives_is_reported_and_the_context_survives(gpu):
    T, dim = 16, 256
    _, fb, eb = gpu.tp_sizes()
    part = [gpu.alloc(T * dim * 4) for _ in range(2)]
    x, h = gpu.alloc(T * dim * 4), gpu.alloc(T * dim * 2)
    stage = gpu.alloc(T * dim * 4)
    flags = [gpu.alloc(fb), gpu.alloc(fb)]  # [0]: what rank 0 polls (never written); [1]: the absent peer's
    epoch = gpu.alloc(eb)
    raw = gpu.tp_table(0, 2, [part[0]] * 2, [part[1]] * 2, [x] * 2, [h] * 2, [stage] * 2, flags, epoch)
    table = gpu.tensor(np.frombuffer(raw, np.uint8).copy())
    w = gpu.tensor(np.ones(dim, np.float16))
    k = gpu.kernel("tp_reduce_norm", [[table.bytes], [dim], [T, dim]])
    t0 = time.perf_counter()
    gpu.launch(k, [table, w, x, F32(1e-5), I32(0), I32(1), I32(2)])
    with pytest.raises(GpuError, match="gave up a bounded wait"):
        gpu.sync()
    waited = time.perf_counter() - t0
    assert 0.5 < waited < 10.0, f"the wait limit is one second, the call took {waited:.2f} s"
    # The context is intact: the status was cleared by the report, and kernels run as before.
    gpu.sync()
    a, b = gpu.tensor(np.full((4, 8), 1.5, np.float32)), gpu.tensor(np.full((4, 8), 2.0, np.float32))
    gpu.launch(gpu.kernel("residual_add", [[4, 8], [4, 8]]), [a, b])
    gpu.sync()
    assert np.array_equal(gpu.fetch(a, np.float32, (4, 8)), np.full((4, 8), 3.5, np.float32))
    with pytest.raises(GpuError, match="nranks"):
        gpu.launch(k, [table, w, x, F32(1e-5), I32(0), I32(1), I32(1)])


def test_the_x_gather_stays_until_the_peers_have_finished_reading(gpu):
    """The last call of a step (do_norm = 0) lets the peers copy rows straight out of this rank's
    x, and the next step's first kernel overwrites x: the call must not return before every peer
    has said it is done. Here the peer's "partial ready" and "rows ready" flags are preset and
    its "finished reading" flag never comes: the kernel must give up in exactly that wait
    (status 404), which shows the wait is there; the context stays usable."""
    n, T, dim = 2, 16, 256
    _, fb, eb = gpu.tp_sizes()
    z = lambda nbytes: gpu.alloc(nbytes)
    parts = [[z(T * dim * 4) for _ in range(n)] for _ in range(2)]
    xs, hs, stages = [z(T * dim * 4) for _ in range(n)], [z(T * dim * 2) for _ in range(n)], [z(T * dim * 4) for _ in range(n)]
    fl = np.full(fb // 4, 1000, np.uint32).reshape(-1, 4, 8)   # [slot][phase][sender]
    fl[:, 2, :] = 0                                             # nobody ever finishes reading
    flags = [gpu.tensor(fl), z(fb)]
    raw = gpu.tp_table(0, n, parts[0], parts[1], xs, hs, stages, flags, z(eb))
    table = gpu.tensor(np.frombuffer(raw, np.uint8).copy())
    w = gpu.tensor(np.ones(dim, np.float16))
    k = gpu.kernel("tp_reduce_norm", [[table.bytes], [dim], [T, dim]])
    gpu.launch(k, [table, w, xs[0], F32(1e-5), I32(1), I32(0), I32(n)])
    with pytest.raises(GpuError, match="status 404"):
        gpu.sync()
    gpu.sync()


@pytest.mark.parametrize("n,T,dim", [(2, 16, 256), (3, 20, 8192), (8, 256, 4096), (4, 37, 1024)])
def test_one_rank_of_a_group_whose_peers_are_buffers(gpu, n, T, dim):
    """The arithmetic and the data movement of ``tp_reduce_norm`` for rank 0 of ``n``, on one GPU
    and with no second kernel: the peers are local buffers the host fills with what they would
    hold (partials, staged h rows tagged with the first call's epoch, x rows), and the flags rank
    0 polls are preset to a later epoch, so it never waits."""
    import oracle
    from refs import rel_err
    f, hf = np.float32, np.float16
    r = oracle.Rng(41 + n)
    _, fb, eb = gpu.tp_sizes()
    parts = [[r.tensor(f, (T, dim)) for _ in range(n)] for _ in range(2)]
    x0 = r.tensor(f, (T, dim))
    w = r.tensor(hf, (dim,))
    xs = [x0] + [r.tensor(f, (T, dim)) for _ in range(n - 1)]          # the peers' residual rows
    hs = [r.tensor(hf, (T, dim)) for _ in range(n)]                    # what the peers would have normalised
    stages = []
    for q in range(n):
        st = np.zeros((T, dim // 2, 2), np.uint32)
        if q:
            st[:, :, 0] = hs[q].view(np.uint32).reshape(T, dim // 2)
            st[:, :, 1] = 1                                            # the first call's epoch
        stages.append(st)
    up = gpu.tensor
    d_parts = [[up(a) for a in row] for row in parts]
    d_x, d_stage = [up(a) for a in xs], [up(a) for a in stages]
    d_h = [gpu.alloc(T * dim * 2) for _ in range(n)]
    d_flags = [up(np.full(fb // 4, 1000, np.uint32))] + [gpu.alloc(fb) for _ in range(n - 1)]
    epoch = gpu.alloc(eb)
    raw = gpu.tp_table(0, n, d_parts[0], d_parts[1], d_x, d_h, d_stage, d_flags, epoch)
    table = up(np.frombuffer(raw, np.uint8).copy())
    k = gpu.kernel("tp_reduce_norm", [[table.bytes], [dim], [T, dim]])
    eps = 1e-5
    own = np.arange(T) % n == 0

    # Call 1: partial buffer 0, normalise, gather h.
    gpu.launch(k, [table, up(w), d_x[0], F32(eps), I32(0), I32(1), I32(n)])
    gpu.sync()
    want_x = x0.copy()
    acc = parts[0][0].copy()
    for q in range(1, n):
        acc = acc + parts[0][q]                                        # rank order, one rounded add each
    want_x[own] = (x0 + acc)[own]
    got_x = gpu.fetch(d_x[0], f, (T, dim))
    assert np.array_equal(got_x, want_x), "own rows take the sum in rank order, the others stay"
    got_h = gpu.fetch(d_h[0], hf, (T, dim))
    want_h = oracle.rmsnorm(want_x, w, eps)
    assert rel_err(got_h[own], want_h[own]) < 2e-3
    for q in range(1, n):
        rows = np.arange(T) % n == q
        assert np.array_equal(got_h[rows].view(np.uint16), hs[q][rows].view(np.uint16)), "h rows copied from their owners"
    staged = gpu.fetch(d_stage[0], np.uint32, (T, dim // 2, 2))
    assert np.array_equal(staged[own][:, :, 0], got_h[own].view(np.uint32).reshape(-1, dim // 2))
    assert (staged[own][:, :, 1] == 1).all() and not staged[~own].any()

    # Call 2 (epoch 2): partial buffer 1, no norm, gather x.
    gpu.launch(k, [table, up(w), d_x[0], F32(eps), I32(1), I32(0), I32(n)])
    gpu.sync()
    acc = parts[1][0].copy()
    for q in range(1, n):
        acc = acc + parts[1][q]
    want2 = want_x.copy()
    want2[own] = (want_x + acc)[own]
    for q in range(1, n):
        rows = np.arange(T) % n == q
        want2[rows] = xs[q][rows]
    assert np.array_equal(gpu.fetch(d_x[0], f, (T, dim)), want2)
    assert np.array_equal(gpu.fetch(d_h[0], hf, (T, dim)).view(np.uint16), got_h.view(np.uint16)), "h untouched"
