"""Failure detection of the fused tensor-parallel exchange without a second GPU: a rank whose
peer never arrives. The table names this GPU's own buffers as "rank 1" as well, so every pointer
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
