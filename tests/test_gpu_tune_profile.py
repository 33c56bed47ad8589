"""Two services of the boundary that the reference keeps on its host side: choosing a
projection's tile by timing the candidates on the device (Engine::mm, src/llm/engine.rs:233-270)
and the per-kernel profile (Gpu::profile, src/gpu.rs:38-42, :198-222), both through the C ABI."""
import numpy as np
import pytest

import oracle
from refs import rel_err
from tessel_b200.gpu import F32

pytestmark = pytest.mark.gpu
h, f = np.float16, np.float32


def test_tuning_picks_a_tile_and_keeps_the_result(gpu):
    M, N, K = 256, 1544, 2056
    r = oracle.Rng(51)
    x, w = r.tensor(h, (M, K)), r.tensor(h, (N, K), 0.1)
    res = r.tensor(f, (M, N))
    bx, bw = gpu.tensor(x), gpu.tensor(w)
    for name, out0, want in (("linear", np.zeros((M, N), h), oracle.linear(x, w)),
                             ("linear_residual", res, oracle.linear_residual(x, w, res))):
        by = gpu.tensor(out0)
        k = gpu.kernel(name, [[M, K], [N, K], [M, N]])
        plan, us = gpu.tune(k, [bx, bw, by])
        assert plan[0] in (1, 2, 3) and plan[1] in (32, 64, 96, 128, 192, 224, 256) and 1 <= plan[2] <= 4, plan
        assert 1.0 < us < 1000.0, us
        gpu.write(by, 0, out0)  # tuning clobbered (or accumulated into) the output
        gpu.launch(k, [bx, bw, by])
        gpu.sync()
        assert rel_err(gpu.fetch(by, out0.dtype, (M, N)), want) <= 2e-3
        assert gpu.tune(k, [bx, bw, by])[0] in [(1, b, s) for b in (32, 64, 128, 256) for s in (1, 2, 4)] + \
            [(2, b, s) for b in (32, 64, 128, 192, 256) for s in (1, 2, 4)] + [(3, b, s) for b in (64, 96, 128, 192, 224, 256) for s in (1, 2)]
    # A kernel without tile candidates: nothing to tune, no error.
    a = gpu.tensor(np.ones((4, 8), f))
    k = gpu.kernel("residual_add", [[4, 8], [4, 8]])
    assert gpu.tune(k, [a, a]) == ((0, 0, 0), 0.0)


def test_forced_plan_is_not_overridden_by_tuning(gpu, monkeypatch):
    monkeypatch.setenv("TB200_GEMM_PLAN", "2,64,1")
    M, N, K = 256, 328, 520
    r = oracle.Rng(52)
    x, w = r.tensor(h, (M, K)), r.tensor(h, (N, K), 0.1)
    bufs = [gpu.tensor(x), gpu.tensor(w), gpu.alloc(M * N * 2)]
    k = gpu.kernel("linear", [[M, K], [N, K], [M, N]])
    assert gpu.tune(k, bufs)[0] == (2, 64, 1)


def test_profile_counts_launches_by_phase_and_kernel(gpu):
    a, b = gpu.tensor(np.ones((4, 8), f)), gpu.tensor(np.ones((4, 8), f))
    k = gpu.kernel("residual_add", [[4, 8], [4, 8]])
    x = gpu.tensor(np.ones((16, 64), f))
    y = gpu.alloc(16 * 64 * 2)
    wn = gpu.tensor(np.ones(64, h))
    kn = gpu.kernel("rmsnorm", [[16, 64], [64], [16, 64]])
    assert gpu.profile is None
    gpu.profile = {}
    gpu.phase = "decode"
    for _ in range(3):
        gpu.launch(k, [a, b])
    gpu.phase = "prefill"
    gpu.launch(kn, [x, wn, y, F32(1e-5)])
    rows = gpu.profile_rows()
    gpu.profile = None
    got = {(p, name): n for p, name, n, ms in rows}
    assert got == {("decode", "residual_add -> [4, 8]"): 3, ("prefill", "rmsnorm -> [16, 64]"): 1}
    assert all(ms > 0 for _, _, _, ms in rows) and rows == sorted(rows, key=lambda r: -r[3])
    gpu.launch(k, [a, b])  # not profiled any more
    gpu.sync()
    assert len(gpu.profile_rows()) == 2
    assert np.array_equal(gpu.fetch(a, f, (4, 8)), np.full((4, 8), 5.0, f))
