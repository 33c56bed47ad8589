"""The tcgen05 projections against the CPU oracle, through the C ABI: every epilogue, the
decode and prompt row counts the engine uses, ragged sizes (rows and columns that are not
tile multiples, K that is not a multiple of 64), the reference's tuning-test shapes
(tests/llm.rs:107-187) and its (100, 70, 90) matmul whose pitch TMA cannot address; and at
4096^3 sampled entries in f64 (src/bench.rs:86-98) plus linearity."""
import numpy as np
import pytest

import oracle
from refs import matmul_ref, rel_err
from tessel_b200.gpu import F32

pytestmark = pytest.mark.gpu
h, f, i32 = np.float16, np.float32, np.int32
TOL = 2e-3


def launch(gpu, name, arrays, out):
    bufs = [gpu.tensor(a) for a in arrays]
    k = gpu.kernel(name, [a.shape for a in arrays])
    gpu.launch(k, bufs)
    gpu.sync()
    y = gpu.fetch(bufs[out], arrays[out].dtype, arrays[out].shape)
    for b in bufs:
        gpu.free(b)
    return y


SHAPES = [(16, 96, 256), (32, 96, 256), (64, 96, 256),       # tests/llm.rs:118-119
          (16, 512, 128), (256, 6144, 4096), (256, 4096, 512), (100, 200, 72),
          (256, 768, 4096), (256, 4096, 1792),                # an 8-way tensor-parallel rank's QKV and down_proj
          (128, 256, 64), (129, 264, 200), (300, 40, 1032), (2048, 512, 256), (1, 8, 8)]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_linear_family(gpu, M, N, K):
    r = oracle.Rng(31)
    x, w = r.tensor(h, (M, K)), r.tensor(h, (N, K), 0.1)
    res = r.tensor(f, (M, N))
    big = M * N * K > 1 << 28
    rows = np.unique(np.linspace(0, M - 1, 16).astype(int)) if big else np.arange(M)
    y = launch(gpu, "linear", [x, w, np.zeros((M, N), h)], 2)
    assert rel_err(y[rows], oracle.linear(x[rows], w)) <= TOL
    y = launch(gpu, "logits", [x, w, np.full((M, N), 3, f)], 2)
    assert rel_err(y[rows], oracle.logits(x[rows], w)) <= TOL
    y = launch(gpu, "linear_f32", [x, w, np.full((M, N), 3, f)], 2)
    assert rel_err(y[rows], oracle.logits(x[rows], w)) <= TOL
    y = launch(gpu, "linear_residual", [x, w, res.copy()], 2)
    assert rel_err(y[rows], oracle.linear_residual(x[rows], w, res[rows])) <= TOL


@pytest.mark.parametrize("M,F,K", [(16, 96, 256), (64, 96, 256), (16, 256, 128), (256, 14336 // 8, 4096),
                                   (130, 200, 136), (2048, 256, 128)])
def test_gate_up(gpu, M, F, K):
    r = oracle.Rng(32)
    x, wg, wu = r.tensor(h, (M, K)), r.tensor(h, (F, K), 0.1), r.tensor(h, (F, K), 0.1)
    y = launch(gpu, "gate_up", [x, wg, wu, np.zeros((M, F), h)], 3)
    rows = np.unique(np.linspace(0, M - 1, 24).astype(int))
    assert rel_err(y[rows], oracle.gate_up(x[rows], wg, wu)) <= TOL


@pytest.mark.parametrize("M,K,N", [(100, 70, 90), (128, 64, 64), (256, 128, 256), (200, 136, 328), (512, 1024, 2048)])
def test_matmul_row_major_b(gpu, M, K, N):
    """kernels/matmul.tl:3-17: B is [K, N] row-major (an N-major operand for the tensor core)."""
    r = oracle.Rng(3)
    a, b = r.tensor(h, (M, K)), r.tensor(h, (K, N))
    c = launch(gpu, "matmul", [a, b, np.zeros((M, N), h)], 2)
    assert rel_err(c, matmul_ref(a, b, False)) <= TOL
    if M * N * K <= 1 << 24:
        assert rel_err(c, oracle.matmul(a, b)) <= TOL


def test_matmul_4096_cubed(gpu):
    """benchmark configuration 2: A, B ~U[-1,1] seeded, f16, f32 accumulation, f16 out; 256 sampled
    entries in f64, whole rows against the oracle, and C(A, B1 + B2) = C(A, B1) + C(A, B2)
    for operands chosen so that the sums are exact."""
    n = 4096
    r = oracle.Rng(1)
    a, b = r.tensor(h, (n, n)), r.tensor(h, (n, n))
    c = launch(gpu, "matmul", [a, b, np.zeros((n, n), h)], 2)
    g = np.random.default_rng(0)
    ii, jj = g.integers(0, n, 256), g.integers(0, n, 256)
    want = np.einsum("sk,ks->s", a[ii].astype(np.float64), b[:, jj].astype(np.float64))
    assert np.abs(c[ii, jj].astype(np.float64) - want).max() / np.abs(want).max() <= TOL
    rows = [0, 1, 2047, 4095]
    want_rows = np.concatenate([oracle.matmul_block(a, b, i, i + 1, 0, n) for i in rows])
    assert rel_err(c[rows], want_rows) <= TOL
    # Linearity with small-integer operands: every product and sum is exact in f32 and f16.
    ai = g.integers(-2, 3, (256, 256)).astype(h)
    b1, b2 = g.integers(-2, 3, (256, 256)).astype(h), g.integers(-2, 3, (256, 256)).astype(h)
    c1 = launch(gpu, "matmul", [ai, b1, np.zeros((256, 256), h)], 2).astype(f)
    c2 = launch(gpu, "matmul", [ai, b2, np.zeros((256, 256), h)], 2).astype(f)
    c12 = launch(gpu, "matmul", [ai, (b1 + b2).astype(h), np.zeros((256, 256), h)], 2).astype(f)
    assert np.array_equal(c12, c1 + c2)
    assert np.array_equal(c1, (ai.astype(f) @ b1.astype(f)))


@pytest.mark.parametrize("plan,M,N,K", [
    ("1,128,1", 200, 392, 1024), ("2,128,1", 256, 520, 1032), ("2,256,1", 256, 776, 1040),
    ("2,128,2", 256, 264, 2048), ("2,128,4", 256, 4096, 4096), ("2,192,4", 256, 6144, 4096),
    ("2,256,4", 250, 1288, 4104), ("2,256,2", 256, 1296, 1096), ("1,128,4", 100, 136, 2056),
    ("2,64,4", 256, 200, 3080), ("2,128,4", 256, 4104, 14336),
    # MT = 3: a CTA pair (tcgen05 cta_group::2) on a 256-row tile, each CTA holding 128 rows of X
    # and half of the weight slice; alone, with cluster split-K, and over several row pairs.
    ("3,256,1", 256, 784, 1048), ("3,128,1", 200, 400, 1032), ("3,192,1", 129, 584, 520),
    ("3,256,2", 256, 1304, 2056), ("3,192,2", 256, 6152, 4096), ("3,256,4", 250, 4112, 4104),
    ("3,128,4", 256, 272, 2048), ("3,256,1", 600, 528, 512), ("3,128,2", 1000, 136, 1096),
    # the pair tiles between the powers of two (they put a projection on more SMs in one wave)
    ("3,224,1", 256, 1000, 1056), ("3,96,1", 256, 6144, 1064), ("3,64,1", 200, 328, 1072), ("3,64,2", 256, 392, 2064),
])
def test_forced_tiles_and_cluster_split_k(gpu, plan, M, N, K, monkeypatch):
    """Every tile shape, the CTA-pair kernel and the cluster split-K exchange (TB200_GEMM_PLAN = MT,BN,splits), on shapes
    no other test uses (a kernel is made once per shape), for all four epilogues; and the split
    sum is the same bits on every run (partials are added in rank order)."""
    monkeypatch.setenv("TB200_GEMM_PLAN", plan)
    r = oracle.Rng(33)
    x, w = r.tensor(h, (M, K)), r.tensor(h, (N, K), 0.1)
    res = r.tensor(f, (M, N))
    rows = np.unique(np.linspace(0, M - 1, 12).astype(int))
    y = launch(gpu, "linear", [x, w, np.zeros((M, N), h)], 2)
    assert rel_err(y[rows], oracle.linear(x[rows], w)) <= TOL
    y2 = launch(gpu, "linear", [x, w, np.zeros((M, N), h)], 2)
    assert np.array_equal(y.view(np.uint16), y2.view(np.uint16))
    y = launch(gpu, "logits", [x, w, np.full((M, N), 3, f)], 2)
    assert rel_err(y[rows], oracle.logits(x[rows], w)) <= TOL
    y = launch(gpu, "linear_residual", [x, w, res.copy()], 2)
    assert rel_err(y[rows], oracle.linear_residual(x[rows], w, res[rows])) <= TOL
    if plan.endswith(",1") and not plan.startswith("2,256"):
        wu = r.tensor(h, (N, K), 0.1)
        y = launch(gpu, "gate_up", [x, w, wu, np.zeros((M, N), h)], 3)
        assert rel_err(y[rows], oracle.gate_up(x[rows], w, wu)) <= TOL


def test_gate_up_ragged_tile(gpu, monkeypatch):
    """The 112-column gate_up tile (224-wide MMA, last epilogue chunk 16 columns wide), which lets
    14336 MLP columns fill 128 SMs in one wave; columns beyond a tile must not be written."""
    monkeypatch.setenv("TB200_GEMM_PLAN", "2,112,1")
    r = oracle.Rng(34)
    M, F, K = 256, 1000, 512  # 9 tiles of 112, the last one partial
    x, wg, wu = r.tensor(h, (M, K)), r.tensor(h, (F, K), 0.1), r.tensor(h, (F, K), 0.1)
    y = launch(gpu, "gate_up", [x, wg, wu, np.zeros((M, F), h)], 3)
    assert rel_err(y, oracle.gate_up(x, wg, wu)) <= TOL


def test_empty_shapes(gpu):
    x = np.zeros((0, 64), h)
    w = np.ones((32, 64), h)
    assert launch(gpu, "linear", [x, w, np.zeros((0, 32), h)], 2).shape == (0, 32)
    y = launch(gpu, "linear", [np.zeros((4, 0), h), np.zeros((8, 0), h), np.ones((4, 8), h)], 2)
    assert not y.any()
