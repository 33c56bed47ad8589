"""The FP8 mode (E4M3 operands, per-row scales, f32 accumulation): a separate, non-parity mode,
so it is held not against the reference's f16 arithmetic but against its own definition in numpy
(tessel_b200/fp8.py, the kernels of tests/emu.py): the quantiser byte for byte, the projections
within 2e-3 of exact products of the same bytes, and the engine within 1e-2 of the same engine
on the CPU stand-in - and, loosely, near the f16 engine."""
import numpy as np
import pytest

import oracle
from emu import EmuGpu
from refs import rel_err
from tessel_b200 import fp8
from tessel_b200.engine import Decode, Engine, Limits, Prefill
from tessel_b200.gpu import F32
from tessel_b200.model import Config, Weights, argmax

pytestmark = pytest.mark.gpu
h, f, u8 = np.float16, np.float32, np.uint8


def run(gpu, name, arrays, outs, scalars=()):
    bufs = [gpu.tensor(a) for a in arrays]
    k = gpu.kernel(name, [a.shape for a in arrays])
    gpu.launch(k, bufs + [F32(s) for s in scalars])
    gpu.sync()
    res = [gpu.fetch(bufs[i], arrays[i].dtype, arrays[i].shape) for i in outs]
    for b in bufs:
        gpu.free(b)
    return res


def test_host_encoder_round_trips_and_saturates():
    codes = np.arange(256, dtype=u8)
    vals = fp8.decode(codes)
    ok = ~np.isnan(vals)
    assert np.array_equal(fp8.encode(vals[ok]), codes[ok])
    assert fp8.encode(np.float32([1000.0, -1000.0, 448.0, 464.0]))[:].tolist() == [0x7E, 0xFE, 0x7E, 0x7E]


@pytest.mark.parametrize("M,K", [(16, 256), (256, 4096), (100, 14336), (7, 24)])
def test_quant_rows_bytes_are_the_host_quantisers(gpu, M, K):
    r = oracle.Rng(81)
    x = r.tensor(h, (M, K))
    x[0] = 0  # a zero row: scale 1, bytes 0
    x[1, 3] = 300.0
    q, s = run(gpu, "quant_rows", [x, np.zeros((M, K), u8), np.zeros(M, f)], [1, 2])
    wq, ws = fp8.quantize_rows(x.astype(f))
    assert np.array_equal(s, ws)
    assert np.array_equal(q, wq)


def test_rmsnorm_q8_is_rmsnorm_then_quant_rows(gpu):
    r = oracle.Rng(82)
    T, Dm = 64, 4096
    x, w = r.tensor(f, (T, Dm)), r.tensor(h, (Dm,))
    q, s = run(gpu, "rmsnorm_q8", [x, w, np.zeros((T, Dm), u8), np.zeros(T, f)], [2, 3], [1e-5])
    want = oracle.rmsnorm(x, w, 1e-5).astype(f)
    # The norm's sum order may move an f16 value by one step, and with it a byte: compare values.
    assert rel_err(fp8.decode(q) * s[:, None], want) <= 0.07          # E4M3 has 3 mantissa bits
    wq, ws = fp8.quantize_rows(want)
    assert np.abs(s - ws).max() <= 2e-3 * ws.max()
    assert (q != wq).mean() < 0.01


@pytest.mark.parametrize("M,N,K", [(256, 6144, 4096), (16, 256, 512), (100, 200, 272), (256, 4096, 14336),
                                   (600, 512, 1040)])
def test_projections_on_quantised_operands(gpu, M, N, K):
    r = oracle.Rng(83)
    xq, sx = fp8.quantize_rows(r.tensor(f, (M, K)))
    wq, sw = fp8.quantize_rows(r.tensor(f, (N, K), 0.1))
    uq, su = fp8.quantize_rows(r.tensor(f, (N, K), 0.1))
    res = r.tensor(f, (M, N))
    rows = np.unique(np.linspace(0, M - 1, 16).astype(int))

    def product(a, sa, b, sb):
        return (fp8.decode(a[rows]).astype(np.float64) @ fp8.decode(b).astype(np.float64).T) * (sa[rows, None] * sb[None, :])

    (y,) = run(gpu, "linear_q8", [xq, sx, wq, sw, np.zeros((M, N), h)], [4])
    assert rel_err(y[rows], product(xq, sx, wq, sw)) <= 2e-3
    (y,) = run(gpu, "linear_residual_q8", [xq, sx, wq, sw, res.copy()], [4])
    assert rel_err(y[rows], res[rows] + product(xq, sx, wq, sw)) <= 2e-3
    (y,) = run(gpu, "gate_up_q8", [xq, sx, wq, sw, uq, su, np.zeros((M, N), h)], [6])
    g, u = product(xq, sx, wq, sw), product(xq, sx, uq, su)
    assert rel_err(y[rows], g / (1 + np.exp(-g)) * u) <= 2e-3


def test_engine_in_fp8_mode(gpu):
    cfg = Config(dim=256, layers=2, heads=8, kv_heads=2, head_dim=64, ffn=512, vocab=1000, eps=1e-5,
                 rope_theta=10000.0, max_pos=512, bos=1, eos=-1)
    w = Weights.random(cfg, 13)
    lim = Limits(page=16, pages=40, max_tokens=64, max_seq_pages=8)
    prompt = np.random.default_rng(0).integers(0, cfg.vocab, 30).tolist()
    n = len(prompt)
    out = {}
    for name, dev, q8 in (("gpu8", gpu, True), ("cpu8", EmuGpu(), True), ("gpu16", gpu, False)):
        e = Engine(dev, w, lim, fp8=q8)
        pre = e.step(prompt, list(range(n)), list(range(n)), Prefill(), [n - 1]).copy()
        tok = argmax(pre[0])
        dec = e.step([tok], [n], [n], Decode([[0, 1]], [n + 1]), [0]).copy()
        out[name] = (pre, dec, tok)
    for i in (0, 1):
        assert rel_err(out["gpu8"][i], out["cpu8"][i]) <= 1e-2, "FP8 engine differs from its numpy definition"
        assert rel_err(out["gpu8"][i], out["gpu16"][i]) <= 0.15, "FP8 engine is far from the f16 engine"
    assert out["gpu8"][2] == out["cpu8"][2]
