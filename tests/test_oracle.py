"""Pins the CPU oracle: f16 rounding against the reference's known answers and its own
helpers compiled from the reference tree, and every kernel restatement against the plain
f64 procedures of the reference's tests, on the same seeded generator, shapes and
tolerances (tests/interp.rs, tests/common/mod.rs, examples/metal_cases.rs:159-324)."""
import ctypes as C
import json
import os

import numpy as np
import pytest

import oracle
from refs import assert_close, attention_ref, matmul_ref, paged_case, paged_ref, rmsnorm_ref

HERE = os.path.dirname(os.path.abspath(__file__))
h, f, i32 = np.float16, np.float32, np.int32


# ---- f16 ---------------------------------------------------------------------------
def test_f16_known_answers():
    """src/half.rs:69-77."""
    L = oracle.lib()
    for x in [0.0, 1.0, -2.5, 65504.0, 6.1e-5, 1e-7, 3.140625]:
        b = L.orc_f2h(C.c_float(x))
        assert L.orc_f2h(C.c_float(L.orc_h2f(b))) == b
    r16 = lambda x: L.orc_h2f(L.orc_f2h(C.c_float(x)))
    assert r16(1.0 + 1.0 / 4096.0) == 1.0
    assert r16(70000.0) == float("inf")


def test_f16_matches_numpy_and_reference_prelude():
    """All 65536 halves widen as numpy's IEEE binary16 does; a sweep of floats (every exponent,
    ties, subnormals, overflow) rounds as numpy and as kf2h of src/prelude.cuh:104-121."""
    allh = np.arange(65536, dtype=np.uint16)
    wide = oracle.h2f_bits(allh)
    want = allh.view(np.float16).astype(np.float32)
    assert np.array_equal(wide.view(np.uint32), want.view(np.uint32))
    rng = np.random.default_rng(0)
    bits = rng.integers(0, 1 << 32, 400000, dtype=np.uint64).astype(np.uint32)
    # Exact ties and near-ties around every half value.
    mid = (allh[:-1].view(np.float16).astype(np.float64) + allh[1:].view(np.float16).astype(np.float64)) / 2
    mid = mid[np.isfinite(mid)].astype(np.float32)
    x = np.concatenate([bits.view(np.float32), mid, np.nextafter(mid, np.float32(np.inf)),
                        np.nextafter(mid, np.float32(-np.inf)), wide])
    nan = np.isnan(x)
    got = oracle.f2h_bits(x)
    with np.errstate(over="ignore"):
        ref = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(got[~nan], ref[~nan])
    assert ((got[nan] & 0x7c00) == 0x7c00).all() and ((got[nan] & 0x3ff) != 0).all()
    probe = os.path.join(os.path.dirname(HERE), "oracle", "_ref", "libprelude_probe.so")
    if not os.path.exists(probe):
        pytest.skip("oracle/_ref not built (reference tree absent)")
    P = C.CDLL(probe)
    P.probe_f2h.restype, P.probe_f2h.argtypes = C.c_uint16, [C.c_float]
    P.probe_h2f.restype, P.probe_h2f.argtypes = C.c_float, [C.c_uint16]
    sub = np.concatenate([x[~nan][::97], mid[::7]])
    for v, g in zip(sub, oracle.f2h_bits(sub)):
        assert P.probe_f2h(C.c_float(float(v))) == int(g), float(v)
    for b in range(0, 65536, 13):
        a, w = P.probe_h2f(b), float(wide[b])
        assert (a == w) or (np.isnan(a) and np.isnan(w))


def test_rng_is_the_reference_generator():
    """src/bench.rs:13-35 restated in pure Python for the first draws."""
    s = (7 * 0x9e3779b97f4a7c15) & (2 ** 64 - 1) | 1
    want = []
    for _ in range(5):
        s ^= (s << 13) & (2 ** 64 - 1)
        s ^= s >> 7
        s ^= (s << 17) & (2 ** 64 - 1)
        want.append(np.float32(np.float32(s >> 40) / np.float32(1 << 24)) * np.float32(2) - np.float32(1))
    assert np.array_equal(oracle.Rng(7).uniform(5), np.asarray(want, f))


# ---- the reference's interpreter tests ------------------------------------------------
def test_matmul_like_tests_interp_rs():
    """tests/interp.rs:63-82: seed 3, (100, 70, 90), BK 16, tolerance 2e-3."""
    r = oracle.Rng(3)
    a, b = r.tensor(h, (100, 70)), r.tensor(h, (70, 90))
    assert_close("matmul", oracle.matmul(a, b, bk=16), matmul_ref(a, b, False), 2e-3)


def test_flash_attention_like_tests_interp_rs():
    """tests/interp.rs:103-124: seed 4, (2, 150, 32), tolerance 5e-3."""
    r = oracle.Rng(4)
    q, k, v = (r.tensor(h, (2, 150, 32)) for _ in range(3))
    scale = float(np.float32(1.0) / np.sqrt(np.float32(32)))
    assert_close("flash attention", oracle.flash_attention(q, k, v, scale), attention_ref(q, k, v, scale), 5e-3)


def test_paged_attention_like_tests_interp_rs():
    """tests/interp.rs:126-136: seed 5, b 3, h 2, d 32, p 16, lens 37/1/64, tolerance 5e-3."""
    r = oracle.Rng(5)
    q, kc, vc, table, lens, scale = paged_case(r, 3, 2, 32, 16, [37, 1, 64])
    assert_close("paged attention", oracle.decode_attention(q, kc, vc, table, lens, scale),
                 paged_ref(q, kc, vc, table, lens, scale), 5e-3)


# ---- every llm.tl kernel at the small shapes of examples/metal_cases.rs:159-324 ----------
DM, NH, NG, HD, F_, V, NPOS = 128, 4, 2, 64, 256, 300, 64
T, W, NS = 16, (4 + 2 * 2) * 64, 64


@pytest.fixture()
def r():
    return oracle.Rng(11)


def test_embed(r):
    tok = np.asarray([(i * 37) % V for i in range(T)], i32)
    tok[3], tok[5] = -1, V  # outside the table: zeros
    E = r.tensor(h, (V, DM))
    x = oracle.embed(tok, E)
    want = E.astype(f)[np.clip(tok, 0, V - 1)]
    want[3] = want[5] = 0
    assert np.array_equal(x, want)


def test_rmsnorm_and_rows(r):
    x, w = r.tensor(f, (T, DM), 2.0), r.tensor(h, (DM,))
    assert_close("rmsnorm", oracle.rmsnorm(x, w, 1e-5), rmsnorm_ref(x, w, 1e-5), 2e-3)
    idx = np.asarray([15, 3, 0, 9], i32)
    assert np.array_equal(oracle.rmsnorm_rows(x, idx, w, 1e-5), oracle.rmsnorm(x, w, 1e-5)[idx])


def test_linear_family(r):
    x, w = r.tensor(h, (T, DM)), r.tensor(h, (W, DM), 0.1)
    assert_close("linear", oracle.linear(x, w), matmul_ref(x, w, True), 2e-3)
    x2, w2, res = r.tensor(h, (T, F_)), r.tensor(h, (DM, F_), 0.1), r.tensor(f, (T, DM))
    assert_close("linear_residual", oracle.linear_residual(x2, w2, res), res + matmul_ref(x2, w2, True), 1e-4)
    wv = r.tensor(h, (V, DM), 0.1)
    assert_close("logits", oracle.logits(x, wv), matmul_ref(x, wv, True), 1e-4)
    wg, wu = r.tensor(h, (F_, DM), 0.1), r.tensor(h, (F_, DM), 0.1)
    g, u = matmul_ref(x, wg, True).astype(np.float64), matmul_ref(x, wu, True).astype(np.float64)
    assert_close("gate_up", oracle.gate_up(x, wg, wu, bk=32), g / (1 + np.exp(-g)) * u, 2e-3)


def _rope_ref(x, c, s):
    d2 = x.shape[-1] // 2
    x1, x2 = x[..., :d2].astype(np.float64), x[..., d2:].astype(np.float64)
    return np.concatenate([x1 * c - x2 * s, x2 * c + x1 * s], -1).astype(f)


def test_rope_q_and_kv_write(r):
    qkv = r.tensor(h, (T, W))
    pos = np.asarray([(i * 3) % NPOS for i in range(T)], i32)
    Ct, St = r.tensor(f, (NPOS, HD // 2)), r.tensor(f, (NPOS, HD // 2))
    q = oracle.rope_q(qkv, pos, Ct, St, NH, HD)
    c, s = Ct[pos][:, None, :], St[pos][:, None, :]
    assert_close("rope_q", q, _rope_ref(qkv[:, :NH * HD].reshape(T, NH, HD), c, s), 2e-3)
    # The last two tokens are padding: slots out of range, writes dropped.
    slot = np.asarray([(i * 5) % NS if i < T - 2 else NS for i in range(T)], i32)
    kc0 = np.zeros((NS, NG, HD), h)
    kc, vc, kd, vd = oracle.kv_write(qkv, pos, slot, Ct, St, kc0, kc0, NG, HD)
    kref = _rope_ref(qkv[:, NH * HD:(NH + NG) * HD].reshape(T, NG, HD), c, s)
    vref = qkv[:, (NH + NG) * HD:].reshape(T, NG, HD)
    assert_close("kv_write K", kd, kref, 2e-3)
    assert np.array_equal(vd, vref)
    for t in range(T - 2):
        assert np.array_equal(kc[slot[t]], kd[t]) and np.array_equal(vc[slot[t]], vd[t])
    untouched = np.setdiff1d(np.arange(NS), slot[:T - 2])
    assert not kc[untouched].any() and not vc[untouched].any()


def test_prefill_attention_packed(r):
    """Two prompts of 70 and 26 tokens in one step (examples/metal_cases.rs:176-177), BM = BN = 32."""
    S = 96
    q, k, v = r.tensor(h, (S, NH, HD)), r.tensor(h, (S, NG, HD)), r.tensor(h, (S, NG, HD))
    starts = np.asarray([0 if i < 70 else 70 for i in range(S)], i32)
    got = oracle.prefill_attention(q, k, v, starts, 0.125, BM=32, BN=32)
    rep = NH // NG
    want = attention_ref(q.transpose(1, 0, 2), np.repeat(k, rep, 1).transpose(1, 0, 2),
                         np.repeat(v, rep, 1).transpose(1, 0, 2), 0.125, starts).transpose(1, 0, 2)
    assert_close("prefill_attention", got, want, 2e-3)
    # Tile shapes only move rounding.
    assert_close("tiles", oracle.prefill_attention(q, k, v, starts, 0.125, BM=64, BN=64), got, 2e-3)


def test_decode_attention_gqa(r):
    """examples/metal_cases.rs:296-309: lens 5 / 64 / 0; the empty sequence is 0/0 = NaN."""
    b, npg, p, mp = 3, 12, 16, 4
    q = r.tensor(h, (b, NH, HD))
    kc, vc = r.tensor(h, (npg, p, NG, HD)), r.tensor(h, (npg, p, NG, HD))
    table = np.asarray([7, 2, 9, 0, 4, 11, 1, 6, 3, 10, 5, 8], i32).reshape(b, mp)
    lens = np.asarray([5, 64, 0], i32)
    got = oracle.decode_attention(q, kc, vc, table, lens, 0.125).astype(f)
    want = paged_ref(q, kc, vc, table, lens, 0.125)
    assert np.isnan(got[2]).all()
    assert_close("decode_attention", got[:2], want[:2], 2e-3)


def test_config1_golden():
    """benchmark configuration 1 (ctx 37/128/300/511, 8 heads, 2 kv heads, D 64, 128-page pool): the
    committed fixture, generated by tests/golden/make_golden.py, still matches the oracle."""
    from golden.make_golden import config1_inputs
    c = config1_inputs()
    want = np.load(os.path.join(HERE, "golden", "decode_config1.npz"))["o"]
    got = oracle.decode_attention(c["q"], c["kc"], c["vc"], c["table"], c["lens"], float(c["scale"]))
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    assert_close("config 1 vs f64", got,
                 paged_ref(c["q"], c["kc"], c["vc"], c["table"], c["lens"], float(c["scale"])), 2e-3)
