"""numpy front end of the CPU oracle (``oracle/tessel_oracle.cpp``).

Test infrastructure only: the test-suite, the smoke check and the CPU-baseline
leg of the benchmark import this; nothing in ``tessel_b200`` does. Every
function takes and returns numpy arrays; f16 tensors are ``np.float16`` (whose
bits are IEEE binary16, the same bits tessel's ``src/half.rs`` produces).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libtessel_oracle.so")


def reference_tree() -> str:
    """A checkout of the reference to build the f16 probe from: ``$TESSEL_REFERENCE``, else a
    directory ``reference`` beside this repository; "" when neither holds ``src/prelude.cuh``."""
    for cand in (os.environ.get("TESSEL_REFERENCE", ""), os.path.join(_HERE, "..", "..", "reference")):
        if cand and os.path.isfile(os.path.join(cand, "src", "prelude.cuh")):
            return os.path.abspath(cand)
    return ""


def build(force: bool = False) -> str:
    """Compiles the oracle (and the reference f16 probe when a reference tree is found)."""
    src = os.path.join(_HERE, "tessel_oracle.cpp")
    ref = reference_tree()
    probe = os.path.join(_HERE, "_ref", "libprelude_probe.so")
    stale = not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src)
    if force or stale or (ref and not os.path.exists(probe)):
        env = dict(os.environ)
        env.pop("CXX", None)
        subprocess.check_call(["make", "-C", _HERE, "CXX=g++", "REF=" + ref], env=env, stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.orc_h2f.restype = C.c_float
        _lib.orc_f2h.restype = C.c_uint16
        _lib.orc_f2h.argtypes = [C.c_float]
        _lib.orc_h2f.argtypes = [C.c_uint16]
        _lib.orc_rng_seed.restype = C.c_uint64
        _lib.orc_rng_seed.argtypes = [C.c_uint64]
    return _lib


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return a.ctypes.data_as(C.c_void_p)


def _h(a) -> np.ndarray:
    a = np.ascontiguousarray(a)
    assert a.dtype == np.float16, a.dtype
    return a


def _f(a) -> np.ndarray:
    a = np.ascontiguousarray(a)
    assert a.dtype == np.float32, a.dtype
    return a


def _i(a) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.int32)
    return a


def threads() -> int:
    return int(lib().orc_threads())


# ---- f16 ---------------------------------------------------------------------
def f2h_bits(x: np.ndarray) -> np.ndarray:
    x = _f(x)
    y = np.empty(x.shape, np.uint16)
    lib().orc_f2h_n(_p(x), _p(y), C.c_longlong(x.size))
    return y


def h2f_bits(h: np.ndarray) -> np.ndarray:
    h = np.ascontiguousarray(h, dtype=np.uint16)
    y = np.empty(h.shape, np.float32)
    lib().orc_h2f_n(_p(h), _p(y), C.c_longlong(h.size))
    return y


def to_f16(x: np.ndarray) -> np.ndarray:
    """f32 -> f16 with the oracle's own rounding (not numpy's)."""
    return f2h_bits(np.asarray(x, np.float32)).view(np.float16)


class Rng:
    """The reference tests' seeded xorshift generator (src/bench.rs:13-35)."""

    def __init__(self, seed: int):
        self.state = C.c_uint64(lib().orc_rng_seed(C.c_uint64(seed)))

    def uniform(self, n: int) -> np.ndarray:
        out = np.empty(int(n), np.float32)
        lib().orc_rng_uniform(C.byref(self.state), _p(out), C.c_longlong(out.size))
        return out

    def tensor(self, dtype, shape, scale: float = 1.0) -> np.ndarray:
        """``Rng::tensor``: uniform * scale (an f32 product), rounded to dtype."""
        n = int(np.prod(shape)) if len(shape) else 1
        v = self.uniform(n) * np.float32(scale)
        if dtype == np.float16:
            return to_f16(v).reshape(shape)
        return v.astype(np.float32).reshape(shape)


# ---- kernels -------------------------------------------------------------------
def embed(tok, E):
    tok, E = _i(tok), _h(E)
    T, (V, Dm) = tok.shape[0], E.shape
    X = np.empty((T, Dm), np.float32)
    lib().orc_embed(_p(tok), _p(E), _p(X), T, V, Dm)
    return X


def rmsnorm(X, W, eps):
    X, W = _f(X), _h(W)
    T, Dm = X.shape
    Y = np.empty((T, Dm), np.float16)
    lib().orc_rmsnorm(_p(X), _p(W), _p(Y), C.c_float(eps), T, Dm)
    return Y


def rmsnorm_rows(X, idx, W, eps):
    X, idx, W = _f(X), _i(idx), _h(W)
    T, Dm = X.shape
    B = idx.shape[0]
    Y = np.empty((B, Dm), np.float16)
    lib().orc_rmsnorm_rows(_p(X), _p(idx), _p(W), _p(Y), C.c_float(eps), T, B, Dm)
    return Y


def linear(X, W, bk=64):
    X, W = _h(X), _h(W)
    (M, K), N = X.shape, W.shape[0]
    Y = np.empty((M, N), np.float16)
    lib().orc_linear_family(_p(X), _p(W), _p(Y), M, N, K, bk, 0)
    return Y


def linear_residual(X, W, R, bk=64):
    X, W = _h(X), _h(W)
    R = _f(R).copy()
    (M, K), N = X.shape, W.shape[0]
    lib().orc_linear_family(_p(X), _p(W), _p(R), M, N, K, bk, 1)
    return R


def logits(X, W, bk=64):
    X, W = _h(X), _h(W)
    (M, K), N = X.shape, W.shape[0]
    Y = np.empty((M, N), np.float32)
    lib().orc_linear_family(_p(X), _p(W), _p(Y), M, N, K, bk, 2)
    return Y


def gate_up(X, Wg, Wu, bk=64):
    X, Wg, Wu = _h(X), _h(Wg), _h(Wu)
    (M, K), F = X.shape, Wg.shape[0]
    Y = np.empty((M, F), np.float16)
    lib().orc_gate_up(_p(X), _p(Wg), _p(Wu), _p(Y), M, F, K, bk)
    return Y


def matmul(A, B, bk=32):
    A, B = _h(A), _h(B)
    (M, K), N = A.shape, B.shape[1]
    Cm = np.empty((M, N), np.float16)
    lib().orc_matmul(_p(A), _p(B), _p(Cm), M, N, K, bk)
    return Cm


def matmul_block(A, B, r0, r1, c0, c1, bk=32):
    A, B = _h(A), _h(B)
    (M, K), N = A.shape, B.shape[1]
    Cs = np.empty((r1 - r0, c1 - c0), np.float16)
    lib().orc_matmul_block(_p(A), _p(B), _p(Cs), M, N, K, bk, r0, r1, c0, c1)
    return Cs


def rope_q(QKV, pos, Ct, St, H, D):
    QKV, pos, Ct, St = _h(QKV), _i(pos), _f(Ct), _f(St)
    T, W = QKV.shape
    Q = np.zeros((T, H, D), np.float16)
    lib().orc_rope_q(_p(QKV), _p(pos), _p(Ct), _p(St), _p(Q), T, W, Ct.shape[0], H, D)
    return Q


def kv_write(QKV, pos, slot, Ct, St, Kc, Vc, G, D):
    """Returns (Kc, Vc, K, V); Kc/Vc are updated copies of the [NS, G, D] caches."""
    QKV, pos, slot, Ct, St = _h(QKV), _i(pos), _i(slot), _f(Ct), _f(St)
    Kc, Vc = _h(Kc).copy(), _h(Vc).copy()
    T, W = QKV.shape
    NS = Kc.size // (G * D)
    Kd = np.zeros((T, G, D), np.float16)
    Vd = np.zeros((T, G, D), np.float16)
    lib().orc_kv_write(_p(QKV), _p(pos), _p(slot), _p(Ct), _p(St), _p(Kc), _p(Vc), _p(Kd), _p(Vd), T, W, Ct.shape[0],
                       NS, G, D)
    return Kc, Vc, Kd, Vd


def decode_attention(Q, Kc, Vc, table, lens, scale):
    Q, Kc, Vc, table, lens = _h(Q), _h(Kc), _h(Vc), _i(table), _i(lens)
    B, H, D = Q.shape
    NP, P, G, _ = Kc.shape
    MP = table.shape[1]
    O = np.zeros((B, H, D), np.float16)
    lib().orc_decode_attention(_p(Q), _p(Kc), _p(Vc), _p(table), _p(lens), _p(O), C.c_float(scale), B, H, G, D, NP, P,
                               MP)
    return O


def prefill_attention(Q, K, V, starts, scale, BM=64, BN=64):
    Q, K, V, starts = _h(Q), _h(K), _h(V), _i(starts)
    S, H, D = Q.shape
    G = K.shape[1]
    O = np.zeros((S, H, D), np.float16)
    lib().orc_prefill_attention(_p(Q), _p(K), _p(V), _p(starts), _p(O), C.c_float(scale), S, H, G, D, BM, BN)
    return O


def flash_attention(Q, K, V, scale, BM=64, BN=64, heads=None, blocks=None):
    """[H,S,D] causal attention; `heads`/`blocks` = (lo, hi) restrict the programs run (rest stays 0)."""
    Q, K, V = _h(Q), _h(K), _h(V)
    H, S, D = Q.shape
    O = np.zeros((H, S, D), np.float16)
    if heads is None and blocks is None:
        lib().orc_flash_attention(_p(Q), _p(K), _p(V), _p(O), C.c_float(scale), H, S, D, BM, BN)
    else:
        h0, h1 = heads or (0, H)
        b0, b1 = blocks or (-1, -1)
        lib().orc_flash_attention_part(_p(Q), _p(K), _p(V), _p(O), C.c_float(scale), H, S, D, BM, BN, h0, h1, b0, b1)
    return O


def rope_tables(max_pos, head_dim, theta):
    Ct = np.empty((max_pos, head_dim // 2), np.float32)
    St = np.empty((max_pos, head_dim // 2), np.float32)
    lib().orc_rope_tables(_p(Ct), _p(St), max_pos, head_dim, C.c_float(theta))
    return Ct, St


def argmax(x) -> int:
    x = _f(x)
    return int(lib().orc_argmax(_p(x), x.size))


def reference_forward(cfg, weights, tokens):
    """The f32 one-sequence model (src/llm/reference.rs:38-108): logits [ntok, vocab]."""
    tokens = _i(tokens)
    keep = []
    ptrs = (C.c_void_p * (7 * cfg.layers))()
    for i, l in enumerate(weights.layers):
        for j, name in enumerate(("attn_norm", "wqkv", "wo", "mlp_norm", "wg", "wu", "wd")):
            a = _h(getattr(l, name))
            keep.append(a)
            ptrs[7 * i + j] = a.ctypes.data
    embed_, norm_, head_ = _h(weights.embed), _h(weights.norm), _h(weights.head())
    out = np.empty((tokens.size, cfg.vocab), np.float32)
    lib().orc_reference_forward(_p(embed_), ptrs, _p(norm_), _p(head_), _p(tokens), int(tokens.size), _p(out), cfg.dim,
                                cfg.layers, cfg.heads, cfg.kv_heads, cfg.head_dim, cfg.ffn, cfg.vocab,
                                C.c_float(cfg.eps), C.c_float(cfg.rope_theta), cfg.max_pos)
    return out
