"""The model's shape, weights, rotary tables and greedy choice.

Host-side mirror of tessel's ``src/llm/mod.rs``: ``Config`` (:15-53),
``Layer`` / ``Weights`` (:55-114), ``rope_tables`` (:116-129) and ``argmax``
(:131-140). Weights are numpy ``float16`` arrays, matrices ``[out, in]``.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np


@dataclass
class Config:
    dim: int
    layers: int
    heads: int
    kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    eps: float = 1e-5
    rope_theta: float = 10000.0
    max_pos: int = 2048
    bos: int = 1
    eos: int = 2

    def qkv(self) -> int:
        """Width of the fused QKV projection's output."""
        return (self.heads + 2 * self.kv_heads) * self.head_dim

    @staticmethod
    def tiny() -> "Config":
        """A small model for tests (src/llm/mod.rs:37-52)."""
        return Config(dim=64, layers=2, heads=4, kv_heads=2, head_dim=16, ffn=128, vocab=256, eps=1e-5,
                      rope_theta=10000.0, max_pos=256, bos=1, eos=2)

    @staticmethod
    def tinyllama(max_pos: int = 2048) -> "Config":
        """TinyLlama-1.1B's shape."""
        return Config(dim=2048, layers=22, heads=32, kv_heads=4, head_dim=64, ffn=5632, vocab=32000, eps=1e-5,
                      rope_theta=10000.0, max_pos=max_pos, bos=1, eos=-1)

    @staticmethod
    def llama3_8b(max_pos: int = 2304) -> "Config":
        """Llama-3-8B's shape."""
        return Config(dim=4096, layers=32, heads=32, kv_heads=8, head_dim=128, ffn=14336, vocab=128256, eps=1e-5,
                      rope_theta=500000.0, max_pos=max_pos, bos=1, eos=-1)


@dataclass
class DevArray:
    """A tensor that already lives in device memory (allocated by another library of this
    process, which ``keep`` keeps alive): accepted wherever weights take a numpy array."""
    ptr: int
    shape: tuple
    dtype: object
    keep: object = None

    @property
    def nbytes(self) -> int:
        return int(np.prod(self.shape)) * np.dtype(self.dtype).itemsize


@dataclass
class Layer:
    attn_norm: np.ndarray
    wqkv: np.ndarray  # [(H + 2G) * D, dim]: q, k and v projections stacked
    wo: np.ndarray
    mlp_norm: np.ndarray
    wg: np.ndarray
    wu: np.ndarray
    wd: np.ndarray


class Rng:
    """The reference's seeded xorshift generator (src/bench.rs:13-35), run in the native library."""

    def __init__(self, seed: int):
        from . import _lib
        self._l = _lib.lib()
        self.state = C.c_uint64(self._l.tb200_rng_seed(seed))

    def uniform(self, n: int) -> np.ndarray:
        out = np.empty(int(n), np.float32)
        self._l.tb200_rng_uniform(C.byref(self.state), out.ctypes.data_as(C.c_void_p), out.size)
        return out


@dataclass
class Weights:
    cfg: Config
    embed: np.ndarray
    layers: List[Layer]
    norm: np.ndarray
    lm_head: Optional[np.ndarray] = None  # None when tied to the embedding

    def head(self) -> np.ndarray:
        return self.lm_head if self.lm_head is not None else self.embed

    @staticmethod
    def random(cfg: Config, seed: int) -> "Weights":
        """Uniform weights scaled by 1/sqrt(fan-in), drawn in the order of src/llm/mod.rs:80-108."""
        r = Rng(seed)

        def m(rows: int, cols: int) -> np.ndarray:
            s = np.float32(1.0) / np.sqrt(np.float32(cols))
            return (r.uniform(rows * cols) * s).astype(np.float16).reshape(rows, cols)

        one = np.ones(cfg.dim, np.float16)
        layers = []
        for _ in range(cfg.layers):
            layers.append(Layer(attn_norm=one.copy(), wqkv=m(cfg.qkv(), cfg.dim), wo=m(cfg.dim, cfg.heads * cfg.head_dim),
                                mlp_norm=one.copy(), wg=m(cfg.ffn, cfg.dim), wu=m(cfg.ffn, cfg.dim),
                                wd=m(cfg.dim, cfg.ffn)))
        embed = (m(cfg.vocab, cfg.dim).astype(np.float32) * np.float32(8.0)).astype(np.float16)
        return Weights(cfg, embed, layers, one.copy(), m(cfg.vocab, cfg.dim))

    @staticmethod
    def gaussian(cfg: Config, seed: int, std: float = 0.02, tied: bool = False) -> "Weights":
        """Random-init weights ~N(0, std), RMSNorm gains 1: the benchmark configurations' initialisation."""
        g = np.random.default_rng(seed)

        def m(rows: int, cols: int) -> np.ndarray:
            out = np.empty((rows, cols), np.float16)
            step = max(1, (1 << 24) // cols)
            for r0 in range(0, rows, step):
                r1 = min(rows, r0 + step)
                out[r0:r1] = (g.standard_normal((r1 - r0, cols), dtype=np.float32) * np.float32(std)).astype(np.float16)
            return out

        one = np.ones(cfg.dim, np.float16)
        layers = [Layer(one.copy(), m(cfg.qkv(), cfg.dim), m(cfg.dim, cfg.heads * cfg.head_dim), one.copy(),
                        m(cfg.ffn, cfg.dim), m(cfg.ffn, cfg.dim), m(cfg.dim, cfg.ffn)) for _ in range(cfg.layers)]
        embed = m(cfg.vocab, cfg.dim)
        return Weights(cfg, embed, layers, one.copy(), None if tied else m(cfg.vocab, cfg.dim))


def rope_tables(cfg: Config):
    """cos and sin of every position's rotation angles, [max_pos, D/2] each, computed in f64."""
    h = cfg.head_dim // 2
    # f32 theta widened to f64, as `cfg.rope_theta as f64` does.
    theta = np.float64(np.float32(cfg.rope_theta))
    inv = np.power(theta, -(2.0 * np.arange(h, dtype=np.float64)) / np.float64(cfg.head_dim))
    a = np.arange(cfg.max_pos, dtype=np.float64)[:, None] * inv[None, :]
    return np.cos(a).astype(np.float32), np.sin(a).astype(np.float32)


def argmax(xs: np.ndarray) -> int:
    """The index of the largest value (the first, on ties; a NaN never beats anything)."""
    xs = np.asarray(xs)
    if xs.size == 0 or np.isnan(xs[0]):
        return 0
    return int(np.argmax(np.where(np.isnan(xs), -np.inf, xs)))
