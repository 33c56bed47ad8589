"""A small fixed-seed model run through the engine, for comparing a tensor-parallel run with
the single-rank run of the SAME model.

One rank of an ``nranks``-way run calls :func:`run`; every rank shards the same full weights
(``Weights.random`` with a fixed seed), so the logits, the greedy tokens and the KV pages of a
run over N ranks can be held against those of one rank: logits within 2e-3 of the largest,
32 greedy decode steps with the same tokens (also with a prompt fed in chunks beside the decodes), pages equal to the
single-rank pages sliced along the KV-head axis, and the normalised activations h (and the final residual stream x)
the same bits on every rank. The tests drive it on the CPU stand-in and on GPUs; the benchmark
prints its summary beside a multi-GPU number (:func:`summary`).

The model has 16 query heads, 8 KV heads and 512 MLP columns, so it shards over 2, 4 and 8
ranks, and a head_dim of 64, so the attention kernels take their tensor-core paths.
"""
from __future__ import annotations

import hashlib
from typing import Callable, Dict, List, Optional

import numpy as np

from .engine import Decode, Engine, Limits, Packed
from .model import Config, Weights, argmax
from .sched import Request, generate_with

DECODE_STEPS = 32


def model():
    cfg = Config(dim=256, layers=2, heads=16, kv_heads=8, head_dim=64, ffn=512, vocab=1000, eps=1e-5,
                 rope_theta=10000.0, max_pos=512, bos=1, eos=-1)
    return cfg, Weights.random(cfg, 13)


def requests(cfg: Config) -> List[Request]:
    g = np.random.default_rng(2)
    return [Request(g.integers(0, cfg.vocab, n).tolist(), DECODE_STEPS + 1) for n in (40, 7, 33)]


CHUNK, CHUNK_NEW = 32, 8


def chunk_requests(cfg: Config) -> List[Request]:
    """A short prompt and one of 100 tokens, which is fed 32 tokens at a time beside the decodes."""
    g = np.random.default_rng(3)
    return [Request(g.integers(0, cfg.vocab, n).tolist(), CHUNK_NEW) for n in (9, 100)]


def run(gpu, rank: int, nranks: int, exchange: Optional[Callable] = None) -> Dict[str, np.ndarray]:
    """Two packed prompts, one decode step, a 3-request greedy generation of 1 + 32 tokens, and a
    2-request generation with one prompt fed in chunks, on rank ``rank`` of ``nranks``. Returns
    the prefill logits ``pre`` [2, vocab], the decode step's logits ``dec`` [2, vocab], layer 1's
    cache shard ``kc``/``vc``, the real rows of x and h after the decode step, ``tokens`` [3, 33]
    and ``chunk_tokens`` [2, 8]."""
    cfg, w = model()
    lim = Limits(page=16, pages=40, max_tokens=128, max_seq_pages=8)
    e = Engine(gpu, w, lim, rank=rank, nranks=nranks, exchange=exchange)
    g = np.random.default_rng(1)
    p1, p2 = g.integers(0, cfg.vocab, 37).tolist(), g.integers(0, cfg.vocab, 20).tolist()
    toks, pos = p1 + p2, list(range(37)) + list(range(20))
    slots = [16 * 3 + i for i in range(37)] + [16 * 9 + i for i in range(20)]
    pre = e.step(toks, pos, slots, Packed([0] * 37 + [37] * 20), [36, 56]).copy()
    t1, t2 = argmax(pre[0]), argmax(pre[1])
    dec = e.step([t1, t2], [37, 20], [16 * 5 + 5, 16 * 10 + 4], Decode([[3, 4, 5], [9, 10]], [38, 21]), [0, 1]).copy()
    kc, vc = e.read_cache(1)
    x = gpu.fetch(e.x, np.float32, (e.tmax, cfg.dim))[:2].copy()
    h = gpu.fetch(e.h, np.float16, (e.tmax, cfg.dim))[:2].copy()
    e2 = Engine(gpu, w, Limits(page=16, pages=64, max_tokens=128, max_seq_pages=8), rank=rank, nranks=nranks,
                exchange=exchange)
    outs, _ = generate_with(e2, requests(cfg), 3, True, device_argmax=True)
    e3 = Engine(gpu, w, Limits(page=16, pages=64, max_tokens=64, max_seq_pages=8), rank=rank, nranks=nranks,
                exchange=exchange)
    couts, _ = generate_with(e3, chunk_requests(cfg), 2, True, device_argmax=True, chunk=CHUNK)
    return dict(pre=pre, dec=dec, kc=kc, vc=vc, x=x, h=h, tokens=np.asarray([o.tokens for o in outs]),
                chunk_tokens=np.asarray([o.tokens for o in couts]))


def rel_err(got: np.ndarray, want: np.ndarray) -> float:
    """max|got - want| / max|want|, the reference's metric (tests/llm.rs:20-23)."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))


def digest(r: Dict[str, np.ndarray]) -> str:
    """A hash of the bits of x and h, to compare ranks without moving the arrays."""
    m = hashlib.sha256()
    m.update(np.ascontiguousarray(r["x"]).tobytes())
    m.update(np.ascontiguousarray(r["h"]).tobytes())
    return m.hexdigest()


def gathered_cache(shards: List[Dict[str, np.ndarray]], name: str) -> np.ndarray:
    """The ranks' cache shards [pages, page, kv_heads / n, head_dim] joined along the KV-head axis."""
    return np.concatenate([np.asarray(r[name]) for r in shards], axis=2)


def summary(one: Dict[str, np.ndarray], shards: List[Dict[str, np.ndarray]], digests: List[str]) -> dict:
    """What a multi-rank run shows against the single-rank run ``one`` of the same model.
    ``shards``: every rank's results in rank order (rank 0's logits and tokens are compared; all
    ranks' cache shards are joined); ``digests``: every rank's :func:`digest`. ``tokens_equal``
    counts the greedy decode steps (of ``decode_steps``) before the first sequence parts ways
    with the single-rank run."""
    mine = shards[0]
    ta, tb = np.asarray(one["tokens"]), np.asarray(mine["tokens"])
    steps = ta.shape[1] - 1
    same = ta == tb
    first_bad = min(int(np.argmin(row)) if not row.all() else row.size for row in same)
    out = {
        "ranks": len(digests),
        "logits_rel_err": max(rel_err(mine["pre"], one["pre"]), rel_err(mine["dec"], one["dec"])),
        "tokens_equal": int(min(steps, max(0, first_bad - 1))) if first_bad < same.shape[1] else int(steps),
        "decode_steps": int(steps),
        "h_bit_identical": len(set(digests)) == 1,
        "chunked_prompt_tokens_equal": bool(np.array_equal(np.asarray(one["chunk_tokens"]), np.asarray(mine["chunk_tokens"]))),
    }
    worst, same_pages = 0.0, True
    for name in ("kc", "vc"):
        full = np.asarray(one[name], np.float32)
        got = gathered_cache(shards, name).astype(np.float32)
        used = np.abs(full).sum(axis=(1, 2, 3)) > 0
        same_pages = same_pages and bool(np.array_equal(np.abs(got).sum(axis=(1, 2, 3)) > 0, used))
        worst = max(worst, rel_err(got[used], full[used]))
    out["kv_pages_rel_err"] = worst
    out["same_pages_written"] = same_pages
    return out
