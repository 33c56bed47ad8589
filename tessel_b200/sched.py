"""Continuous batching: sequences join the running batch as cache pages allow,
every step decodes one token for each running sequence, and a sequence leaves
(freeing its pages) as soon as it finishes.

Host-side mirror of tessel's ``src/llm/sched.rs`` (``generate_with``, :52-179):
the same admission rule (pages for the whole sequence reserved up front, the
step's token budget, the batch limit), the same page order (the free list pops
0, 1, 2, ...), slots ``page * P + offset``, packed prefill with per-row
``starts``, and decode steps with block tables and lengths.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import List, Sequence, Tuple

import numpy as np

from .engine import Decode, Engine, Packed, Prefill
from .model import argmax


@dataclass
class Request:
    prompt: Sequence[int]
    max_new: int


@dataclass
class Output:
    tokens: List[int] = field(default_factory=list)
    first_token_s: float = 0.0  # seconds from the start of `generate` to the first new token
    done_s: float = 0.0


@dataclass
class Stats:
    prefill_steps: int = 0
    decode_steps: int = 0
    prompt_tokens: int = 0
    generated: int = 0
    seconds: float = 0.0
    decode_seconds: float = 0.0  # seconds in decode steps, and the tokens they produced
    decode_tokens: int = 0
    largest_batch: int = 0


@dataclass
class _Seq:
    id: int
    pages: List[int]
    len: int  # tokens in the cache
    last: int
    left: int


def generate(e: Engine, reqs: Sequence[Request], max_batch: int) -> Tuple[List[Output], Stats]:
    """Greedy generation for every request; stops a sequence at ``max_new`` tokens or the
    model's end-of-sequence token."""
    return generate_with(e, reqs, max_batch, True)


def generate_with(e: Engine, reqs: Sequence[Request], max_batch: int, packed: bool,
                  device_argmax: bool = False) -> Tuple[List[Output], Stats]:
    """``generate``, choosing whether new prompts share prefill steps (``packed``) or each takes
    its own. ``device_argmax`` picks the tokens on the GPU (``Engine.step_greedy``) instead of
    reading the logits back and choosing on the host as the reference does."""
    start = time.perf_counter()
    p = e.lim.page
    free: List[int] = list(range(e.lim.pages - 1, -1, -1))
    waiting = deque(range(len(reqs)))
    running: List[_Seq] = []
    out = [Output() for _ in reqs]
    st = Stats()
    max_batch = min(max_batch, e.lim.max_tokens)
    eos = e.cfg.eos

    def choose(attn, toks, pos, slots, want) -> List[int]:
        if device_argmax:
            return [int(t) for t in e.step_greedy(toks, pos, slots, attn, want)]
        return [argmax(row) for row in e.step(toks, pos, slots, attn, want)]

    while waiting or running:
        # Admit what fits, packing the new prompts into one prefill step.
        admit: List[Tuple[int, List[int]]] = []
        tokens = 0
        while waiting:
            rid = waiting[0]
            r = reqs[rid]
            need = -(-(len(r.prompt) + r.max_new) // p)
            if len(r.prompt) == 0 or len(r.prompt) > e.lim.max_tokens or need > e.lim.max_seq_pages:
                raise ValueError(f"request {rid}: prompt of {len(r.prompt)} tokens does not fit")
            room = len(running) + len(admit) < max_batch and tokens + len(r.prompt) <= e.lim.max_tokens
            if not room or need > len(free) or (not packed and admit):
                break
            waiting.popleft()
            tokens += len(r.prompt)
            admit.append((rid, [free.pop() for _ in range(need)]))
        if admit:
            toks, pos, slots, starts, last = [], [], [], [], []
            for rid, pages in admit:
                pr = reqs[rid].prompt
                s0 = len(toks)
                n = len(pr)
                toks.extend(pr)
                pos.extend(range(n))
                pg = np.asarray(pages, np.int64)
                i = np.arange(n)
                slots.extend((pg[i // p] * p + i % p).tolist())
                starts.extend([s0] * n)
                last.append(len(toks) - 1)
            attn = Prefill() if len(admit) == 1 else Packed(starts)
            picks = choose(attn, toks, pos, slots, last)
            st.prefill_steps += 1
            st.prompt_tokens += len(toks)
            for (rid, pages), t in zip(admit, picks):
                n = len(reqs[rid].prompt)
                out[rid].tokens.append(t)
                out[rid].first_token_s = time.perf_counter() - start
                s = _Seq(rid, pages, n, t, reqs[rid].max_new - 1)
                if s.left == 0 or t == eos:
                    out[rid].done_s = time.perf_counter() - start
                    free.extend(s.pages)
                else:
                    running.append(s)
            continue
        if not running:
            continue
        # One token for every running sequence.
        t0 = time.perf_counter()
        toks = [s.last for s in running]
        pos = [s.len for s in running]
        slots = [s.pages[s.len // p] * p + s.len % p for s in running]
        tables = [s.pages for s in running]
        lens = [s.len + 1 for s in running]
        want = list(range(len(running)))
        picks = choose(Decode(tables, lens), toks, pos, slots, want)
        st.decode_steps += 1
        st.largest_batch = max(st.largest_batch, len(running))
        st.decode_tokens += len(running)
        keep = []
        for s, t in zip(running, picks):
            s.len += 1
            s.last = t
            s.left -= 1
            out[s.id].tokens.append(t)
            if s.left == 0 or t == eos:
                out[s.id].done_s = time.perf_counter() - start
                free.extend(s.pages)
            else:
                keep.append(s)
        running = keep
        st.decode_seconds += time.perf_counter() - t0
    st.generated = sum(len(o.tokens) for o in out)
    st.seconds = time.perf_counter() - start
    return out, st
