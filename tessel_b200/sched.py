"""Continuous batching: sequences join the running batch as cache pages allow,
every step decodes one token for each running sequence, and a sequence leaves
(freeing its pages) as soon as it finishes.

Host-side mirror of tessel's ``src/llm/sched.rs`` (``generate_with``, :52-179):
the same admission rule (pages for the whole sequence reserved up front, the
step's token budget, the batch limit), the same page order (the free list pops
0, 1, 2, ...), slots ``page * P + offset``, packed prefill with per-row
``starts``, and decode steps with block tables and lengths.

One extension (off by default): ``chunk``. The reference needs a prompt to fit
one step (src/llm/sched.rs:76-81). With ``chunk > 0`` a longer prompt is
admitted anyway and fed ``chunk`` tokens at a time as extra rows of the decode
steps, each row attending, through the sequence's block table, to the keys
cached so far (its own chunk's earlier tokens included: a step writes all its
keys before its attention runs). The step says which rows are such pieces
(``engine.Mixed``), and the engine runs them through ``chunk_attention``: the
prefill kernel's tensor-core pipeline with the paged cache as K and V, one CTA
per 256 rows and head, instead of one decode query per token.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import List, Sequence, Tuple

import numpy as np

from .engine import Decode, Engine, Mixed, Packed, Prefill
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
    todo: int = 0  # prompt tokens not yet in the cache (a prompt fed in chunks)


class Scheduler:
    """The state of ``generate_with`` (src/llm/sched.rs:58-68) with its loop body as ``step``:
    one call admits and prefills what fits, or decodes one token for every running sequence."""

    def __init__(self, e: Engine, reqs: Sequence[Request], max_batch: int, packed: bool = True,
                 device_argmax: bool = False, chunk: int = 0):
        self.e, self.reqs, self.packed, self.device_argmax = e, reqs, packed, device_argmax
        self.chunk = max(0, min(chunk, e.lim.max_tokens - 1))
        self.feeding: List[_Seq] = []  # sequences whose (long) prompt is still being fed in chunks
        self.start = time.perf_counter()
        # Pops yield pages 0, 1, 2, ...
        self.free: List[int] = list(range(e.lim.pages - 1, -1, -1))
        self.waiting = deque(range(len(reqs)))
        self.running: List[_Seq] = []
        self.out = [Output() for _ in reqs]
        self.st = Stats()
        self.max_batch = min(max_batch, e.lim.max_tokens)
        # The running sequences' block tables as one padded array, rebuilt only when the set of
        # running sequences changes (pages are reserved for a sequence's whole life).
        self._table_ids: tuple = ()
        self._table_np = np.zeros((0, 0), np.int32)

    def done(self) -> bool:
        return not self.waiting and not self.running and not self.feeding

    def _choose(self, attn, toks, pos, slots, want) -> List[int]:
        if self.device_argmax:
            return [int(t) for t in self.e.step_greedy(toks, pos, slots, attn, want)]
        return [argmax(row) for row in self.e.step(toks, pos, slots, attn, want)]

    def _admit(self) -> List[Tuple[int, List[int]]]:
        """As many waiting prompts as the step's token budget, the batch and the free cache pages
        allow. Pages for a whole sequence are reserved up front."""
        e, p = self.e, self.e.lim.page
        admit: List[Tuple[int, List[int]]] = []
        tokens = 0
        while self.waiting:
            rid = self.waiting[0]
            r = self.reqs[rid]
            need = -(-(len(r.prompt) + r.max_new) // p)
            long = len(r.prompt) > e.lim.max_tokens
            if len(r.prompt) == 0 or (long and not self.chunk) or need > e.lim.max_seq_pages:
                raise ValueError(f"request {rid}: prompt of {len(r.prompt)} tokens does not fit")
            busy = len(self.running) + len(self.feeding) + len(admit)
            if long:
                # Fed in chunks alongside the decode rows: it takes a place in the batch and its pages now.
                if busy >= self.max_batch or need > len(self.free):
                    break
                self.waiting.popleft()
                self.feeding.append(_Seq(rid, [self.free.pop() for _ in range(need)], 0, -1, r.max_new,
                                         len(r.prompt)))
                continue
            room = busy < self.max_batch and tokens + len(r.prompt) <= e.lim.max_tokens
            if not room or need > len(self.free) or (not self.packed and admit):
                break
            self.waiting.popleft()
            tokens += len(r.prompt)
            admit.append((rid, [self.free.pop() for _ in range(need)]))
        return admit

    def decode_inputs(self):
        """One row per running sequence: (tokens, positions, slots, Decode(tables, lens), want)."""
        p = self.e.lim.page
        run = self.running
        toks = [s.last for s in run]
        pos = [s.len for s in run]
        slots = [s.pages[s.len // p] * p + s.len % p for s in run]
        ids = tuple(s.id for s in run)
        if ids != self._table_ids:
            width = max(len(s.pages) for s in run)
            tb = np.zeros((len(run), width), np.int32)
            for b, s in enumerate(run):
                tb[b, :len(s.pages)] = s.pages
            self._table_ids, self._table_np = ids, tb
        return toks, pos, slots, Decode(self._table_np, [s.len + 1 for s in run]), list(range(len(run)))

    def absorb(self, picks: Sequence[int]) -> None:
        """Books one decode step's picks: lengths, outputs, finished sequences and their pages."""
        st, eos = self.st, self.e.cfg.eos
        st.decode_steps += 1
        st.largest_batch = max(st.largest_batch, len(self.running))
        st.decode_tokens += len(self.running)
        keep = []
        for s, t in zip(self.running, picks):
            t = int(t)
            s.len += 1
            s.last = t
            s.left -= 1
            self.out[s.id].tokens.append(t)
            if s.left == 0 or t == eos:
                self.out[s.id].done_s = time.perf_counter() - self.start
                self.free.extend(s.pages)
            else:
                keep.append(s)
        self.running = keep

    def step(self) -> str:
        """Runs one engine step; returns "prefill", "decode", or "idle" when nothing can run."""
        e, p, st, reqs = self.e, self.e.lim.page, self.st, self.reqs
        admit = self._admit()
        if admit:
            toks, pos, slots, starts, last = [], [], [], [], []
            for rid, pages in admit:
                pr = reqs[rid].prompt
                s0, n = len(toks), len(pr)
                toks.extend(pr)
                pos.extend(range(n))
                pg = np.asarray(pages, np.int64)
                i = np.arange(n)
                slots.extend((pg[i // p] * p + i % p).tolist())
                starts.extend([s0] * n)
                last.append(len(toks) - 1)
            attn = Prefill() if len(admit) == 1 else Packed(starts)
            picks = self._choose(attn, toks, pos, slots, last)
            st.prefill_steps += 1
            st.prompt_tokens += len(toks)
            for (rid, pages), t in zip(admit, picks):
                self.out[rid].tokens.append(t)
                self.out[rid].first_token_s = time.perf_counter() - self.start
                s = _Seq(rid, pages, len(reqs[rid].prompt), t, reqs[rid].max_new - 1)
                if s.left == 0 or t == e.cfg.eos:
                    self.out[rid].done_s = time.perf_counter() - self.start
                    self.free.extend(s.pages)
                else:
                    self.running.append(s)
            return "prefill"
        if self.feeding:
            return self._mixed_step()
        if not self.running:
            return "idle"
        t0 = time.perf_counter()
        toks, pos, slots, attn, want = self.decode_inputs()
        self.absorb(self._choose(attn, toks, pos, slots, want))
        st.decode_seconds += time.perf_counter() - t0
        return "decode"

    def _mixed_step(self) -> str:
        """A decode step whose extra rows are the next chunk of each prompt that is being fed."""
        e, p, st, reqs = self.e, self.e.lim.page, self.st, self.reqs
        run = list(self.running)
        toks = [s.last for s in run]
        pos = [s.len for s in run]
        slots = [s.pages[s.len // p] * p + s.len % p for s in run]
        lens = [s.len + 1 for s in run]
        want = list(range(len(run)))
        budget = e.lim.max_tokens - len(run)
        fed = []  # (sequence, tokens fed, row of its last prompt token or -1)
        chunks = []  # (first row, rows, first position) of each piece, for the chunk attention
        first_rows = []  # (row, pages) of each piece's first row: the only row whose table is read
        for s in self.feeding:
            c = min(self.chunk, s.todo, budget)
            if c <= 0:
                continue
            budget -= c
            pr = reqs[s.id].prompt
            chunks.append((len(toks), c, s.len))
            first_rows.append((len(toks), s.pages))
            i = np.arange(s.len, s.len + c)
            toks.extend(pr[s.len:s.len + c])
            pos.extend(i.tolist())
            slots.extend((np.asarray(s.pages, np.int64)[i // p] * p + i % p).tolist())
            lens.extend((i + 1).tolist())
            last = -1
            if c == s.todo:
                last = len(toks) - 1
                want.append(last)
            fed.append((s, c, last))
        # One padded table for the step: a decode row carries its sequence's pages, a piece's
        # first row the piece's; the other rows of a piece are never looked up.
        owners = [(b, s.pages) for b, s in enumerate(run)] + first_rows
        width = max([len(pg) for _, pg in owners] + [1])
        tables = np.zeros((len(toks), width), np.int32)
        for row, pg in owners:
            tables[row, :len(pg)] = pg
        picks = self._choose(Mixed(tables, lens, chunks), toks, pos, slots, want)
        if run:
            self.absorb(picks[:len(run)])
        st.prompt_tokens += sum(c for _, c, _ in fed)
        k = len(run)
        for s, c, last in fed:
            s.len += c
            s.todo -= c
            if last < 0:
                continue
            t = int(picks[k])
            k += 1
            self.feeding.remove(s)
            self.out[s.id].tokens.append(t)
            self.out[s.id].first_token_s = time.perf_counter() - self.start
            s.last, s.left = t, s.left - 1
            if s.left == 0 or t == e.cfg.eos:
                self.out[s.id].done_s = time.perf_counter() - self.start
                self.free.extend(s.pages)
            else:
                self.running.append(s)
        return "mixed"

    def finish(self) -> Tuple[List[Output], Stats]:
        self.st.generated = sum(len(o.tokens) for o in self.out)
        self.st.seconds = time.perf_counter() - self.start
        return self.out, self.st


def generate(e: Engine, reqs: Sequence[Request], max_batch: int) -> Tuple[List[Output], Stats]:
    """Greedy generation for every request; stops a sequence at ``max_new`` tokens or the
    model's end-of-sequence token."""
    return generate_with(e, reqs, max_batch, True)


def generate_with(e: Engine, reqs: Sequence[Request], max_batch: int, packed: bool,
                  device_argmax: bool = False, chunk: int = 0) -> Tuple[List[Output], Stats]:
    """``generate``, choosing whether new prompts share prefill steps (``packed``) or each takes
    its own. ``device_argmax`` picks the tokens on the GPU (``Engine.step_greedy``) instead of
    reading the logits back and choosing on the host as the reference does. ``chunk > 0`` admits
    prompts longer than a step and feeds them that many tokens at a time (see the module text)."""
    s = Scheduler(e, reqs, max_batch, packed, device_argmax, chunk)
    while not s.done():
        if s.step() == "idle" and s.waiting:
            raise ValueError(f"request {s.waiting[0]} cannot be admitted: not enough cache pages")
    return s.finish()
