"""The model on the device: weights, the paged KV cache, activation buffers for
the largest step, and one step of the decoder as a sequence of kernel launches.

Host-side mirror of tessel's ``src/llm/engine.rs``: ``Limits`` (:21-32),
``Attn`` (:35-45), ``padded`` (:94-98), ``Engine::new`` (:150-226),
``Engine::step`` (:275-354) and ``Engine::launch_all`` (:359-529), with the
same padding rules, buffer dtypes and launch order, driving
``libtessel_b200`` through :class:`tessel_b200.gpu.Gpu`.

Beyond the reference: the step's integer inputs go up from page-locked memory
in asynchronous copies; ``rope_q`` and ``kv_write`` run as one launch; prefill
steps beyond 256 rows are padded to a multiple of 256, not to a power of two;
``step_greedy`` picks the tokens on the device so that only ``len(want)``
integers come back instead of ``len(want) * vocab`` floats, and
``decode_resident`` runs decode steps back to back with no host input; and the
model can be tensor-parallel (``rank``/``nranks``): attention and KV heads and
the MLP columns are sharded, o_proj and down_proj produce f32 partials that
are summed across ranks before they are added to the residual stream, by one
NCCL allreduce each or, given ``exchange``, over peer memory: the projection
stores every row into its owner rank's memory and one more kernel sums, adds
the residual, normalises and hands the rows round; greedy steps then split the
LM head's rows across the ranks too.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np

from .gpu import Buf, F32, Gpu, K
from .model import Config, Weights, rope_tables


@dataclass
class Limits:
    """Engine limits (src/llm/engine.rs:21-32)."""
    page: int           # tokens per cache page
    pages: int          # pages in the cache (shared by all sequences)
    max_tokens: int     # most tokens in one step (a prompt, or a batch of decodes)
    max_seq_pages: int  # most pages one sequence holds


class Prefill:
    """One sequence's prompt from position 0: causal over the step's tokens."""


@dataclass
class Packed:
    """Several prompts packed into the step: row r belongs to the sequence whose first row is starts[r]."""
    starts: Sequence[int]


@dataclass
class Decode:
    """One token per sequence against its cache: page tables and lengths (including the token itself).
    ``tables`` is a list of page lists, or an int32 array ``[sequences, pages]`` padded with zeros."""
    tables: Sequence[Sequence[int]]
    lens: Sequence[int]


@dataclass
class Mixed(Decode):
    """A decode step that also carries the next pieces of prompts that do not fit one step:
    ``chunks`` lists (row0, nrows, pos0) for each piece - rows [row0, row0 + nrows) of the step
    are the tokens at positions pos0, pos0 + 1, ... of one sequence, whose pages are
    ``tables[row0]``. Those rows are attended by ``chunk_attention`` (tensor cores, the paged
    cache as K and V); their ``lens`` entries are ignored. Every other row is a decode row."""
    chunks: Sequence[Sequence[int]] = ()


def padded(n: int) -> int:
    """Rows a step is made for: at least 16, rounded up to a power of two (src/llm/engine.rs:94-98)."""
    n = max(n, 16)
    return 1 << (n - 1).bit_length()


def padded_prefill(n: int) -> int:
    """Rows a prefill step is made for. The reference pads every step to a power of two because
    its kernels are compiled per shape; here a prefill step's kernels take ragged row counts and
    are not replayed as graphs, so beyond 256 rows the step is padded to the next multiple of 256
    only (a 1300-token step runs 1536 rows, not 2048). Padding rows write to no slot and no
    wanted row is one of them, so results do not depend on the choice."""
    return padded(n) if n <= 256 else -(-n // 256) * 256


def shard_weights(w: Weights, rank: int, nranks: int) -> Weights:
    """Rank ``rank``'s slice of the model under ``nranks``-way tensor parallelism.

    Query heads, KV heads and MLP columns are split evenly: the three row
    blocks of wqkv are sliced separately, wo and wd keep the matching input
    columns. Norms, embedding and LM head are replicated.
    """
    from .model import Layer
    cfg = w.cfg
    if nranks == 1:
        return w
    if cfg.heads % nranks or cfg.kv_heads % nranks or cfg.ffn % nranks:
        raise ValueError(f"heads {cfg.heads}, kv_heads {cfg.kv_heads} and ffn {cfg.ffn} must divide by {nranks}")
    hd, H, G = cfg.head_dim, cfg.heads, cfg.kv_heads
    hl, gl, fl = H // nranks, G // nranks, cfg.ffn // nranks
    local = Config(**{**cfg.__dict__, "heads": hl, "kv_heads": gl, "ffn": fl})
    layers = []
    for l in w.layers:
        q = l.wqkv[rank * hl * hd:(rank + 1) * hl * hd]
        k = l.wqkv[H * hd + rank * gl * hd:H * hd + (rank + 1) * gl * hd]
        v = l.wqkv[(H + G) * hd + rank * gl * hd:(H + G) * hd + (rank + 1) * gl * hd]
        layers.append(Layer(
            attn_norm=l.attn_norm, wqkv=np.ascontiguousarray(np.concatenate([q, k, v], 0)),
            wo=np.ascontiguousarray(l.wo[:, rank * hl * hd:(rank + 1) * hl * hd]), mlp_norm=l.mlp_norm,
            wg=np.ascontiguousarray(l.wg[rank * fl:(rank + 1) * fl]),
            wu=np.ascontiguousarray(l.wu[rank * fl:(rank + 1) * fl]),
            wd=np.ascontiguousarray(l.wd[:, rank * fl:(rank + 1) * fl])))
    return Weights(local, w.embed, layers, w.norm, w.lm_head)


@dataclass
class _DevLayer:
    n1: Buf
    wqkv: Buf
    wo: Buf
    n2: Buf
    wg: Buf
    wu: Buf
    wd: Buf
    kc: Buf
    vc: Buf


class Engine:
    """``w`` holds the full model; with ``nranks > 1`` this engine keeps rank ``rank``'s shard of it."""

    def __init__(self, gpu: Gpu, w: Weights, lim: Limits, rank: int = 0, nranks: int = 1, sharded: bool = False,
                 exchange=None, fp8: bool = False):
        """``sharded``: ``w`` already is this rank's shard (its ``cfg`` the local shape).
        ``exchange``: with ``nranks > 1``, a function that takes this rank's list of byte strings and
        returns every rank's list (an all-gather on the host). When given, the ranks map each
        other's buffers and the cross-rank sum after o_proj and down_proj runs fused with the
        residual add and the next RMSNorm in one kernel over NVLink (``tp_reduce_norm``) instead
        of linear_f32 -> NCCL allreduce -> residual_add -> rmsnorm.
        ``fp8``: a separate, NON-PARITY mode (single rank): the five projection matrices of every
        layer are quantised to E4M3 with one f32 scale per output row when they are uploaded,
        activations are quantised per row on the device in front of each projection, and the
        projections run on the tensor cores' 8-bit path. Attention, RoPE, the cache, the norms'
        arithmetic and the LM head stay as they are."""
        full = w.cfg
        if fp8 and nranks != 1:
            raise ValueError("the FP8 mode runs on a single rank")
        self.fp8 = fp8
        if full.heads % full.kv_heads or full.head_dim % 2:
            raise ValueError("heads must be a multiple of kv_heads, head_dim even")
        if not sharded:
            w = shard_weights(w, rank, nranks)
        cfg = w.cfg
        self.gpu = gpu
        self.cfg = cfg
        self.full_cfg = full
        self.lim = lim
        self.rank, self.nranks = rank, nranks
        # Time the candidate tiles of each projection on the device the first time a step size is
        # seen and keep the fastest (src/llm/engine.rs:52, :233-270), for steps of at most
        # ``tune_rows`` rows: decode steps are what is replayed thousands of times, while every
        # new prompt length would pay for a tuning pass of its own.
        self.tune = True
        self.tune_rows = 256
        # Run rope_q and kv_write as the epilogue of the QKV projection (head_dim 64 or 128): True,
        # False, or None = decide per step size by timing both forms on the device (where tuning
        # is on; elsewhere fuse when the projection is at least 2048 columns wide: a narrow one,
        # such as an 8-way tensor-parallel rank's, has too few whole-head tiles to fill the SMs).
        self.fuse_rope: Optional[bool] = None
        self._fuse_by_rows: Dict[int, bool] = {}
        # Replay decode steps as CUDA graphs (one launch instead of hundreds).
        self.graphs = True
        self._graph: Dict[tuple, int] = {}
        up = gpu.tensor
        self.embed = up(w.embed)
        self.head = up(w.lm_head) if w.lm_head is not None else self.embed
        self.norm = up(w.norm)
        slots = lim.pages * lim.page
        kv_bytes = slots * cfg.kv_heads * cfg.head_dim * 2
        self.layers: List[_DevLayer] = []
        self.q8: List[Dict[str, Buf]] = []
        for l in w.layers:
            if fp8:
                # E4M3 bytes and row scales instead of the f16 matrices (which are not uploaded).
                from . import fp8 as f8
                q = {}
                for name in ("wqkv", "wo", "wg", "wu", "wd"):
                    m = getattr(l, name)
                    if isinstance(m, np.ndarray):
                        bytes_, scale = f8.quantize_rows(m.astype(np.float32))
                        q[name], q[name + "_s"] = up(bytes_), up(scale)
                    else:
                        # Already on the device: the same rule, by the kernel that quantises activations.
                        rows, cols = m.shape
                        q[name], q[name + "_s"] = gpu.alloc(rows * cols), gpu.alloc(rows * 4)
                        gpu.launch(gpu.kernel("quant_rows", [[rows, cols], [rows, cols], [rows]]),
                                   [up(m), q[name], q[name + "_s"]])
                self.q8.append(q)
                none = Buf(0, 0)
                self.layers.append(_DevLayer(up(l.attn_norm), none, none, up(l.mlp_norm), none, none, none,
                                             gpu.alloc(kv_bytes), gpu.alloc(kv_bytes)))
                continue
            self.layers.append(_DevLayer(up(l.attn_norm), up(l.wqkv), up(l.wo), up(l.mlp_norm), up(l.wg), up(l.wu),
                                         up(l.wd), gpu.alloc(kv_bytes), gpu.alloc(kv_bytes)))
        c, s = rope_tables(cfg)
        self.cos, self.sin = up(c), up(s)
        t = padded(lim.max_tokens)
        self.tmax = t
        hd, gd = cfg.heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim
        a = gpu.alloc
        self.x = a(t * cfg.dim * 4)
        self.h = a(t * cfg.dim * 2)
        self.qkv = a(t * cfg.qkv() * 2)
        self.q = a(t * hd * 2)
        self.k = a(t * gd * 2)
        self.v = a(t * gd * 2)
        self.o = a(t * hd * 2)
        self.mlp = a(t * cfg.ffn * 2)
        self.last = a(t * cfg.dim * 2)
        self.logits = a(t * cfg.vocab * 4)
        # A rank's partial o_proj / down_proj [t, dim] f32 on the NCCL path (sized as an inbox of
        # the peer-memory exchange, whose tile tuning uses it as a stand-in for the real ones).
        self.part = a((t + nranks) * cfg.dim * 4) if nranks > 1 else None
        self.tok, self.pos, self.slot, self.idx = a(t * 4), a(t * 4), a(t * 4), a(t * 4)
        self.table = a(t * lim.max_seq_pages * 4)
        self.lens, self.starts = a(t * 4), a(t * 4)
        self.picked = a(t * 4)
        # Page-locked staging for a step's inputs and results.
        mp = lim.max_seq_pages
        self._stage = gpu.host_array((6 * t + t * mp,), np.int32)
        if fp8:
            # Quantised activations in front of the projections: bytes and one scale per row.
            self.hq, self.hs = a(t * cfg.dim), a(t * 4)
            self.oq, self.os = a(t * hd), a(t * 4)
            self.mq, self.ms = a(t * cfg.ffn), a(t * 4)
        self.meta = a(t * 4 * 4)  # chunk descriptors of a mixed step: (row0, nrows, pos0, -)
        self._meta_stage = gpu.host_array((t, 4), np.int32)
        self._chunks = 0
        self._picked_host = gpu.host_array((t,), np.int32)
        self._logits_host: Optional[np.ndarray] = None
        self._hist: Optional[Buf] = None
        self._hist_rows = 0
        # Greedy steps under tensor parallelism split the LM head's rows (the vocabulary) across the
        # ranks: each rank reads 1/nranks of the head, finds its own first maximum, and the
        # (value, index) pairs are gathered by one small allreduce. Logits for ``step`` still come
        # from the whole head, which every rank keeps (it is the embedding when the two are tied).
        self.vocab_parallel = nranks > 1 and cfg.vocab % nranks == 0 and cfg.vocab <= 1 << 24
        if self.vocab_parallel:
            vs = cfg.vocab // nranks
            self.head_slice = Buf(self.head.ptr + rank * vs * cfg.dim * 2, vs * cfg.dim * 2)
            self.pairs = a(nranks * t * 2 * 4)
        self.tp_table: Optional[Buf] = None
        # With the peer-memory exchange set up, ``fused = False`` falls back to the NCCL path
        # (linear_f32 -> allreduce -> residual_add -> rmsnorm) from the next step on; every rank
        # must switch at the same step.
        self.fused = nranks > 1 and exchange is not None
        if nranks > 1 and exchange is not None:
            # Two inboxes for the projections' partial rows and the landing area for the other
            # owners' finished rows, every word "empty" (0xffffffff) until something arrives; the
            # kernels put that back into what they consume. Separate from ``part``, which the
            # NCCL path fills with partial products.
            inbox = [a((t + nranks) * cfg.dim * 4), a((t + nranks) * cfg.dim * 4)]
            self.tp_landing = a(t * cfg.dim * 4)
            mine = inbox + [self.tp_landing]
            for b in mine:
                gpu.fill(b, 0xFF)
            gpu.sync()  # before any peer may store into them
            self.tp_trace = a(gpu.tp_sizes()[1])
            everyone = exchange([gpu.ipc_export(b) for b in mine])
            cols = [[] for _ in mine]
            for r in range(nranks):
                for i, b in enumerate(mine):
                    cols[i].append(b if r == rank else gpu.ipc_import(everyone[r][i], b.bytes))
            raw = gpu.tp_table(rank, nranks, cols[0], cols[1], cols[2], self.x, self.h, self.tp_trace)
            self.tp_table = gpu.tensor(np.frombuffer(raw, np.uint8).copy())
            # Timing the candidate tiles of ``linear_scatter`` must not leave partial rows in the
            # real inboxes (a word that is not empty counts as arrived): those launches get a
            # table whose every inbox is this rank's own ``part``.
            local = [self.part] * nranks
            raw = gpu.tp_table(rank, nranks, local, local, local, self.x, self.h, None)
            self.tp_tune_table = gpu.tensor(np.frombuffer(raw, np.uint8).copy())

    # -- one step ----------------------------------------------------------------
    def _upload(self, tokens, pos, slots, attn, want):
        """Pads the step's integer inputs and sends them up. Returns (n, t, bw, prefill)."""
        n = len(tokens)
        if n == 0 or n > self.lim.max_tokens or len(pos) != n or len(slots) != n:
            raise ValueError(f"a step of {n} tokens (at most {self.lim.max_tokens})")
        prefill = not isinstance(attn, Decode)
        t = padded_prefill(n) if prefill else padded(n)
        ns = self.lim.pages * self.lim.page
        mp = self.lim.max_seq_pages
        T = self.tmax
        st = self._stage
        g = self.gpu
        # Inputs, padded: token 0 at position 0, writing to no slot.
        tk, ps, sl = st[0:t], st[T:T + t], st[2 * T:2 * T + t]
        tk[:n], tk[n:] = tokens, 0
        ps[:n], ps[n:] = pos, 0
        sl[:n], sl[n:] = slots, ns
        g.write_async(self.tok, 0, tk)
        g.write_async(self.pos, 0, ps)
        g.write_async(self.slot, 0, sl)
        if prefill:
            # Where each row's sequence begins (padding rows: at themselves).
            sr = st[5 * T:5 * T + t]
            if isinstance(attn, Packed):
                if len(attn.starts) != n:
                    raise ValueError("packed prefill: one start per token")
                sr[:n] = attn.starts
            else:
                sr[:n] = 0
            sr[n:] = np.arange(n, t, dtype=np.int32)
            g.write_async(self.starts, 0, sr)
        else:
            tb = st[6 * T:6 * T + t * mp].reshape(t, mp)
            ln = st[4 * T:4 * T + t]
            ln[:] = 0
            if isinstance(attn.tables, np.ndarray):
                # Already padded by the caller (the scheduler keeps it between steps): one copy.
                rows, cols = attn.tables.shape
                tb[:rows, :cols] = attn.tables
                tb[:rows, cols:] = 0
                tb[rows:] = 0
            else:
                tb[:] = 0
                for b, row in enumerate(attn.tables):
                    tb[b, :len(row)] = row
            ln[:len(attn.lens)] = attn.lens
            self._chunks = 0
            if isinstance(attn, Mixed) and len(attn.chunks):
                # Chunk rows are not decode rows: an empty length makes the decode kernel skip them.
                nc = len(attn.chunks)
                self._chunks = padded(nc) if nc > 16 else 1 << (nc - 1).bit_length()
                mt = self._meta_stage[:self._chunks]
                mt[:] = 0
                for c, (row0, nrows, pos0) in enumerate(attn.chunks):
                    mt[c, :3] = (row0, nrows, pos0)
                    ln[row0:row0 + nrows] = 0
                g.write_async(self.meta, 0, mt)
            g.write_async(self.table, 0, tb)
            g.write_async(self.lens, 0, ln)
        # Rows whose logits are wanted.
        bw = padded(len(want)) if len(want) else None
        if bw is not None:
            ix = st[3 * T:3 * T + bw]
            ix[:len(want)] = want
            ix[len(want):] = 0
            g.write_async(self.idx, 0, ix)
        return n, t, bw, prefill

    def _run(self, t: int, prefill: bool, bw: Optional[int], greedy: bool) -> None:
        g = self.gpu
        g.phase = "prefill" if prefill else "decode"
        # Profiling times every launch on its own, so it runs without graphs.
        profiling = g._profiling if hasattr(g, "_profiling") else g.profile is not None
        if (not prefill) and self.graphs and not profiling and bw == t and not self._chunks:
            # A decode step of this size: replay its recorded launches, or run
            # them and record them for the next time.
            key = (t, greedy, self.fused)
            if key in self._graph:
                g.replay(self._graph[key])
            else:
                self.launch_all(t, False, bw, greedy)
                g.sync()
                g.capture_begin()
                try:
                    self.launch_all(t, False, bw, greedy)
                finally:
                    gr = g.capture_end()
                self._graph[key] = gr
        else:
            self.launch_all(t, prefill, bw, greedy)

    def step(self, tokens, pos, slots, attn, want: Sequence[int]) -> np.ndarray:
        """Runs the decoder over ``tokens`` at positions ``pos``, writing their keys and values
        to cache slots ``slots``, and returns the logits of the rows in ``want``: f32
        ``[len(want), vocab]`` (a view of page-locked memory, valid until the next step)."""
        n, t, bw, prefill = self._upload(tokens, pos, slots, attn, want)
        self._run(t, prefill, bw, False)
        if not len(want):
            self.gpu.sync()
            return np.empty((0, self.cfg.vocab), np.float32)
        v = self.cfg.vocab
        if self._logits_host is None or self._logits_host.shape[0] < len(want):
            self._logits_host = self.gpu.host_array((padded(len(want)), v), np.float32)
        out = self._logits_host[:len(want)]
        self.gpu.read(self.logits, 0, out)
        return out

    def step_greedy(self, tokens, pos, slots, attn, want: Sequence[int]) -> np.ndarray:
        """As ``step``, but the first-maximum choice of src/llm/mod.rs:132-140 is made on the
        device: returns int32 ``[len(want)]`` token ids."""
        n, t, bw, prefill = self._upload(tokens, pos, slots, attn, want)
        self._run(t, prefill, bw, True)
        if not len(want):
            self.gpu.sync()
            return np.empty((0,), np.int32)
        out = self._picked_host[:len(want)]
        self.gpu.read(self.picked, 0, out)
        return out

    def decode_resident(self, n: int, steps: int) -> np.ndarray:
        """``steps`` more greedy decode steps for the ``n`` sequences of the decode step that just
        ran (``step_greedy`` with ``Decode``), with no host input in between: after each step a
        small kernel turns the picks into the next step's token, position, cache slot and length
        on the device, and the recorded step is replayed. Returns int32 ``[steps, n]``: the token
        picked by each of these steps. The sequences' block tables must already hold the pages
        their new tokens land in (the scheduler reserves them up front)."""
        from .gpu import I32
        t = padded(n)
        if steps < 1:
            return np.empty((0, n), np.int32)
        if self._hist is None or self._hist_rows < steps:
            self._hist_rows = max(steps, 512)
            self._hist = self.gpu.alloc(self._hist_rows * self.tmax * 4)
        g = self.gpu
        adv = g.kernel("decode_advance", [[t], [t], [t], [t], [t], [t, self.lim.max_seq_pages], [self._hist_rows, t]])
        for s in range(steps):
            g.launch(adv, [self.picked, self.tok, self.pos, self.slot, self.lens, self.table, self._hist, I32(n),
                           I32(self.lim.page), I32(s)])
            self._run(t, False, t, True)
        # Row s of the history holds the picks that FED step s; the last step's own picks are in `picked`.
        out = np.empty((steps, n), np.int32)
        if steps > 1:
            h = np.empty((steps, t), np.int32)
            g.read(self._hist, 0, h)
            out[:-1] = h[1:, :n]
        g.read(self.picked, 0, self._picked_host[:n])
        out[-1] = self._picked_host[:n]
        return out

    # -- the launch sequence -------------------------------------------------------
    def _mm(self, name: str, shapes, args, t: int) -> K:
        """The projection kernel ``name`` for these shapes; the first time (on a device that can),
        its tile candidates are timed on ``args`` - the engine's own buffers with layer 0's
        weights; anything they write, the step rewrites - and the fastest is kept
        (``Engine::mm``, src/llm/engine.rs:233-270)."""
        g = self.gpu
        kern = g.kernel(name, shapes)
        tuned = getattr(g, "tuned", None)
        if self.tune and t <= self.tune_rows and tuned is not None and kern.id not in tuned:
            tuned[kern.id] = g.tune(kern, args)
        return kern

    def _fuse_rope_for(self, t: int, fused_shapes, fused_args, rope_shapes, kv_shapes) -> bool:
        """Whether steps of ``t`` rows run the QKV projection with rope_q / kv_write as its
        epilogue (one kernel) or as projection + ``rope_kv`` (two). Undecided (``fuse_rope`` is
        None) and able to time kernels: both forms are timed once on the engine's buffers, before
        the step's own launches rewrite what they wrote, and the faster is kept."""
        cfg, g = self.cfg, self.gpu
        w, dm, hd = cfg.qkv(), cfg.dim, cfg.head_dim
        if hd not in (64, 128) or dm % 8:
            return False
        if self.fuse_rope is not None:
            return self.fuse_rope
        if t in self._fuse_by_rows:
            return self._fuse_by_rows[t]
        choice = w >= 2048
        if self.tune and t <= self.tune_rows and getattr(g, "tuned", None) is not None:
            l0 = self.layers[0]
            kf, kp = g.kernel("linear_rope_kv", fused_shapes), g.kernel("linear", [[t, dm], [w, dm], [t, w]])
            if kf.id in g.fusion:   # decided by an earlier engine on this context: same kernels, same plans
                self._fuse_by_rows[t] = g.fusion[kf.id]
                return g.fusion[kf.id]
            g.tuned[kf.id] = g.tune(kf, fused_args)
            g.tuned[kp.id] = g.tune(kp, [self.h, l0.wqkv, self.qkv])
            fused_us, plain_us = g.tuned[kf.id][1], g.tuned[kp.id][1]
            rk = g.kernel("rope_kv", [[t, w]] + rope_shapes + kv_shapes)
            args = [self.qkv, self.pos, self.slot, self.cos, self.sin, self.q, l0.kc, l0.vc, self.k, self.v]
            for _ in range(2):
                g.launch(rk, args)
            g.sync()
            g.time_begin()
            for _ in range(8):
                g.launch(rk, args)
            rope_us = g.time_end() * 1000.0 / 8
            if fused_us > 0 and plain_us > 0:
                choice = fused_us < plain_us + rope_us
            g.fusion[kf.id] = choice
        self._fuse_by_rows[t] = choice
        return choice

    def launch_all(self, t: int, prefill: bool, bw: Optional[int], greedy: bool = False) -> None:
        """Launches one step's kernels for ``t`` rows: the decoder, then, for ``bw`` rows of
        logits, the final norm and the LM head (and the token choice when ``greedy``)."""
        cfg, lim, g = self.cfg, self.lim, self.gpu
        dm, nh, ng, hd = cfg.dim, cfg.heads, cfg.kv_heads, cfg.head_dim
        w, f, v = cfg.qkv(), cfg.ffn, cfg.vocab
        ns, mp, npos = lim.pages * lim.page, lim.max_seq_pages, cfg.max_pos
        scale = F32(1.0 / math.sqrt(hd))
        eps = F32(cfg.eps)
        tp = self.nranks > 1
        k = g.kernel
        embed = k("embed", [[t], [v, dm], [t, dm]])
        norm = k("rmsnorm", [[t, dm], [dm], [t, dm]])
        if prefill:
            att = k("prefill_attention", [[t, nh, hd], [t, ng, hd], [t, ng, hd], [t], [t, nh, hd]])
        else:
            att = k("decode_attention", [[t, nh, hd], [lim.pages, lim.page, ng, hd], [lim.pages, lim.page, ng, hd],
                                         [t, mp], [t], [t, nh, hd]])
        chunk_att = None
        if not prefill and self._chunks:
            cache = [lim.pages, lim.page, ng, hd]
            chunk_att = k("chunk_attention", [[t, nh, hd], cache, cache, [t, mp], [self._chunks, 4], [t, nh, hd]])
        if self.fp8:
            g.launch(embed, [self.tok, self.embed, self.x])
            self._launch_layers_q8(t, prefill, att, chunk_att, eps, scale)
            self._launch_head(t, bw, greedy, eps)
            return
        l0 = self.layers[0]
        rope_shapes = [[t], [t], [npos, hd // 2], [npos, hd // 2]]
        kv_shapes = [[t, nh, hd], [ns, ng, hd], [ns, ng, hd], [t, ng, hd], [t, ng, hd]]
        fused_shapes = [[t, dm], [w, dm]] + rope_shapes + [[t, w]] + kv_shapes
        fused_args = [self.h, l0.wqkv, self.pos, self.slot, self.cos, self.sin, self.qkv, self.q, l0.kc, l0.vc,
                      self.k, self.v]
        if self._fuse_rope_for(t, fused_shapes, fused_args, rope_shapes, kv_shapes):
            # The QKV projection rotates and scatters its own output (src/llm/engine.rs:473-488 as
            # one kernel): Q, the dense K and V and the cache pages come straight from the accumulators.
            qkv = self._mm("linear_rope_kv", fused_shapes, fused_args, t)
            ropekv = None
        else:
            qkv = self._mm("linear", [[t, dm], [w, dm], [t, w]], [self.h, l0.wqkv, self.qkv], t)
            # rope_q and kv_write of the reference (src/llm/engine.rs:391-418) run as one launch.
            ropekv = k("rope_kv", [[t, w]] + rope_shapes + kv_shapes)
        gu = self._mm("gate_up", [[t, dm], [f, dm], [f, dm], [t, f]], [self.h, l0.wg, l0.wu, self.mlp], t)
        if self.tp_table is not None and self.fused:
            # Each row of a partial product goes straight into its owner rank's inbox.
            from .gpu import I32
            tb = self.tp_table
            tt = self.tp_tune_table
            oproj = self._mm("linear_scatter", [[t, nh * hd], [dm, nh * hd], [tb.bytes]], [self.o, l0.wo, tt, I32(0)], t)
            down = self._mm("linear_scatter", [[t, f], [dm, f], [tb.bytes]], [self.mlp, l0.wd, tt, I32(1)], t)
        else:
            proj = "linear_f32" if tp else "linear_residual"
            acc = self.part if tp else self.x
            oproj = self._mm(proj, [[t, nh * hd], [dm, nh * hd], [t, dm]], [self.o, l0.wo, acc], t)
            down = self._mm(proj, [[t, f], [dm, f], [t, dm]], [self.mlp, l0.wd, acc], t)
        radd = k("residual_add", [[t, dm], [t, dm]]) if tp else None

        def project(kern: K, x: Buf, wt: Buf) -> None:
            if not tp:
                g.launch(kern, [x, wt, self.x])
                return
            g.launch(kern, [x, wt, self.part])
            g.allreduce(self.part, t * dm, 0)
            g.launch(radd, [self.x, self.part])

        g.launch(embed, [self.tok, self.embed, self.x])
        if self.tp_table is not None and self.fused:
            self._launch_layers_fused(t, prefill, norm, qkv, ropekv, att, oproj, gu, down, eps, scale, chunk_att)
            self._launch_head(t, bw, greedy, eps)
            return
        for l in self.layers:
            g.launch(norm, [self.x, l.n1, self.h, eps])
            self._launch_qkv(qkv, ropekv, l)
            if prefill:
                g.launch(att, [self.q, self.k, self.v, self.starts, self.o, scale])
            else:
                g.launch(att, [self.q, l.kc, l.vc, self.table, self.lens, self.o, scale])
                if chunk_att is not None:
                    g.launch(chunk_att, [self.q, l.kc, l.vc, self.table, self.meta, self.o, scale])
            project(oproj, self.o, l.wo)
            g.launch(norm, [self.x, l.n2, self.h, eps])
            g.launch(gu, [self.h, l.wg, l.wu, self.mlp])
            project(down, self.mlp, l.wd)
        self._launch_head(t, bw, greedy, eps)

    def _launch_qkv(self, qkv: K, ropekv: Optional[K], l: _DevLayer) -> None:
        """QKV projection, rotary embedding and the KV-cache write of one layer: one kernel, or
        (``ropekv`` given) the projection followed by ``rope_kv``."""
        g = self.gpu
        if ropekv is None:
            g.launch(qkv, [self.h, l.wqkv, self.pos, self.slot, self.cos, self.sin, self.qkv, self.q, l.kc, l.vc,
                           self.k, self.v])
            return
        g.launch(qkv, [self.h, l.wqkv, self.qkv])
        g.launch(ropekv, [self.qkv, self.pos, self.slot, self.cos, self.sin, self.q, l.kc, l.vc, self.k, self.v])

    def _launch_layers_q8(self, t, prefill, att, chunk_att, eps, scale) -> None:
        """The decoder layers in the FP8 mode: rmsnorm_q8 / quant_rows hand E4M3 rows and their
        scales to linear_q8, gate_up_q8 and linear_residual_q8; the rest of a layer is unchanged."""
        cfg, lim, g, k = self.cfg, self.lim, self.gpu, self.gpu.kernel
        dm, nh, ng, hd = cfg.dim, cfg.heads, cfg.kv_heads, cfg.head_dim
        w, f = cfg.qkv(), cfg.ffn
        ns, npos = lim.pages * lim.page, cfg.max_pos
        normq = k("rmsnorm_q8", [[t, dm], [dm], [t, dm], [t]])
        qkv = k("linear_q8", [[t, dm], [t], [w, dm], [w], [t, w]])
        ropekv = k("rope_kv", [[t, w], [t], [t], [npos, hd // 2], [npos, hd // 2], [t, nh, hd], [ns, ng, hd],
                               [ns, ng, hd], [t, ng, hd], [t, ng, hd]])
        quant_o = k("quant_rows", [[t, nh * hd], [t, nh * hd], [t]])
        oproj = k("linear_residual_q8", [[t, nh * hd], [t], [dm, nh * hd], [dm], [t, dm]])
        gu = k("gate_up_q8", [[t, dm], [t], [f, dm], [f], [f, dm], [f], [t, f]])
        quant_m = k("quant_rows", [[t, f], [t, f], [t]])
        down = k("linear_residual_q8", [[t, f], [t], [dm, f], [dm], [t, dm]])
        for l, q in zip(self.layers, self.q8):
            g.launch(normq, [self.x, l.n1, self.hq, self.hs, eps])
            g.launch(qkv, [self.hq, self.hs, q["wqkv"], q["wqkv_s"], self.qkv])
            g.launch(ropekv, [self.qkv, self.pos, self.slot, self.cos, self.sin, self.q, l.kc, l.vc, self.k, self.v])
            if prefill:
                g.launch(att, [self.q, self.k, self.v, self.starts, self.o, scale])
            else:
                g.launch(att, [self.q, l.kc, l.vc, self.table, self.lens, self.o, scale])
                if chunk_att is not None:
                    g.launch(chunk_att, [self.q, l.kc, l.vc, self.table, self.meta, self.o, scale])
            g.launch(quant_o, [self.o, self.oq, self.os])
            g.launch(oproj, [self.oq, self.os, q["wo"], q["wo_s"], self.x])
            g.launch(normq, [self.x, l.n2, self.hq, self.hs, eps])
            g.launch(gu, [self.hq, self.hs, q["wg"], q["wg_s"], q["wu"], q["wu_s"], self.mlp])
            g.launch(quant_m, [self.mlp, self.mq, self.ms])
            g.launch(down, [self.mq, self.ms, q["wd"], q["wd_s"], self.x])

    def _launch_layers_fused(self, t, prefill, norm, qkv, ropekv, att, oproj, gu, down, eps, scale, chunk_att=None) -> None:
        """The decoder layers under tensor parallelism with the fused cross-rank reduction: o_proj
        and down_proj store each row of their partial product into the inbox of the rank that owns
        the row (``linear_scatter``), and one ``tp_reduce_norm`` then sums the inbox into the
        residual stream and leaves the next layer input h on every rank."""
        from .gpu import I32
        g, dm = self.gpu, self.cfg.dim
        tpk = g.kernel("tp_reduce_norm", [[self.tp_table.bytes], [dm], [t, dm]])
        g.launch(norm, [self.x, self.layers[0].n1, self.h, eps])
        for i, l in enumerate(self.layers):
            self._launch_qkv(qkv, ropekv, l)
            if prefill:
                g.launch(att, [self.q, self.k, self.v, self.starts, self.o, scale])
            else:
                g.launch(att, [self.q, l.kc, l.vc, self.table, self.lens, self.o, scale])
                if chunk_att is not None:
                    g.launch(chunk_att, [self.q, l.kc, l.vc, self.table, self.meta, self.o, scale])
            g.launch(oproj, [self.o, l.wo, self.tp_table, I32(0)])
            g.launch(tpk, [self.tp_table, l.n2, self.x, eps, I32(0), I32(1), I32(self.nranks)])
            g.launch(gu, [self.h, l.wg, l.wu, self.mlp])
            g.launch(down, [self.mlp, l.wd, self.tp_table, I32(1)])
            last = i + 1 == len(self.layers)
            nxt = l.n2 if last else self.layers[i + 1].n1
            g.launch(tpk, [self.tp_table, nxt, self.x, eps, I32(1), I32(0 if last else 1), I32(self.nranks)])

    def _launch_head(self, t: int, bw: Optional[int], greedy: bool, eps) -> None:
        cfg, g, k = self.cfg, self.gpu, self.gpu.kernel
        dm, v = cfg.dim, cfg.vocab
        if bw is None:
            return
        fin = k("rmsnorm_rows", [[t, dm], [bw], [dm], [bw, dm]])
        g.launch(fin, [self.x, self.idx, self.norm, self.last, eps])
        if greedy and self.vocab_parallel:
            from .gpu import I32
            r, n = self.rank, self.nranks
            vs = v // n
            part = self._mm("logits", [[bw, dm], [vs, dm], [bw, vs]], [self.last, self.head_slice, self.logits], bw)
            g.launch(part, [self.last, self.head_slice, self.logits])
            g.launch(k("argmax_partial", [[bw, vs], [n, bw, 2]]), [self.logits, self.pairs, I32(r), I32(r * vs)])
            g.allreduce(self.pairs, n * bw * 2, 0)
            g.launch(k("argmax_merge", [[n, bw, 2], [bw]]), [self.pairs, self.picked])
            return
        # Under tensor parallelism every rank computes these logits from the same x and the host
        # picks from its own copy: the ranks must run the same tile, so this one is not tuned.
        if self.nranks == 1:
            head = self._mm("logits", [[bw, dm], [v, dm], [bw, v]], [self.last, self.head, self.logits], bw)
        else:
            head = k("logits", [[bw, dm], [v, dm], [bw, v]])
        g.launch(head, [self.last, self.head, self.logits])
        if greedy:
            pick = k("argmax_rows", [[bw, v], [bw]])
            g.launch(pick, [self.logits, self.picked])

    # -- inspection (tests, parity checks) ------------------------------------------
    def read_cache(self, layer: int):
        """The K and V caches of one layer as f16 ``[pages, page, kv_heads, head_dim]`` arrays."""
        shape = (self.lim.pages, self.lim.page, self.cfg.kv_heads, self.cfg.head_dim)
        l = self.layers[layer]
        return self.gpu.fetch(l.kc, np.float16, shape), self.gpu.fetch(l.vc, np.float16, shape)
