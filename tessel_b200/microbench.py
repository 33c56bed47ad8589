"""Single-kernel timings at the benchmark configurations' shapes, through the C ABI.

    python -m tessel_b200.microbench decode [--seqs 256 --ctx-lo 512 --ctx-hi 2304 --heads 32 --kv-heads 8 --dim 128]
    python -m tessel_b200.microbench gemm   [--m 4096 --n 4096 --k 4096] [--kind matmul|linear|gate_up|linear_residual]
    python -m tessel_b200.microbench flash  [--heads 256 --seq 4096 --dim 128]
    python -m torch.distributed.run --nproc-per-node N -m tessel_b200.microbench exchange [--k-cols 4096]
    python -m tessel_b200.microbench qkv    [--m 256 --k 4096 --heads 32 --kv-heads 8 --dim 128]
    python -m tessel_b200.microbench chunked [--prompt 4096 --chunk 512 --layers 32]
    python -m tessel_b200.microbench flash --packed [--prompts 8 --seq 4096 --heads 32 --kv-heads 8 --dim 128]

Each prints one JSON line: the mean device time per launch (CUDA events on the launching
stream, one pair per iteration, after warm-up; a 256 MB buffer is overwritten between
iterations so that nothing is served from L2 by accident), the algorithmic bytes and flops of
the launch (byte/flop conventions of tessel's src/bench.rs:83-84 and :132-133; KV counted once
per KV head), and the fraction of the measured peak. Inputs are generated on the device.
Small sizes of the same commands are what the profiler captures are taken on.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import numpy as np


def _peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        j = json.load(open(p))
        return float(j["hbm_gbs"]), float(j["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


class Timer:
    """Times `fn` per launch on torch's current stream, which the library is switched to."""

    def __init__(self, gpu, torch):
        self.gpu, self.torch = gpu, torch
        self.stream = torch.cuda.Stream()
        torch.cuda.set_stream(self.stream)
        gpu.set_stream(self.stream.cuda_stream)
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def run(self, fn, iters: int, warmup: int = 3):
        torch = self.torch
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        ms = []
        for _ in range(iters):
            self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(self.stream)
            fn()
            b.record(self.stream)
            b.synchronize()
            ms.append(a.elapsed_time(b))
        self.gpu.sync()
        return float(np.mean(ms)), float(np.min(ms))


def decode(gpu, torch, seqs=256, ctx_lo=512, ctx_hi=2304, heads=32, kv_heads=8, dim=128, iters=20, seed=0):
    from .gpu import Buf, F32
    P = 16
    g = np.random.default_rng(seed)
    lens = g.integers(ctx_lo, ctx_hi + 1, seqs).astype(np.int32)
    pages = [-(-int(l) // P) for l in lens]
    NP, MP = sum(pages) + 3, max(pages)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    kc = torch.empty((NP, P, kv_heads, dim), dtype=torch.float16, device="cuda").normal_(generator=gen)
    vc = torch.empty((NP, P, kv_heads, dim), dtype=torch.float16, device="cuda").normal_(generator=gen)
    q = torch.empty((seqs, heads, dim), dtype=torch.float16, device="cuda").normal_(generator=gen)
    o = torch.zeros_like(q)
    perm = g.permutation(NP).astype(np.int32)
    table = np.zeros((seqs, MP), np.int32)
    at = 0
    for b, n in enumerate(pages):
        table[b, :n] = perm[at:at + n]
        at += n
    tb, ln = torch.from_numpy(table).cuda(), torch.from_numpy(lens).cuda()
    k = gpu.kernel("decode_attention", [list(q.shape), list(kc.shape), list(vc.shape), list(tb.shape), [seqs],
                                        list(q.shape)])
    args = [Buf(t.data_ptr(), t.numel() * t.element_size()) for t in (q, kc, vc, tb, ln, o)] + [F32(1 / math.sqrt(dim))]
    t = Timer(gpu, torch)
    mean, best = t.run(lambda: gpu.launch(k, args), iters)
    kv = 4.0 * kv_heads * dim * float(lens.sum())
    nbytes = kv + 4.0 * seqs * heads * dim + 4.0 * sum(pages) + 4.0 * seqs
    hbm, _, kind = _peaks()
    gbs = nbytes / (mean * 1e-3) / 1e9
    return {"kernel": "decode_attention", "seqs": seqs, "ctx": [ctx_lo, ctx_hi], "heads": heads, "kv_heads": kv_heads,
            "head_dim": dim, "ms": mean, "ms_min": best, "algorithmic_bytes": nbytes, "gbs": gbs, "peak_gbs": hbm,
            "frac": gbs / hbm, "peak_kind": kind, "device_bytes": int(kc.numel() * 4)}


def gemm(gpu, torch, m=4096, n=4096, k=4096, kind="matmul", iters=20, seed=0):
    from .gpu import Buf
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)

    def u(*shape, scale=1.0):
        return (torch.rand(shape, dtype=torch.float32, device="cuda", generator=gen) * 2 - 1).mul_(scale).half()

    buf = lambda t: Buf(t.data_ptr(), t.numel() * t.element_size())
    a = u(m, k)
    if kind == "matmul":
        b, c = u(k, n), torch.zeros((m, n), dtype=torch.float16, device="cuda")
        kern, args, nb = gpu.kernel("matmul", [[m, k], [k, n], [m, n]]), [buf(a), buf(b), buf(c)], 1
        out_bytes = 2
    elif kind in ("linear_q8", "linear_residual_q8", "gate_up_q8"):
        # FP8 mode: E4M3 bytes (finite codes only) with per-row scales; flops as the f16 kinds, bytes halved.
        def q(*shape):
            mag = torch.randint(0, 0x78, shape, dtype=torch.uint8, device="cuda", generator=gen)
            sign = torch.randint(0, 2, shape, dtype=torch.uint8, device="cuda", generator=gen) * 0x80
            return mag | sign

        sc = lambda r: torch.full((r,), 1.0 / 448.0, dtype=torch.float32, device="cuda")
        aq, sa, bq, sb = q(m, k), sc(m), q(n, k), sc(n)
        f32 = kind == "linear_residual_q8"
        c = torch.zeros((m, n), dtype=torch.float32 if f32 else torch.float16, device="cuda")
        if kind == "gate_up_q8":
            b2q, sb2 = q(n, k), sc(n)
            kern = gpu.kernel(kind, [[m, k], [m], [n, k], [n], [n, k], [n], [m, n]])
            args, nb = [buf(aq), buf(sa), buf(bq), buf(sb), buf(b2q), buf(sb2), buf(c)], 2
        else:
            kern = gpu.kernel(kind, [[m, k], [m], [n, k], [n], [m, n]])
            args, nb = [buf(aq), buf(sa), buf(bq), buf(sb), buf(c)], 1
        t = Timer(gpu, torch)
        mean, best = t.run(lambda: gpu.launch(kern, args), iters)
        flops = 2.0 * m * n * k * nb
        nbytes = 1.0 * (m * k + nb * k * n) + (8 if f32 else 2) * m * n
        hbm, tf, kindp = _peaks()
        return {"kernel": kind, "m": m, "n": n, "k": k, "ms": mean, "ms_min": best, "flops": flops,
                "algorithmic_bytes": nbytes, "tflops": flops / (mean * 1e-3) / 1e12, "gbs": nbytes / (mean * 1e-3) / 1e9,
                "frac_hbm": nbytes / (mean * 1e-3) / 1e9 / hbm, "peak_kind": kindp,
                "note": "the tensor peak of record is the f16 one; no FP8 peak is measured on this pool"}
    elif kind == "gate_up":
        b, b2 = u(n, k, scale=0.05), u(n, k, scale=0.05)
        c = torch.zeros((m, n), dtype=torch.float16, device="cuda")
        kern = gpu.kernel("gate_up", [[m, k], [n, k], [n, k], [m, n]])
        args, nb, out_bytes = [buf(a), buf(b), buf(b2), buf(c)], 2, 2
    else:
        b = u(n, k, scale=0.05)
        f32 = kind in ("linear_residual", "logits", "linear_f32")
        c = torch.zeros((m, n), dtype=torch.float32 if f32 else torch.float16, device="cuda")
        kern, args, nb = gpu.kernel(kind, [[m, k], [n, k], [m, n]]), [buf(a), buf(b), buf(c)], 1
        out_bytes = (8 if kind == "linear_residual" else 4) if f32 else 2
    t = Timer(gpu, torch)
    mean, best = t.run(lambda: gpu.launch(kern, args), iters)
    flops = 2.0 * m * n * k * nb
    nbytes = 2.0 * (m * k + nb * k * n) + out_bytes * m * n
    hbm, tf, kindp = _peaks()
    return {"kernel": kind, "m": m, "n": n, "k": k, "ms": mean, "ms_min": best, "flops": flops,
            "algorithmic_bytes": nbytes, "tflops": flops / (mean * 1e-3) / 1e12, "peak_tflops": tf,
            "frac_tensor": flops / (mean * 1e-3) / 1e12 / tf, "gbs": nbytes / (mean * 1e-3) / 1e9,
            "frac_hbm": nbytes / (mean * 1e-3) / 1e9 / hbm, "peak_kind": kindp}


def flash(gpu, torch, heads=256, seq=4096, dim=128, iters=10, seed=0):
    from .gpu import Buf, F32
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    q, k, v = (torch.empty((heads, seq, dim), dtype=torch.float16, device="cuda").normal_(generator=gen)
               for _ in range(3))
    o = torch.zeros_like(q)
    kern = gpu.kernel("flash_attention", [list(q.shape)] * 4)
    args = [Buf(t.data_ptr(), t.numel() * t.element_size()) for t in (q, k, v, o)] + [F32(1 / math.sqrt(dim))]
    t = Timer(gpu, torch)
    mean, best = t.run(lambda: gpu.launch(kern, args), iters)
    flops = 2.0 * 2.0 * heads * seq * seq * dim / 2.0
    nbytes = 2.0 * 4.0 * heads * seq * dim
    _, tf, kindp = _peaks()
    return {"kernel": "flash_attention", "heads": heads, "seq": seq, "head_dim": dim, "ms": mean, "ms_min": best,
            "flops": flops, "algorithmic_bytes": nbytes, "tflops": flops / (mean * 1e-3) / 1e12, "peak_tflops": tf,
            "frac_tensor": flops / (mean * 1e-3) / 1e12 / tf, "peak_kind": kindp}


def flash_packed(gpu, torch, prompts=8, seq=4096, heads=32, kv_heads=32, dim=128, iters=10, seed=0):
    """Benchmark configuration 3 in the engine's own form: `prompts` prompts of `seq` tokens packed
    into one step of `prefill_attention` (Q/O [S,H,D], K/V [S,G,D], per-row starts)."""
    from .gpu import Buf, F32
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    S = prompts * seq
    q = torch.empty((S, heads, dim), dtype=torch.float16, device="cuda").normal_(generator=gen)
    k, v = (torch.empty((S, kv_heads, dim), dtype=torch.float16, device="cuda").normal_(generator=gen) for _ in range(2))
    o = torch.zeros_like(q)
    starts = (torch.arange(S, dtype=torch.int32, device="cuda") // seq) * seq
    kern = gpu.kernel("prefill_attention", [list(q.shape), list(k.shape), list(v.shape), [S], list(q.shape)])
    args = [Buf(t.data_ptr(), t.numel() * t.element_size()) for t in (q, k, v, starts, o)] + [F32(1 / math.sqrt(dim))]
    t = Timer(gpu, torch)
    mean, best = t.run(lambda: gpu.launch(kern, args), iters)
    flops = 2.0 * 2.0 * prompts * heads * seq * seq * dim / 2.0
    _, tf, kindp = _peaks()
    return {"kernel": "prefill_attention", "prompts": prompts, "seq": seq, "heads": heads, "kv_heads": kv_heads,
            "head_dim": dim, "ms": mean, "ms_min": best, "flops": flops, "tflops": flops / (mean * 1e-3) / 1e12,
            "peak_tflops": tf, "frac_tensor": flops / (mean * 1e-3) / 1e12 / tf, "peak_kind": kindp}


def qkv_rope(gpu, torch, m=256, k=4096, heads=32, kv_heads=8, dim=128, iters=20, seed=0):
    """The QKV projection with rope_q and kv_write as its epilogue (`linear_rope_kv`) at a decode
    shape, tile chosen by `tb200_tune` unless TB200_GEMM_PLAN forces one; beside it the two-kernel
    form (`linear` + `rope_kv`) on the same inputs."""
    from .gpu import Buf
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    npos, ns = 2304, 4096
    wd = (heads + 2 * kv_heads) * dim
    x = torch.empty((m, k), dtype=torch.float16, device="cuda").normal_(generator=gen)
    w = torch.empty((wd, k), dtype=torch.float16, device="cuda").normal_(0, 0.02, generator=gen)
    pos = (torch.arange(m, dtype=torch.int32, device="cuda") * 7) % npos
    slot = torch.randperm(ns, device="cuda")[:m].to(torch.int32)
    c, s_ = torch.rand((npos, dim // 2), device="cuda"), torch.rand((npos, dim // 2), device="cuda")
    h = lambda *shape: torch.zeros(shape, dtype=torch.float16, device="cuda")
    qkv, q, kc, vc, kd, vd = h(m, wd), h(m, heads, dim), h(ns, kv_heads, dim), h(ns, kv_heads, dim), \
        h(m, kv_heads, dim), h(m, kv_heads, dim)
    buf = lambda t: Buf(t.data_ptr(), t.numel() * t.element_size())
    fused = [x, w, pos, slot, c, s_, qkv, q, kc, vc, kd, vd]
    kf = gpu.kernel("linear_rope_kv", [list(a.shape) for a in fused])
    kl = gpu.kernel("linear", [[m, k], [wd, k], [m, wd]])
    rope = [qkv, pos, slot, c, s_, q, kc, vc, kd, vd]
    kr = gpu.kernel("rope_kv", [list(a.shape) for a in rope])
    fa, la, ra = [buf(a) for a in fused], [buf(x), buf(w), buf(qkv)], [buf(a) for a in rope]
    plan_f, _ = gpu.tune(kf, fa)
    plan_l, _ = gpu.tune(kl, la)
    t = Timer(gpu, torch)
    f_ms, _ = t.run(lambda: gpu.launch(kf, fa), iters)
    l_ms, _ = t.run(lambda: gpu.launch(kl, la), iters)
    r_ms, _ = t.run(lambda: gpu.launch(kr, ra), iters)
    return {"kernel": "linear_rope_kv", "m": m, "k": k, "heads": heads, "kv_heads": kv_heads, "head_dim": dim,
            "fused_us": f_ms * 1e3, "fused_plan": list(plan_f), "linear_us": l_ms * 1e3, "linear_plan": list(plan_l),
            "rope_kv_us": r_ms * 1e3}


def exchange_timeline(gpu, trace, grid):
    """The stamps a trace build of the exchange kernel left in the table's trace buffer
    (tessel_b200/build.py --trace): for the last two calls, thread 0 of each CTA at kernel start
    (the projection before it on the stream is complete), when the partials of its first row
    have all landed, when its rows are summed, normalised and sent, and when the other owners'
    rows have landed. Returns microseconds: medians over the CTAs per phase, the span of the
    whole launch, and the time from the end of the previous call to the start of the last (the
    projection between them), or None when the library is not a trace build."""
    words = gpu.fetch(trace, np.uint32, (trace.bytes // 4,))
    tail = words[64:].view(np.uint64).reshape(2, 64, 4)[:, :min(grid, 64)]
    if not tail.all():
        return None
    last = int(tail[1, 0, 0] > tail[0, 0, 0])
    cur, prev = tail[last].astype(np.int64), tail[1 - last].astype(np.int64)
    us = lambda a: float(np.median(a)) / 1e3
    return {"partials_landed_us": us(cur[:, 1] - cur[:, 0]), "sum_norm_send_us": us(cur[:, 2] - cur[:, 1]),
            "gather_us": us(cur[:, 3] - cur[:, 2]), "launch_span_us": float(cur[:, 3].max() - cur[:, 0].min()) / 1e3,
            "projection_between_calls_us": float(cur[:, 0].min() - prev[:, 3].max()) / 1e3, "ctas": int(cur.shape[0])}


def exchange(torch, tokens=256, dim=4096, k_cols=4096, calls=64, reps=10):
    """Per-call device time of the tensor-parallel exchange, replayed as a graph of `calls`
    projection + exchange pairs (what a decode step does `2 x layers` times): the peer-memory
    form (`linear_scatter` + `tp_reduce_norm`) and the NCCL form (`linear_f32` + allreduce +
    `residual_add` + `rmsnorm`), each rank projecting `k_cols / N` input columns onto `dim`
    outputs. Launch under torchrun, one rank per GPU; rank 0 returns the result, the others None."""
    import torch.distributed as dist
    from .gpu import Buf, F32, Gpu, I32
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group(backend="gloo", rank=rank, world_size=world)
    gpu = Gpu(local)
    ids = [gpu.comm_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    gpu.comm_init(rank, world, ids[0])
    T, kl = tokens, k_cols // world
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1 + rank)
    xin = torch.empty((T, kl), dtype=torch.float16, device="cuda").normal_(generator=gen)
    wt = torch.empty((dim, kl), dtype=torch.float16, device="cuda").normal_(0, 0.02, generator=gen)
    gain = torch.ones((dim,), dtype=torch.float16, device="cuda")
    tbuf = lambda t: Buf(t.data_ptr(), t.numel() * t.element_size())
    a = gpu.alloc
    x, h, trace = a(T * dim * 4), a(T * dim * 2), a(gpu.tp_sizes()[1])
    mine = [a((T + world) * dim * 4), a((T + world) * dim * 4), a(T * dim * 4)]  # two inboxes, the landing area
    for b in mine:
        gpu.fill(b, 0xFF)
    gpu.sync()
    everyone = [None] * world
    dist.all_gather_object(everyone, [gpu.ipc_export(b) for b in mine])
    cols = [[b if r == rank else gpu.ipc_import(everyone[r][i], b.bytes) for r in range(world)]
            for i, b in enumerate(mine)]
    table = gpu.tensor(np.frombuffer(gpu.tp_table(rank, world, cols[0], cols[1], cols[2], x, h, trace), np.uint8).copy())
    # The tile candidates are timed against a stand-in table (every inbox a local buffer), so that
    # the real inboxes stay empty.
    stand_in = [a((T + world) * dim * 4)] * world
    tune_table = gpu.tensor(np.frombuffer(gpu.tp_table(rank, world, stand_in, stand_in, stand_in, x, h), np.uint8).copy())
    part = a(T * dim * 4)
    ks = gpu.kernel("linear_scatter", [[T, kl], [dim, kl], [table.bytes]])
    kt = gpu.kernel("tp_reduce_norm", [[table.bytes], [dim], [T, dim]])
    kf = gpu.kernel("linear_f32", [[T, kl], [dim, kl], [T, dim]])
    kr = gpu.kernel("residual_add", [[T, dim], [T, dim]])
    kn = gpu.kernel("rmsnorm", [[T, dim], [dim], [T, dim]])
    gpu.tune(ks, [tbuf(xin), tbuf(wt), tune_table, I32(0)])
    gpu.tune(kf, [tbuf(xin), tbuf(wt), part])
    eps = F32(1e-5)

    def peer(n):
        for i in range(n):
            gpu.launch(ks, [tbuf(xin), tbuf(wt), table, I32(i & 1)])
            gpu.launch(kt, [table, tbuf(gain), x, eps, I32(i & 1), I32(1), I32(world)])

    def nccl(n):
        for _ in range(n):
            gpu.launch(kf, [tbuf(xin), tbuf(wt), part])
            gpu.allreduce(part, T * dim, 0)
            gpu.launch(kr, [x, part])
            gpu.launch(kn, [x, tbuf(gain), h, eps])

    out = {"kernel": "tp_exchange", "ranks": world, "tokens": T, "dim": dim, "k_per_rank": kl, "calls_per_graph": calls}
    for name, fn in (("peer_memory", peer), ("nccl", nccl)):
        fn(4)
        gpu.sync()
        dist.barrier()
        gpu.capture_begin()
        fn(calls)
        g = gpu.capture_end()
        for _ in range(3):
            gpu.replay(g)
        gpu.sync()
        dist.barrier()
        gpu.time_begin()
        for _ in range(reps):
            gpu.replay(g)
        ms = gpu.time_end()
        gpu.sync()
        t = torch.tensor([ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[name + "_us_per_pair"] = float(t[0]) / (reps * calls) * 1e3
        if name == "peer_memory":
            lines = [None] * world
            dist.all_gather_object(lines, exchange_timeline(gpu, trace, -(-T // world)))
            if lines[0] is not None:
                out["timeline_by_rank"] = lines
    # The projection alone, for the difference.
    gpu.capture_begin()
    for _ in range(calls):
        gpu.launch(kf, [tbuf(xin), tbuf(wt), part])
    g = gpu.capture_end()
    gpu.replay(g)
    gpu.sync()
    gpu.time_begin()
    for _ in range(reps):
        gpu.replay(g)
    out["linear_f32_alone_us"] = gpu.time_end() / (reps * calls) * 1e3
    gpu.sync()
    dist.barrier()
    dist.destroy_process_group()
    return out if rank == 0 else None


def chunked(gpu, torch, prompt=4096, chunk=512, layers=32, seed=0):
    """Prefill of one `prompt`-token prompt on a `layers`-layer Llama-3-8B-shaped model: in one
    step, and fed `chunk` tokens at a time through the mixed steps (chunk_attention over the paged
    cache). Wall-clock tokens/s of each, after a warm-up run of the same thing."""
    import time
    from .engine import Engine, Limits
    from .model import Config
    from .sched import Request, generate_with
    from .synth import device_weights
    cfg = Config.llama3_8b(max_pos=prompt + 64)
    cfg = Config(**{**cfg.__dict__, "layers": layers, "vocab": 16032})
    w = device_weights(cfg, 0, 1, torch)
    g = np.random.default_rng(seed)
    toks = g.integers(0, cfg.vocab, prompt).tolist()
    pages = -(-(prompt + 8) // 16) + 4
    out = {"kernel": "chunked_prefill", "prompt": prompt, "chunk": chunk, "layers": layers}
    for name, max_tokens, ch in (("one_step", prompt, 0), ("chunked", chunk, chunk)):
        e = Engine(gpu, w, Limits(page=16, pages=pages, max_tokens=max_tokens, max_seq_pages=pages), sharded=True)
        best = None
        for _ in range(3):
            gpu.sync()
            t0 = time.perf_counter()
            outs, st = generate_with(e, [Request(toks, 1)], 1, True, device_argmax=True, chunk=ch)
            gpu.sync()
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        out[name] = {"seconds": best, "tok_s": prompt / best, "first_token": int(outs[0].tokens[0])}
    out["chunked_over_one_step"] = out["chunked"]["tok_s"] / out["one_step"]["tok_s"]
    out["same_first_token"] = out["chunked"]["first_token"] == out["one_step"]["first_token"]
    return out


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    d = sub.add_parser("decode")
    for name, default in (("seqs", 256), ("ctx-lo", 512), ("ctx-hi", 2304), ("heads", 32), ("kv-heads", 8),
                          ("dim", 128), ("iters", 20)):
        d.add_argument("--" + name, type=int, default=default)
    gm = sub.add_parser("gemm")
    for name, default in (("m", 4096), ("n", 4096), ("k", 4096), ("iters", 20)):
        gm.add_argument("--" + name, type=int, default=default)
    gm.add_argument("--kind", default="matmul")
    f = sub.add_parser("flash")
    for name, default in (("heads", 256), ("seq", 4096), ("dim", 128), ("iters", 10)):
        f.add_argument("--" + name, type=int, default=default)
    f.add_argument("--packed", action="store_true",
                   help="the packed prefill form: --prompts prompts of --seq tokens, --heads query heads on --kv-heads")
    f.add_argument("--prompts", type=int, default=8)
    f.add_argument("--kv-heads", type=int, default=0)
    ex = sub.add_parser("exchange", help="under torchrun: python -m torch.distributed.run --nproc-per-node N -m tessel_b200.microbench exchange")
    for name, default in (("tokens", 256), ("dim", 4096), ("k-cols", 4096), ("calls", 64)):
        ex.add_argument("--" + name, type=int, default=default)
    qk = sub.add_parser("qkv")
    for name, default in (("m", 256), ("k", 4096), ("heads", 32), ("kv-heads", 8), ("dim", 128), ("iters", 20)):
        qk.add_argument("--" + name, type=int, default=default)
    ck = sub.add_parser("chunked")
    for name, default in (("prompt", 4096), ("chunk", 512), ("layers", 32)):
        ck.add_argument("--" + name, type=int, default=default)
    a = ap.parse_args()
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("microbench needs a B200: there is no CPU path")
    if a.cmd == "exchange":
        r = exchange(torch, a.tokens, a.dim, a.k_cols, a.calls)
        if r is not None:
            print(json.dumps(r), flush=True)
        return
    from .gpu import Gpu
    gpu = Gpu(0)
    if a.cmd == "decode":
        r = decode(gpu, torch, a.seqs, a.ctx_lo, a.ctx_hi, a.heads, a.kv_heads, a.dim, a.iters)
    elif a.cmd == "gemm":
        r = gemm(gpu, torch, a.m, a.n, a.k, a.kind, a.iters)
    elif a.cmd == "qkv":
        r = qkv_rope(gpu, torch, a.m, a.k, a.heads, a.kv_heads, a.dim, a.iters)
    elif a.cmd == "chunked":
        r = chunked(gpu, torch, a.prompt, a.chunk, a.layers)
    elif a.packed:
        heads = 32 if a.heads == 256 else a.heads
        r = flash_packed(gpu, torch, a.prompts, a.seq, heads, a.kv_heads or heads, a.dim, a.iters)
    else:
        r = flash(gpu, torch, a.heads, a.seq, a.dim, a.iters)
    print(json.dumps(r), flush=True)


if __name__ == "__main__":
    main()
