"""Decode throughput of the Llama-3-8B-shaped engine (benchmark configuration 5) on N B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A "step" is one decode step of the whole batch: 256 sequences (prompts of 512-2048 uniform
random token ids, random-init f16 weights ~N(0, 0.02)), one new token each, greedy. The
prompts are prefilled through the engine first (untimed), then W warm-up decode steps, then

  * `e2e`:   K decode steps through `Engine.step_greedy` with HOST inputs: each step uploads
             the step's tokens, positions, slots, block tables and lengths from page-locked
             memory and reads the picked tokens back;
  * `value`: K decode steps with everything resident on the device (`Engine.decode_resident`:
             a small kernel derives the next step's inputs from the picks, the recorded step
             is replayed).

Both are timed with CUDA events on the stream the kernels run on, between synchronisations,
and the maximum over ranks is taken. With N > 1 the model is tensor-parallel over the N GPUs
(attention/KV heads and MLP columns sharded; the cross-rank sum after o_proj and after
down_proj by the fused peer-memory kernel, or by one NCCL allreduce each with
`--tp-exchange nccl`), so the job is the same 256 sequences: strong scaling.

With N > 1 the line also carries `tp_check` (a small fixed-seed model run at TP N, with both
exchanges, against the same model at TP 1 on rank 0's GPU: logits, greedy tokens, KV pages, and
whether every rank holds the same bits of x and h) and `nccl_exchange` (the same device-resident
step timed with the NCCL exchange when the fused one is the default, and the other way round).

`--impl reference` times the CPU restatement of the reference's interpreter path (the
oracle; the reference itself is Rust and cannot be built on these machines) on the host
cores; each of its steps is the same bounded sample of the decode step that the `cpu_baseline`
of the default arm times once.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode_tokens_per_s"
UNIT = "tok/s"
# DRAM bytes moved per algorithmic byte by the decode-attention kernel, from a profiler capture
# (dram__bytes_read + dram__bytes_write) of ONE launch of the same one-split form on a batch that
# fits the profiler's size rule: 256 sequences at contexts U[256, 768] (2048 CTAs, 0.55 GB):
# 558.32 MB read and 4.73 MB written for 552.52 MB of algorithmic bytes. Traffic grows in
# proportion to the KV bytes read, so the ratio carries to the benchmark's launch.
DRAM_PER_ALGORITHMIC_BYTE = (558.32 + 4.73) / 552.52


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama3-8b", choices=["llama3-8b", "tinyllama"])
    ap.add_argument("--seqs", type=int, default=0, help="sequences (default: the workload's)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-micro", action="store_true", help="skip the single-kernel numbers (N = 1)")
    ap.add_argument("--profile-steps", type=int, default=2)
    ap.add_argument("--fp8", action="store_true",
                    help="N = 1: the NON-PARITY FP8 mode (E4M3 projections); the line says so in `dtype` "
                         "and is not the headline number")
    ap.add_argument("--profiler-range", action="store_true",
                    help="bracket the device-resident timed region with cudaProfilerStart/Stop "
                         "(for `ncu --profile-from-start off`)")
    ap.add_argument("--tp-exchange", default="fused", choices=["fused", "nccl"],
                    help="N > 1: cross-rank sums by the fused peer-memory kernel, or by NCCL allreduce")
    return ap.parse_args()


def workload(name: str):
    from tessel_b200.model import Config
    if name == "llama3-8b":
        return dict(cfg=Config.llama3_8b(max_pos=2304), seqs=256, lo=512, hi=2048, new=256,
                    label="Llama-3-8B shape, 256 seqs, prompts U[512,2048], 256 new tokens, page 16")
    return dict(cfg=Config.tinyllama(max_pos=1152), seqs=64, lo=128, hi=1024, new=128,
                label="TinyLlama-1.1B shape, 64 seqs, prompts U[128,1024], 128 new tokens, page 16")


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        j = json.load(open(p))
        return dict(hbm=float(j["hbm_gbs"]), tflops=float(j["bf16_tflops"]), kind="measured")
    return dict(hbm=6650.0, tflops=1590.0, kind="fallback")


class Clocks:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                       "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.f,
                                      stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.p.terminate()
        self.p.wait()
        self.f.flush()
        rows = [l.strip().split(", ") for l in open(self.f.name) if l.strip()]
        os.unlink(self.f.name)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[4:8]):
                if v.strip().lower() == "active":
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---- the CPU arm: the oracle on the host cores -----------------------------------------------
class CpuSample:
    """One layer and 1/head_div of the LM head of a decode step for `rows` sequences on the
    oracle; `run()` times it and scales to the whole step (all layers, whole head, all
    sequences). Inputs are generated once."""

    def __init__(self, cfg, ctx, rows: int, head_div: int = 8):
        import oracle
        self.o = oracle
        g = np.random.default_rng(0)
        h = np.float16
        self.cfg, self.rows, self.head_div, self.nseq = cfg, rows, head_div, len(ctx)
        dm, H, G, D, F, V = cfg.dim, cfg.heads, cfg.kv_heads, cfg.head_dim, cfg.ffn, cfg.vocab
        W = (H + 2 * G) * D
        P = 16

        def m(r, c):
            return (g.standard_normal((r, c), dtype=np.float32) * np.float32(0.02)).astype(h)

        self.wqkv, self.wo, self.wg, self.wu, self.wd = m(W, dm), m(dm, H * D), m(F, dm), m(F, dm), m(dm, F)
        self.head = m(V // head_div, dm)
        self.one = np.ones(dm, h)
        self.lens = np.asarray(ctx[:rows], np.int32) + 1
        pages = [-(-int(l) // P) for l in self.lens]
        NP = sum(pages) + 1
        self.kc = g.standard_normal((NP * P, G, D), dtype=np.float32).astype(h)
        self.vc = g.standard_normal((NP * P, G, D), dtype=np.float32).astype(h)
        self.NP, self.P = NP, P
        self.table = np.zeros((rows, max(pages)), np.int32)
        at = 0
        for b, n in enumerate(pages):
            self.table[b, :n] = np.arange(at, at + n)
            at += n
        self.x = g.standard_normal((rows, dm), dtype=np.float32)
        self.pos = (self.lens - 1).astype(np.int32)
        self.slot = np.asarray([self.table[b, self.pos[b] // P] * P + self.pos[b] % P for b in range(rows)], np.int32)
        self.Ct, self.St = oracle.rope_tables(cfg.max_pos, D, cfg.rope_theta)

    def run(self, layers: int = 1):
        """Returns (seconds for the sample, extrapolated seconds per full step). ``layers``: how
        many decoder layers the sample runs (the same weights each time, the activations fed on)."""
        o, cfg, rows = self.o, self.cfg, self.rows
        H, G, D, NP, P = cfg.heads, cfg.kv_heads, cfg.head_dim, self.NP, self.P
        t0 = time.perf_counter()
        x = self.x
        for _ in range(layers):
            hh = o.rmsnorm(x, self.one, cfg.eps)
            qkv = o.linear(hh, self.wqkv)
            q = o.rope_q(qkv, self.pos, self.Ct, self.St, H, D)
            kc2, vc2, _, _ = o.kv_write(qkv, self.pos, self.slot, self.Ct, self.St, self.kc, self.vc, G, D)
            att = o.decode_attention(q, kc2.reshape(NP, P, G, D), vc2.reshape(NP, P, G, D), self.table, self.lens,
                                     1.0 / math.sqrt(D))
            x = o.linear_residual(att.reshape(rows, H * D), self.wo, x)
            hh = o.rmsnorm(x, self.one, cfg.eps)
            mlp = o.gate_up(hh, self.wg, self.wu)
            x = o.linear_residual(mlp, self.wd, x)
        t_layer = (time.perf_counter() - t0) / layers
        t0 = time.perf_counter()
        last = o.rmsnorm_rows(x, np.arange(rows, dtype=np.int32), self.one, cfg.eps)
        lg = o.logits(last, self.head)
        [o.argmax(r) for r in lg]
        t_head = time.perf_counter() - t0
        return t_layer * layers + t_head, (t_layer * cfg.layers + t_head * self.head_div) * (self.nseq / rows)


def prompt_lengths(wl, seqs):
    """The batch's prompt lengths: one seeded draw, shared by both arms."""
    return np.random.default_rng(1).integers(wl["lo"], wl["hi"] + 1, seqs)


def timed_contexts(plens, K, Wm):
    """Cached tokens per sequence when the device-resident timed region starts: the prompt, the
    warm-up steps, the three end-to-end regions of K steps, and the three steps that set the
    resident loop up."""
    return np.asarray(plens, np.int64) + max(Wm, 3) + E2E_REPEATS * K + 3


def config_of(args, wl, world, seqs, plens):
    """The `config` object of the JSON line; both arms print the same one."""
    cfg = wl["cfg"]
    K, Wm = args.steps, args.warmup
    ctx_mid = float(np.mean(timed_contexts(plens, K, Wm))) + K / 2.0
    Hl, Gl, Fl, D = cfg.heads // world, cfg.kv_heads // world, cfg.ffn // world, cfg.head_dim
    vocab_parallel = world > 1 and cfg.vocab % world == 0 and cfg.vocab <= 1 << 24
    head_rows = cfg.vocab // world if vocab_parallel else cfg.vocab
    layer_w = cfg.layers * ((Hl + 2 * Gl) * D * cfg.dim + cfg.dim * Hl * D + 3 * Fl * cfg.dim)
    wbytes = (1.0 if getattr(args, "fp8", False) else 2.0) * layer_w + 2.0 * head_rows * cfg.dim
    kvbytes = 4.0 * Gl * D * cfg.layers * ctx_mid * seqs
    par = f"tp{world}" + (f" ({args.tp_exchange} exchange)" if world > 1 else "")
    return ({"workload": wl["label"], "sequences": int(seqs), "parallelism": par,
             "l2": "inputs larger than L2 (weights + KV read per step: %.1f GB per GPU)" % ((wbytes + kvbytes) / 1e9),
             "mean_context": ctx_mid}, wbytes, kvbytes)


E2E_REPEATS = 3
CPU_ROWS, CPU_LAYERS = 128, 4


def cpu_sample_for(cfg, ctx, budget_s=None):
    """The bounded CPU sample both arms time: CPU_LAYERS decoder layers and 1/8 of the LM head
    for CPU_ROWS sequences. With a time budget per step, layers and then rows are halved until
    one run fits it. Returns (sample, layers)."""
    rows, nl = min(len(ctx), CPU_ROWS), min(cfg.layers, CPU_LAYERS)
    smp = CpuSample(cfg, ctx, rows)
    if budget_s is None:
        return smp, nl
    t, _ = smp.run(1)
    est = lambda: t * nl  # one layer dominates; the head slice is a small part
    while est() > budget_s and nl > 1:
        nl //= 2
    while est() > budget_s and rows > 8:
        rows //= 2
        smp = CpuSample(cfg, ctx, rows)
        t, _ = smp.run(1)
    return smp, nl


def run_reference(args, wl):
    """The reference arm: rank 0 times the oracle; other ranks leave."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import oracle
    cfg = wl["cfg"]
    seqs = args.seqs or wl["seqs"]
    world = args.gpus
    plens = prompt_lengths(wl, seqs)
    config, _, _ = config_of(args, wl, world, seqs, plens)
    ctx = timed_contexts(plens, args.steps, args.warmup).tolist()
    # Every step is one run of the sample; K + W of them must end within a few minutes.
    total = args.steps + args.warmup
    smp, nl = cpu_sample_for(cfg, ctx, budget_s=170.0 / max(total, 1))
    for _ in range(args.warmup):
        smp.run(nl)
    measured, full = [], []
    t0 = time.perf_counter()
    for _ in range(args.steps):
        a, b = smp.run(nl)
        measured.append(a)
        full.append(b)
    wall = time.perf_counter() - t0
    sec = statistics.mean(full)
    val = seqs / sec
    sample = (f"per step: {nl} of {cfg.layers} layers and 1/8 of the LM head for {smp.rows} of {seqs} sequences at "
              f"the contexts of the timed region, scaled to the whole decode step; {args.steps} steps measured, "
              f"{wall / max(args.steps, 1):.2f} s of CPU work each")
    line = {"metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": statistics.mean(measured) * 1e3,
            "ms_per_whole_step_extrapolated": sec * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic", "impl": "reference", "config": config,
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": oracle.threads(), "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---- our arm ---------------------------------------------------------------------------------
def tp_check(gpu, rank, world, dist):
    """A small fixed-seed model at TP `world`, with the fused exchange and with NCCL, against the
    same model at TP 1 on rank 0's GPU (tessel_b200/tpcheck.py). Returns the summaries on rank 0."""
    from tessel_b200 import tpcheck

    def gather(x):
        out = [None] * world
        dist.all_gather_object(out, x)
        return out

    res = {}
    one = tpcheck.run(gpu, 0, 1) if rank == 0 else None
    for name, exchange in (("fused", gather), ("nccl", None)):
        mine = tpcheck.run(gpu, rank, world, exchange)
        shards = gather({k: mine[k] for k in ("kc", "vc")} if rank else mine)
        digests = gather(tpcheck.digest(mine))
        if rank == 0:
            res[name] = tpcheck.summary(one, shards, digests)
    return res


def run_ours(args, wl):
    import torch
    import torch.distributed as dist
    from tessel_b200.engine import Engine, Limits, padded
    from tessel_b200.gpu import Gpu
    from tessel_b200.sched import Request, Scheduler

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch with torch.distributed.run")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: there is no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group(backend="gloo", rank=rank, world_size=world)

    def barrier():
        if world > 1:
            dist.barrier()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    cfg = wl["cfg"]
    seqs = args.seqs or wl["seqs"]
    K, Wm = args.steps, args.warmup
    # Decode steps this run needs from every sequence: warm-up, the timed regions, profiling.
    need_new = max(wl["new"], max(Wm, 3) + (E2E_REPEATS + 2) * K + args.profile_steps + 16)
    P = 16
    max_prompt = wl["hi"]
    cfg.max_pos = max(cfg.max_pos, max_prompt + need_new)
    msp = -(-(max_prompt + need_new) // P)
    if cfg.heads % world or cfg.kv_heads % world or cfg.ffn % world:
        raise SystemExit(f"{world} ranks do not divide heads/kv_heads/ffn")
    plens = prompt_lengths(wl, seqs)
    g = np.random.default_rng(2)
    reqs = [Request(g.integers(0, cfg.vocab, int(n)).tolist(), need_new) for n in plens]
    pages = int(sum(-(-(int(n) + need_new) // P) for n in plens)) + 8
    config, wbytes, kvbytes = config_of(args, wl, world, seqs, plens)

    gpu = Gpu(local_rank)
    tpc = None
    if world > 1:
        ids = [gpu.comm_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        gpu.comm_init(rank, world, ids[0])
        tpc = tp_check(gpu, rank, world, dist)
    from tessel_b200.synth import device_weights
    w = device_weights(cfg, rank, world, torch)
    local = w.cfg
    exchange = None
    if world > 1:
        # The peer-memory exchange is always set up; `--tp-exchange nccl` merely does not use it
        # for the headline number (the other mode is timed beside it).
        def exchange(mine):
            everyone = [None] * world
            dist.all_gather_object(everyone, mine)
            return everyone
    if args.fp8 and world > 1:
        raise SystemExit("--fp8 runs on one GPU")
    e = Engine(gpu, w, Limits(page=P, pages=pages, max_tokens=max_prompt, max_seq_pages=msp), rank=rank,
               nranks=world, sharded=True, exchange=exchange, fp8=args.fp8)
    e.fused = world > 1 and args.tp_exchange == "fused"
    s = Scheduler(e, reqs, seqs, packed=True, device_argmax=True)

    # ---- prefill (untimed for the metric; reported for information) ---------------------------
    t0 = time.perf_counter()
    while s.waiting:
        if s.step() != "prefill":
            raise SystemExit("the cache cannot hold the whole batch")
    gpu.sync()
    prefill_s = time.perf_counter() - t0
    n = len(s.running)
    t = padded(n)

    for _ in range(max(Wm, 3)):
        s.step()
    gpu.sync()

    clocks = Clocks(local_rank)
    # ---- e2e: host inputs every step; E2E_REPEATS regions of K steps ----------------------------
    launches0 = gpu.kernel_launches()
    clocks.start()
    e2e_all = []
    for _ in range(E2E_REPEATS):
        barrier()
        gpu.sync()
        gpu.time_begin()
        for _ in range(K):
            s.step()
        ms = gpu.time_end()
        gpu.sync()
        barrier()
        e2e_all.append(max_over_ranks(ms))
    e2e_ms = statistics.median(e2e_all)
    e2e_launches = (gpu.kernel_launches() - launches0) // E2E_REPEATS

    # ---- value: device-resident steps ---------------------------------------------------------
    def resident(steps):
        """`steps` device-resident decode steps between barriers; device ms, max over ranks."""
        barrier()
        gpu.sync()
        gpu.time_begin()
        picks = e.decode_resident(n, steps)
        ms = gpu.time_end()
        gpu.sync()
        barrier()
        for row in picks:
            s.absorb(row)
        return max_over_ranks(ms)

    toks, pos, slots, attn, want = s.decode_inputs()
    s.absorb(e.step_greedy(toks, pos, slots, attn, want))  # uploads the tables the resident loop walks
    for _ in range(2):
        s.absorb(e.decode_resident(n, 1)[0])
    ctx0 = [q.len for q in s.running]
    if ctx0 != timed_contexts(plens, K, Wm).tolist():
        # Not expected (no sequence ends inside this run); state what was measured.
        config["mean_context"] = float(np.mean(ctx0)) + K / 2.0
        kvbytes = 4.0 * local.kv_heads * cfg.head_dim * cfg.layers * config["mean_context"] * n
        config["l2"] = "inputs larger than L2 (weights + KV read per step: %.1f GB per GPU)" % ((wbytes + kvbytes) / 1e9)
    launches0 = gpu.kernel_launches()
    launches_before = launches0  # kernels launched before the device-resident timed region (a profiler's skip count)
    if args.profiler_range:
        torch.cuda.cudart().cudaProfilerStart()
    dev_ms = resident(K)
    if args.profiler_range:
        torch.cuda.cudart().cudaProfilerStop()
    clock_rec = clocks.stop()
    dev_launches = gpu.kernel_launches() - launches0
    ctx_mid = config["mean_context"]

    # ---- the other exchange, same device-resident step (N > 1) -----------------------------------
    other = None
    if world > 1:
        e.fused = not e.fused
        resident(3)  # records this mode's graph
        other = {"exchange": "fused" if e.fused else "nccl", "ms_per_step": resident(K) / K}
        other["value"] = n / (other["ms_per_step"] * 1e-3)
        e.fused = not e.fused
        resident(1)

    # ---- per-kernel times: the same step, every launch timed on its own (graphs off) ------------
    gpu.profile = {}
    ctx_prof = [q.len + 1 for q in s.running]
    for _ in range(args.profile_steps):
        s.step()
    prof = gpu.profile_rows()
    gpu.profile = None
    total_prof = sum(r[3] for r in prof) or 1.0
    att = [r for r in prof if r[1].startswith("decode_attention")]
    pk = peaks()
    lyr = cfg.layers
    Gl, D, Hl = local.kv_heads, cfg.head_dim, local.heads
    sum_ctx = float(sum(ctx_prof)) + (args.profile_steps - 1) * n / 2.0
    att_bytes = 4.0 * Gl * D * sum_ctx + 4.0 * n * Hl * D + 4.0 * sum(-(-c // P) for c in ctx_prof) + 4.0 * n
    roof = None
    if att:
        att_ms = att[0][3] / att[0][2]
        achieved = att_bytes / (att_ms * 1e-3) / 1e9
        roof = {"kernel": "decode_attention", "bound": "hbm", "achieved": achieved, "peak": pk["hbm"], "unit": "GB/s",
                "frac": achieved / pk["hbm"], "peak_kind": pk["kind"], "traffic": att_bytes * DRAM_PER_ALGORITHMIC_BYTE,
                "algorithmic_bytes_per_launch": att_bytes, "ms_per_launch": att_ms,
                "share_of_step": att[0][3] / total_prof}
    # Whole-step HBM roofline (weights once, KV once per KV head), per GPU.
    step_bytes = wbytes + kvbytes
    dev_step_ms = dev_ms / K
    step_roof = {"bytes_per_step_per_gpu": step_bytes, "weights_bytes": wbytes, "kv_bytes": kvbytes,
                 "achieved_gbs": step_bytes / (dev_step_ms * 1e-3) / 1e9, "peak_gbs": pk["hbm"],
                 "frac": step_bytes / (dev_step_ms * 1e-3) / 1e9 / pk["hbm"], "mean_context": ctx_mid}

    if rank != 0:
        barrier()
        return
    value = n * K / (dev_ms * 1e-3)
    mp = msp
    h2d = 4 * (3 * t + t + t + t * mp)  # tok, pos, slot, idx, lens, table
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": max(Wm, 3),
        "ms_per_step": dev_step_ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f8e4m3 projections, f16 elsewhere (non-parity mode)" if args.fp8 else "f16", "data": "synthetic",
        "config": config,
        "e2e": {"value": n * K / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * n,
                "ms_per_step": e2e_ms / K, "ms_per_step_min": min(e2e_all) / K, "ms_per_step_max": max(e2e_all) / K,
                "repeats": E2E_REPEATS, "value_is": "median of the repeats"},
        "gpu_launches": int(dev_launches), "e2e_gpu_launches": int(e2e_launches),
        "launches_before_timed_region": int(launches_before),
        "clocks": clock_rec,
        "roofline": roof, "step_roofline": step_roof,
        "kernel_shares": [{"kernel": r[1], "launches": r[2], "ms": round(r[3], 3), "share": round(r[3] / total_prof, 4)}
                          for r in prof[:12]],
        "prefill": {"seconds": prefill_s, "prompt_tokens": int(s.st.prompt_tokens),
                    "tok_s": s.st.prompt_tokens / prefill_s, "steps": s.st.prefill_steps},
    }
    if tpc is not None:
        line["tp_check"] = tpc[args.tp_exchange]
        line["tp_check_" + ("nccl" if args.tp_exchange == "fused" else "fused")] = tpc["nccl" if args.tp_exchange == "fused" else "fused"]
    if other is not None:
        line[other["exchange"] + "_exchange"] = other
    if world == 1 and not args.no_micro:
        # The two other headline numbers of the path (and the prefill attention), same process:
        # single kernels at the benchmark configurations' shapes, CUDA events per launch, L2 flushed in between.
        from tessel_b200 import microbench as mb
        d = mb.decode(gpu, torch, iters=10)
        gm = mb.gemm(gpu, torch, 4096, 4096, 4096, "matmul", iters=10)
        fl = mb.flash(gpu, torch, 256, 4096, 128, iters=5)
        gpu.set_stream(None)
        line["micro"] = {
            "paged_decode_attention": {"gbs": d["gbs"], "frac_of_hbm_peak": d["frac"], "ms": d["ms"],
                                       "shape": "256 seqs, ctx U[512,2304], 32 heads / 8 kv heads, D 128, page 16"},
            "gemm_4096": {"tflops": gm["tflops"], "frac_of_tensor_peak": gm["frac_tensor"], "ms": gm["ms"],
                          "shape": "f16 4096^3, row-major A and B, f32 accumulate"},
            "flash_attention": {"tflops": fl["tflops"], "frac_of_tensor_peak": fl["frac_tensor"], "ms": fl["ms"],
                                "shape": "causal, batch 8 x 32 heads, S 4096, D 128"},
            "peak_kind": pk["kind"]}
    if world == 1 and not args.no_cpu_baseline:
        import oracle
        # One run of the sample the reference arm times per step, at the timed region's contexts.
        smp, nl = cpu_sample_for(cfg, ctx0)
        sample_s, full_s = smp.run(nl)
        line["cpu_baseline"] = {
            "value": n / full_s, "unit": UNIT, "cores": oracle.threads(), "kind": "port",
            "sample": (f"{nl} of {cfg.layers} layers and 1/8 of the LM head for {smp.rows} of {n} sequences at the "
                       f"contexts of the timed region, scaled to the whole decode step; {sample_s:.1f} s of CPU work")}
    print(json.dumps(line), flush=True)
    barrier()


def main():
    args = parse()
    wl = workload(args.workload)
    if args.impl == "reference":
        run_reference(args, wl)
    else:
        run_ours(args, wl)


if __name__ == "__main__":
    main()
