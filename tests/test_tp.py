"""Tensor parallelism over 2, 4 and 8 ranks: heads, KV heads and MLP columns sharded, one
cross-rank sum after o_proj and one after down_proj. On the CPU (oracle kernels, gloo) here; on
B200s (library kernels; NCCL, and the fused peer-memory kernel) when that many are present.
An N-rank run must give the 1-rank run's logits within 2e-3, the same greedy tokens for 32
decode steps (up to proven near-ties), KV pages that are the 1-rank pages' slices along the
KV-head axis, and x and h that are the same bits on every rank."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

from tessel_b200 import tpcheck

HERE = os.path.dirname(os.path.abspath(__file__))
TOL = 2e-3


def free_port() -> str:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return str(s.getsockname()[1])


def launch(mode, world, tmp):
    port = free_port()
    outs = [os.path.join(tmp, f"{mode}_{world}_{r}.npz") for r in range(world)]
    env = dict(os.environ)
    if mode == "cpu":
        # Few oracle threads per rank: the ranks of a CPU run share this machine's cores.
        env["ORACLE_THREADS"] = str(max(1, (os.cpu_count() or 8) // world))
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "tp_worker.py"), mode, str(r), str(world), port,
                               outs[r]], env=env) for r in range(world)]
    for p in procs:
        assert p.wait(timeout=900) == 0
    return [dict(np.load(o)) for o in outs]


def same_tokens_up_to_near_ties(ta, tb, requests, count):
    """Greedy tokens agree; where two runs part ways, the two choices' logits are a near-tie
    (a different summation order may flip it, as tests/llm.rs:57-78 allows), judged on the f32
    one-sequence model, and the comparison of that sequence ends there."""
    import oracle
    cfg, w = tpcheck.model()
    for r, x, y in zip(requests, ta, tb):
        assert len(x) == len(y) == count
        for i, (u, v) in enumerate(zip(x, y)):
            if u == v:
                continue
            l = oracle.reference_forward(cfg, w, list(r.prompt) + [int(t) for t in x[:i]])[-1]
            assert abs(l[u] - l[v]) < 2e-3 * np.abs(l).max(), f"tokens {u} / {v} are not a near-tie"
            break


def compare(one, many):
    a, b = one[0], many[0]
    assert tpcheck.rel_err(b["pre"], a["pre"]) <= TOL
    assert tpcheck.rel_err(b["dec"], a["dec"]) <= TOL
    cfg, _ = tpcheck.model()
    same_tokens_up_to_near_ties(a["tokens"], b["tokens"], tpcheck.requests(cfg), tpcheck.DECODE_STEPS + 1)
    same_tokens_up_to_near_ties(a["chunk_tokens"], b["chunk_tokens"], tpcheck.chunk_requests(cfg), tpcheck.CHUNK_NEW)
    # Rank r holds KV heads [r G/n, (r+1) G/n): gathered along the KV-head axis they are the 1-rank cache.
    for name in ("kc", "vc"):
        full = a[name].astype(np.float32)
        got = tpcheck.gathered_cache(many, name).astype(np.float32)
        assert got.shape == full.shape
        used = np.abs(full).sum(axis=(1, 2, 3)) > 0
        assert np.array_equal(np.abs(got).sum(axis=(1, 2, 3)) > 0, used), "the same pages are written"
        assert tpcheck.rel_err(got[used], full[used]) <= TOL
    # One owner sums in rank order and everyone copies: the activations are the same bits everywhere.
    assert len({tpcheck.digest(r) for r in many}) == 1, "x and h differ between ranks"
    s = tpcheck.summary(a, many, [tpcheck.digest(r) for r in many])
    assert s["logits_rel_err"] <= TOL and s["h_bit_identical"] and s["same_pages_written"]


_ONE = {}


def single(mode, tmp):
    if mode not in _ONE:
        _ONE[mode] = launch(mode, 1, tmp)
    return _ONE[mode]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ranks_on_cpu(tmp_path, world):
    compare(single("cpu", str(tmp_path)), launch("cpu", world, str(tmp_path)))


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4, 8])
def test_ranks_on_gpus(tmp_path, world):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    one = single("gpu", str(tmp_path))
    compare(one, launch("gpu", world, str(tmp_path)))
    # The same with the sum, the residual add and the RMSNorm fused into one kernel over NVLink.
    compare(one, launch("gpufused", world, str(tmp_path)))
