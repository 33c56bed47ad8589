"""The whole engine on the GPU against the same engine on the CPU stand-in (oracle kernels)
and the f32 one-sequence model: logits within 2e-3 of the largest, greedy tokens identical
for the first 32 steps, block tables and KV pages landing where the scheduler says."""
import numpy as np
import pytest

import oracle
from emu import EmuGpu
from refs import rel_err
from tessel_b200.engine import Decode, Engine, Limits, Prefill
from tessel_b200.model import Config, Weights, argmax
from tessel_b200.sched import Request, generate_with

pytestmark = pytest.mark.gpu
TOL = 2e-3


def small():
    """A model small enough for the CPU oracle, shaped for the tensor-core kernels (head_dim 64)."""
    return Config(dim=256, layers=2, heads=8, kv_heads=2, head_dim=64, ffn=512, vocab=1000, eps=1e-5,
                  rope_theta=10000.0, max_pos=512, bos=1, eos=-1)


def test_tiny_model_like_tests_llm_rs(gpu):
    """tests/llm.rs:25-83 on the GPU (head_dim 16, page 8: the generic attention paths)."""
    cfg = Config.tiny()
    w = Weights.random(cfg, 7)
    e = Engine(gpu, w, Limits(page=8, pages=32, max_tokens=16, max_seq_pages=8))
    prompt = [1, 17, 200, 33, 5, 99, 64, 3, 250, 12]
    n = len(prompt)
    got = e.step(prompt, list(range(n)), list(range(n)), Prefill(), [n - 1]).copy()
    want = oracle.reference_forward(cfg, w, prompt)
    assert rel_err(got[0], want[n - 1]) < 2e-2
    reqs = [Request([1, 5, 9], 6), Request(prompt, 4), Request([1, 100, 101, 102, 103, 104, 105], 9)]
    outs, st = generate_with(e, reqs, 3, True)
    assert st.largest_batch == 3
    for r, o in zip(reqs, outs):
        seq = list(r.prompt)
        for t in o.tokens:
            l = oracle.reference_forward(cfg, w, seq)[-1]
            best = argmax(l)
            assert t == best or l[best] - l[t] < 2e-2 * np.abs(l).max()
            seq.append(t)


def test_engine_matches_cpu_engine(gpu):
    """Same weights, same requests: prefill logits, decode logits, KV pages and 32 greedy tokens."""
    cfg = small()
    w = Weights.random(cfg, 13)
    lim = Limits(page=16, pages=40, max_tokens=128, max_seq_pages=8)
    eg, ec = Engine(gpu, w, lim), Engine(EmuGpu(), w, lim)
    g = np.random.default_rng(1)
    p1, p2 = g.integers(0, cfg.vocab, 37).tolist(), g.integers(0, cfg.vocab, 20).tolist()
    toks = p1 + p2
    pos = list(range(37)) + list(range(20))
    slots = [16 * 3 + i for i in range(37)] + [16 * 9 + i for i in range(20)]  # pages 3,4,5 and 9,10
    from tessel_b200.engine import Packed
    starts = [0] * 37 + [37] * 20
    lg = eg.step(toks, pos, slots, Packed(starts), [36, 56]).copy()
    lc = ec.step(toks, pos, slots, Packed(starts), [36, 56]).copy()
    assert rel_err(lg, lc) <= TOL
    for layer in range(cfg.layers):
        (kg, vg), (kc, vc) = eg.read_cache(layer), ec.read_cache(layer)
        used = np.zeros(lim.pages * lim.page, bool)
        used[slots] = True
        kg, vg, kc, vc = (a.reshape(lim.pages * lim.page, -1) for a in (kg, vg, kc, vc))
        assert not kg[~used].any() and not vg[~used].any(), "only the scheduled slots are written"
        assert rel_err(kg[used], kc[used]) <= TOL and rel_err(vg[used], vc[used]) <= TOL
    # One decode step on both, from the same state.
    t1, t2 = argmax(lc[0]), argmax(lc[1])
    assert (argmax(lg[0]), argmax(lg[1])) == (t1, t2)
    dec = Decode([[3, 4, 5], [9, 10]], [38, 21])
    lg = eg.step([t1, t2], [37, 20], [16 * 5 + 5, 16 * 10 + 4], dec, [0, 1]).copy()
    lc = ec.step([t1, t2], [37, 20], [16 * 5 + 5, 16 * 10 + 4], dec, [0, 1]).copy()
    assert rel_err(lg, lc) <= TOL


def test_greedy_tokens_identical_for_32_steps(gpu):
    cfg = small()
    w = Weights.random(cfg, 17)
    lim = Limits(page=16, pages=64, max_tokens=128, max_seq_pages=8)
    g = np.random.default_rng(2)
    reqs = [Request(g.integers(0, cfg.vocab, n).tolist(), 32) for n in (40, 7, 64, 19)]
    cpu, _ = generate_with(Engine(EmuGpu(), w, lim), reqs, 4, True)
    for device_argmax in (False, True):
        got, st = generate_with(Engine(gpu, w, lim), reqs, 4, True, device_argmax=device_argmax)
        assert st.decode_steps == 31
        for a, b in zip(got, cpu):
            assert a.tokens == b.tokens, (a.tokens, b.tokens)


def test_graph_replay_equals_plain_launches(gpu):
    cfg = small()
    w = Weights.random(cfg, 19)
    lim = Limits(page=16, pages=64, max_tokens=16, max_seq_pages=4)
    g = np.random.default_rng(3)
    reqs = [Request(g.integers(0, cfg.vocab, 5).tolist(), 12) for _ in range(16)]  # 16 rows: bw == t
    e1 = Engine(gpu, w, lim)
    a, _ = generate_with(e1, reqs, 16, False, device_argmax=True)
    assert e1._graph, "a 16-sequence decode step is recorded as a graph"
    e2 = Engine(gpu, w, lim)
    e2.graphs = False
    b, _ = generate_with(e2, reqs, 16, False, device_argmax=True)
    assert [o.tokens for o in a] == [o.tokens for o in b]


def test_engine_from_a_checkpoint_directory(gpu, tmp_path):
    """A model saved as a Hugging Face directory and loaded back generates the same tokens as the
    model it was saved from (src/llm/safetensors.rs:324-443)."""
    from tessel_b200 import checkpoint
    cfg = small()
    w = Weights.random(cfg, 21)
    checkpoint.save(w, str(tmp_path))
    lim = Limits(page=16, pages=32, max_tokens=64, max_seq_pages=8)
    reqs = [Request([1, 5, 9, 200, 31], 8), Request(list(range(40, 70)), 8)]
    a, _ = generate_with(Engine(gpu, w, lim), reqs, 2, True, device_argmax=True)
    b, _ = generate_with(Engine(gpu, checkpoint.load(str(tmp_path)), lim), reqs, 2, True, device_argmax=True)
    assert [o.tokens for o in a] == [o.tokens for o in b]


def test_long_prompt_fed_in_chunks_alongside_decodes(gpu):
    """A prompt longer than the step, fed 48 tokens at a time as rows of the decode steps: the
    GPU engine and the CPU engine (oracle kernels) produce the same tokens."""
    cfg = small()
    w = Weights.random(cfg, 23)
    lim = Limits(page=16, pages=48, max_tokens=64, max_seq_pages=16)
    g = np.random.default_rng(5)
    reqs = [Request(g.integers(0, cfg.vocab, 9).tolist(), 10), Request(g.integers(0, cfg.vocab, 170).tolist(), 8)]
    got, st = generate_with(Engine(gpu, w, lim), reqs, 2, True, device_argmax=True, chunk=48)
    want, _ = generate_with(Engine(EmuGpu(), w, lim), reqs, 2, True, chunk=48)
    assert st.prompt_tokens == 179
    assert [o.tokens for o in got] == [o.tokens for o in want]
