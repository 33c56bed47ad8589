"""The engine and the scheduler on the CPU stand-in (tests/emu.py), following the
reference's own engine tests (tests/llm.rs:25-83 and :193-227): prefill logits and
continuous-batched generation against the f32 one-sequence model, packed prefill against
one prompt per step, and the padding / graph / page bookkeeping of a step."""
import numpy as np
import pytest

import oracle
from emu import EmuGpu
from refs import rel_err
from tessel_b200.engine import Decode, Engine, Limits, Packed, Prefill, padded, padded_prefill, shard_weights
from tessel_b200.model import Config, Weights, argmax
from tessel_b200.sched import Request, generate, generate_with


def limits():
    return Limits(page=8, pages=32, max_tokens=16, max_seq_pages=8)


def test_padded():
    assert [padded(n) for n in (1, 16, 17, 32, 33, 300)] == [16, 16, 32, 32, 64, 512]


def test_long_prefill_steps_pad_to_256_rows_and_change_nothing():
    assert [padded_prefill(n) for n in (1, 17, 256, 257, 300, 512, 1300, 2048)] == [16, 32, 256, 512, 512, 512, 1536,
                                                                                   2048]
    cfg = Config.tiny()
    w = Weights.random(cfg, 5)
    lim = Limits(page=8, pages=128, max_tokens=600, max_seq_pages=80)
    prompt = [1 + (i * 29 % 250) for i in range(250)]
    # 250 + 30 tokens in one packed step: 280 rows run as 512; alone, 250 rows run as 256.
    reqs = [Request(prompt, 3), Request(prompt[:30], 3)]
    g = EmuGpu()
    packed, _ = generate_with(Engine(g, w, lim), reqs, 2, True)
    shapes = {k[1][0] for k in g._kernels if k[0] == "embed"}
    assert (512,) in shapes
    single, _ = generate_with(Engine(EmuGpu(), w, lim), reqs, 2, False)
    for a, b in zip(packed, single):
        assert a.tokens == b.tokens


def test_a_prompt_longer_than_a_step_is_fed_in_chunks():
    """Off by default (the reference refuses such a prompt, src/llm/sched.rs:76-81); with
    ``chunk`` the long prompt rides along the decode steps and ends in the same tokens as a
    prefill in one step on an engine large enough for it."""
    cfg = Config.tiny()
    w = Weights.random(cfg, 9)
    long = [1 + (i * 31 % 250) for i in range(150)]
    reqs = [Request([1, 9, 42, 7, 200, 13], 12), Request(long, 6), Request([3, 5, 8], 10)]
    big = Limits(page=8, pages=96, max_tokens=256, max_seq_pages=24)
    small = Limits(page=8, pages=96, max_tokens=64, max_seq_pages=24)
    want, _ = generate_with(Engine(EmuGpu(), w, big), reqs, 3, True)
    with pytest.raises(ValueError, match="does not fit"):
        generate_with(Engine(EmuGpu(), w, small), reqs, 3, True)
    got, st = generate_with(Engine(EmuGpu(), w, small), reqs, 3, True, chunk=40)
    for a, b in zip(got, want):
        assert a.tokens == b.tokens
    assert st.prompt_tokens == sum(len(r.prompt) for r in reqs)
    # Alone, too: nothing is running while the prompt is fed.
    got, _ = generate_with(Engine(EmuGpu(), w, small), reqs[1:2], 1, True, chunk=33)
    assert got[0].tokens == want[1].tokens


def test_prefill_and_batched_decode_match_the_reference():
    cfg = Config.tiny()
    w = Weights.random(cfg, 7)
    e = Engine(EmuGpu(), w, limits())
    prompt = [1, 17, 200, 33, 5, 99, 64, 3, 250, 12]
    n = len(prompt)
    got = e.step(prompt, list(range(n)), list(range(n)), Prefill(), [n - 1])
    want = oracle.reference_forward(cfg, w, prompt)
    err = rel_err(got[0], want[n - 1])
    assert err < 2e-2, f"prefill logits differ by {err}"
    reqs = [Request([1, 5, 9], 6), Request(prompt, 4), Request([1, 100, 101, 102, 103, 104, 105], 9)]
    outs, st = generate(e, reqs, 3)
    assert st.largest_batch == 3
    for r, o in zip(reqs, outs):
        assert len(o.tokens) == r.max_new
        seq = list(r.prompt)
        for t in o.tokens:
            l = oracle.reference_forward(cfg, w, seq)[-1]
            best = argmax(l)
            scale = np.abs(l).max()
            assert t == best or l[best] - l[t] < 2e-2 * scale
            seq.append(t)


def test_packed_prefill_matches_one_prompt_per_step():
    cfg = Config.tiny()
    w = Weights.random(cfg, 11)
    lim = Limits(page=8, pages=64, max_tokens=128, max_seq_pages=16)
    long = [1 + (i * 37 % 250) for i in range(70)]
    short = [1, 9, 42, 7, 200, 13, 5, 77, 31, 64, 2, 150, 99, 3, 18, 240, 6, 11, 120, 45]
    reqs = [Request(long, 4), Request(short, 4)]
    packed, st = generate_with(Engine(EmuGpu(), w, lim), reqs, 2, True)
    assert st.prefill_steps == 1, "both prompts in one step"
    single, st = generate_with(Engine(EmuGpu(), w, lim), reqs, 2, False)
    assert st.prefill_steps == 2
    for a, b in zip(packed, single):
        assert a.tokens == b.tokens


def test_device_argmax_path_picks_the_same_tokens():
    cfg = Config.tiny()
    w = Weights.random(cfg, 5)
    reqs = [Request([1, 5, 9, 30], 5), Request([7, 8], 6)]
    a, _ = generate_with(Engine(EmuGpu(), w, limits()), reqs, 2, True, device_argmax=False)
    b, _ = generate_with(Engine(EmuGpu(), w, limits()), reqs, 2, True, device_argmax=True)
    assert [o.tokens for o in a] == [o.tokens for o in b]


def test_step_padding_slots_and_graph_replay():
    """Padding rows write to no slot (slot == pages * page); a decode step whose wanted rows fill
    the padded step is recorded once and replayed afterwards (src/llm/engine.rs:287-344)."""
    cfg = Config.tiny()
    w = Weights.random(cfg, 3)
    g = EmuGpu()
    e = Engine(g, w, Limits(page=8, pages=8, max_tokens=16, max_seq_pages=4))
    prompt = [3, 4, 5]
    e.step(prompt, [0, 1, 2], [8, 9, 10], Prefill(), [2])
    kc, vc = e.read_cache(0)
    flat = kc.reshape(64, -1)
    assert flat[8:11].any(axis=1).all()
    assert not flat[:8].any() and not flat[11:].any(), "padding rows must not touch the cache"
    # 16 sequences of one token each fill the padded step: graphs kick in.
    for rep in range(3):
        toks = list(range(16))
        e.step(toks, [0] * 16, list(range(16)), Decode([[0, 1]] * 16, [1] * 16), list(range(16)))
    assert g.captures == 1 and g.replays == 2
    with pytest.raises(ValueError):
        e.step([], [], [], Prefill(), [])
    with pytest.raises(ValueError):
        e.step([1] * 17, [0] * 17, [0] * 17, Prefill(), [])
    with pytest.raises(ValueError):
        e.step([1, 2], [0, 1], [0, 1], Packed([0]), [1])


def test_scheduler_page_accounting():
    """Pages are reserved for the whole sequence up front, handed out 0, 1, 2, ..., and come
    back when a sequence finishes (src/llm/sched.rs:60-89, :124-131)."""
    cfg = Config.tiny()
    w = Weights.random(cfg, 9)
    lim = Limits(page=8, pages=6, max_tokens=16, max_seq_pages=4)
    e = Engine(EmuGpu(), w, lim)
    # Each request needs ceil((5 + 8) / 8) = 2 pages: three run at once, the fourth waits.
    reqs = [Request([1, 2, 3, 4, 5], 8) for _ in range(4)]
    outs, st = generate(e, reqs, 4)
    assert st.largest_batch == 3 and st.prefill_steps == 2
    assert all(len(o.tokens) == 8 for o in outs)
    with pytest.raises(ValueError):
        generate(e, [Request([1] * 17, 2)], 1)
    with pytest.raises(ValueError):
        generate(e, [Request([1] * 4, 100)], 1)


def test_tensor_parallel_shards_reassemble():
    """The shards of wqkv / wo / wg / wu / wd tile the full matrices, and a 2-way split of one
    layer's projections sums to the unsharded result (the allreduce's job)."""
    cfg = Config.tiny()
    w = Weights.random(cfg, 2)
    s = [shard_weights(w, r, 2) for r in range(2)]
    hd, H, G = cfg.head_dim, cfg.heads, cfg.kv_heads
    l, a, b = w.layers[0], s[0].layers[0], s[1].layers[0]
    hl, gl = H // 2, G // 2
    q = np.concatenate([a.wqkv[:hl * hd], b.wqkv[:hl * hd]])
    k = np.concatenate([a.wqkv[hl * hd:(hl + gl) * hd], b.wqkv[hl * hd:(hl + gl) * hd]])
    v = np.concatenate([a.wqkv[(hl + gl) * hd:], b.wqkv[(hl + gl) * hd:]])
    assert np.array_equal(np.concatenate([q, k, v]), l.wqkv)
    assert np.array_equal(np.concatenate([a.wo, b.wo], 1), l.wo)
    assert np.array_equal(np.concatenate([a.wg, b.wg]), l.wg)
    assert np.array_equal(np.concatenate([a.wd, b.wd], 1), l.wd)
    assert s[0].cfg.heads == 2 and s[0].cfg.kv_heads == 1 and s[0].cfg.ffn == 64
