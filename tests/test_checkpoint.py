"""The checkpoint reader, tested as the reference tests its own (tests/llm.rs:84-101 saves the
tiny model of seed 3 with src/llm/safetensors.rs:369-443 and loads it back with :324-367),
plus the dtype conversions, sharded files, per-rank loading and the error cases."""
import json
import os
import struct

import numpy as np
import pytest

from tessel_b200 import checkpoint
from tessel_b200.checkpoint import CheckpointError
from tessel_b200.engine import shard_weights
from tessel_b200.model import Config, Weights


def same(a: Weights, b: Weights) -> None:
    assert a.cfg == b.cfg
    assert np.array_equal(a.embed, b.embed) and np.array_equal(a.norm, b.norm)
    assert (a.lm_head is None) == (b.lm_head is None)
    if a.lm_head is not None:
        assert np.array_equal(a.lm_head, b.lm_head)
    assert len(a.layers) == len(b.layers)
    for x, y in zip(a.layers, b.layers):
        for f in ("attn_norm", "wqkv", "wo", "mlp_norm", "wg", "wu", "wd"):
            assert np.array_equal(getattr(x, f), getattr(y, f)), f


def test_round_trip_f16(tmp_path):
    w = Weights.random(Config.tiny(), 3)
    checkpoint.save(w, str(tmp_path))
    same(checkpoint.load(str(tmp_path)), w)
    # Tied embeddings: no lm_head tensor is written or read.
    w.lm_head = None
    checkpoint.save(w, str(tmp_path / "tied"))
    got = checkpoint.load(str(tmp_path / "tied"))
    assert got.lm_head is None and np.array_equal(got.head(), w.embed)


@pytest.mark.parametrize("nranks", [2, 4])
def test_a_rank_loads_its_own_shard(tmp_path, nranks):
    cfg = Config(dim=64, layers=2, heads=8, kv_heads=4, head_dim=16, ffn=128, vocab=256, max_pos=256)
    w = Weights.random(cfg, 5)
    checkpoint.save(w, str(tmp_path))
    for r in range(nranks):
        same(checkpoint.load(str(tmp_path), r, nranks), shard_weights(w, r, nranks))
    with pytest.raises(CheckpointError, match="must divide"):
        checkpoint.load(str(tmp_path), 0, 3)


def test_bf16_and_f32_are_rounded_to_nearest_even(tmp_path):
    w = Weights.random(Config.tiny(), 4)
    checkpoint.save(w, str(tmp_path / "f32"), "F32")
    same(checkpoint.load(str(tmp_path / "f32")), w)  # f16 -> f32 -> f16 is the identity
    checkpoint.save(w, str(tmp_path / "bf16"), "BF16")
    got = checkpoint.load(str(tmp_path / "bf16"))
    # The writer truncates to bf16; every bf16 value of this size is an f16 value.
    want = ((w.embed.astype(np.float32).view(np.uint32) >> 16) << 16).view(np.float32).astype(np.float16)
    assert np.array_equal(got.embed, want)
    # Rounding, on values f16 cannot hold: ties go to the even neighbour, overflow to infinity.
    ix_dir = tmp_path / "vals"
    os.makedirs(ix_dir)
    vals = np.asarray([1.0 + 2.0 ** -11, 1.0 + 3 * 2.0 ** -11, 1.0 + 2.0 ** -11 + 2.0 ** -20, 65519.0, 65520.0, 1e-8,
                       -2.0 ** -25, 2.0 ** -24], np.float32)
    head = json.dumps({"t": {"dtype": "F32", "shape": [8], "data_offsets": [0, 32]},
                       "__metadata__": {"format": "pt"}}).encode()
    with open(ix_dir / "model.safetensors", "wb") as fh:
        fh.write(struct.pack("<Q", len(head)) + head + vals.tobytes())
    got = checkpoint.Index(str(ix_dir)).f16("t", (8,))
    want = np.asarray([1.0, 1.0 + 2.0 ** -9, 1.0 + 2.0 ** -10, 65504.0, np.inf, 0.0, -0.0, 2.0 ** -24], np.float16)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


def test_fp8_checkpoint_is_dequantised_with_its_row_scales(tmp_path):
    """Beyond the reference: projection matrices stored as F8_E4M3 with a "<name>_scale" tensor
    (one f32 per output row) load as f16(decode(bytes) * scale); a rank's shard takes its rows'
    scales; everything that is not a projection is stored and read as F16."""
    from tessel_b200 import fp8
    cfg = Config(dim=64, layers=2, heads=8, kv_heads=4, head_dim=16, ffn=128, vocab=256, max_pos=256)
    w = Weights.random(cfg, 6)
    checkpoint.save(w, str(tmp_path), "F8_E4M3")
    got = checkpoint.load(str(tmp_path))
    assert np.array_equal(got.embed, w.embed) and np.array_equal(got.norm, w.norm)
    for a, b in zip(got.layers, w.layers):
        assert np.array_equal(a.attn_norm, b.attn_norm)
        for name in ("wqkv", "wo", "wg", "wu", "wd"):
            x, y = getattr(a, name).astype(np.float32), getattr(b, name).astype(np.float32)
            assert np.abs(x - y).max() <= np.abs(y).max() / 14.0, name       # three mantissa bits
            assert np.abs(x - y).max() > 0, name
    # wo is stored whole and quantised by its own rows: the reader must reproduce exactly that.
    q, sc = fp8.quantize_rows(w.layers[0].wo.astype(np.float32))
    assert np.array_equal(got.layers[0].wo, (fp8.decode(q) * sc[:, None]).astype(np.float16))
    shard = checkpoint.load(str(tmp_path), 1, 2)
    assert np.array_equal(shard.layers[1].wg, got.layers[1].wg[cfg.ffn // 2:])


def test_sharded_files_and_config_defaults(tmp_path):
    """Tensors spread over the files of a model.safetensors.index.json; config.json with the
    optional keys absent and a list of end tokens."""
    w = Weights.random(Config.tiny(), 6)
    checkpoint.save(w, str(tmp_path))
    ix = checkpoint.Index(str(tmp_path))
    names = sorted(ix.names())
    wm = {}
    for part, chunk in enumerate((names[::2], names[1::2])):
        fname = f"model-{part + 1:05d}-of-00002.safetensors"
        head, blobs, off = {}, [], 0
        for n in chunk:
            e = ix.entries[n]
            a = np.asarray(ix.raw(n, e.shape))
            head[n] = {"dtype": "F16", "shape": list(e.shape), "data_offsets": [off, off + a.nbytes]}
            off += a.nbytes
            blobs.append(a.tobytes())
            wm[n] = fname
        hb = json.dumps(head).encode()
        with open(tmp_path / fname, "wb") as fh:
            fh.write(struct.pack("<Q", len(hb)) + hb + b"".join(blobs))
    with open(tmp_path / "model.safetensors.index.json", "w") as fh:
        json.dump({"metadata": {}, "weight_map": wm}, fh)
    del ix
    os.remove(tmp_path / "model.safetensors")
    same(checkpoint.load(str(tmp_path)), w)
    with open(tmp_path / "config.json", "w") as fh:
        json.dump({"hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4, "intermediate_size": 128,
                   "vocab_size": 256, "eos_token_id": [7, 9], "max_position_embeddings": 131072}, fh)
    c = checkpoint.config(str(tmp_path))
    assert (c.kv_heads, c.head_dim, c.eos, c.bos, c.max_pos) == (4, 16, 7, 1, 8192)
    assert c.eps == 1e-6 and c.rope_theta == 10000.0


def test_errors(tmp_path):
    w = Weights.random(Config.tiny(), 7)
    d = str(tmp_path)
    with pytest.raises(CheckpointError, match="config.json"):
        checkpoint.load(d)
    checkpoint.save(w, d)
    cfg = json.load(open(tmp_path / "config.json"))
    json.dump({**cfg, "rope_scaling": {"type": "linear", "factor": 2.0}}, open(tmp_path / "config.json", "w"))
    with pytest.raises(CheckpointError, match="rope_scaling is not supported"):
        checkpoint.load(d)
    json.dump({k: v for k, v in cfg.items() if k != "vocab_size"}, open(tmp_path / "config.json", "w"))
    with pytest.raises(CheckpointError, match="no vocab_size"):
        checkpoint.load(d)
    json.dump({**cfg, "intermediate_size": 256}, open(tmp_path / "config.json", "w"))
    with pytest.raises(CheckpointError, match=r"gate_proj.weight: shape \[128, 64\], expected \[256, 64\]"):
        checkpoint.load(d)
    json.dump({**cfg, "num_hidden_layers": 3}, open(tmp_path / "config.json", "w"))
    with pytest.raises(CheckpointError, match="checkpoint has no model.layers.2."):
        checkpoint.load(d)
    json.dump(cfg, open(tmp_path / "config.json", "w"))

    def rewrite(edit):
        raw = open(tmp_path / "model.safetensors", "rb").read()
        (n,) = struct.unpack("<Q", raw[:8])
        head = json.loads(raw[8:8 + n])
        edit(head)
        hb = json.dumps(head).encode()
        open(tmp_path / "model.safetensors", "wb").write(struct.pack("<Q", len(hb)) + hb + raw[8 + n:])

    rewrite(lambda h: h["model.norm.weight"].update(dtype="I8"))
    with pytest.raises(CheckpointError, match="dtype I8 not supported"):
        checkpoint.load(d)
    rewrite(lambda h: h["model.norm.weight"].update(dtype="F16"))
    rewrite(lambda h: h.update({"model.layers.0.self_attn.q_proj.bias": {"dtype": "F16", "shape": [1],
                                                                         "data_offsets": [0, 2]}}))
    with pytest.raises(CheckpointError, match="biases are not supported"):
        checkpoint.load(d)
    rewrite(lambda h: h.pop("model.layers.0.self_attn.q_proj.bias"))
    rewrite(lambda h: h["model.norm.weight"].update(data_offsets=[0, 1 << 40]))
    with pytest.raises(CheckpointError, match="data outside"):
        checkpoint.load(d)
