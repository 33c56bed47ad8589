"""Hugging Face Llama-family checkpoints (config.json + safetensors) to ``Weights``.

Host-side mirror of tessel's ``src/llm/safetensors.rs``: ``config`` (:189-226),
the tensor index over ``model.safetensors`` or the files named by
``model.safetensors.index.json`` (:236-292), dtype conversion to f16 (F16 as is,
BF16 and F32 rounded to nearest even, :295-321; beyond the reference, F8_E4M3 with its scale
tensor is dequantised), ``load`` (:324-367) and ``save``
(:369-443). Unlike the reference, ``load`` can return one tensor-parallel rank's
shard directly: files are memory-mapped and only the rows (wqkv, wg, wu) or
columns (wo, wd) that the rank keeps are read and converted, so eight ranks
loading one checkpoint read it once between them, not eight times.
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .model import Config, Layer, Weights


class CheckpointError(ValueError):
    pass


def config(path: str) -> Config:
    """The model's shape from ``config.json``; rope scaling and biases are not supported, as in the reference."""
    p = os.path.join(path, "config.json")
    try:
        with open(p) as fh:
            j = json.load(fh)
    except OSError as e:
        raise CheckpointError(f"{p}: {e}") from None
    except json.JSONDecodeError as e:
        raise CheckpointError(f"{p}: {e}") from None

    def need(k: str):
        if not isinstance(j.get(k), (int, float)) or isinstance(j.get(k), bool):
            raise CheckpointError(f"config.json: no {k}")
        return j[k]

    def opt(k: str, d):
        v = j.get(k)
        return v if isinstance(v, (int, float)) and not isinstance(v, bool) else d

    if j.get("rope_scaling") is not None:
        raise CheckpointError("config.json: rope_scaling is not supported")
    heads, dim = int(need("num_attention_heads")), int(need("hidden_size"))
    eos = j.get("eos_token_id")
    if isinstance(eos, list):
        eos = eos[0] if eos and isinstance(eos[0], (int, float)) else -1
    elif not isinstance(eos, (int, float)) or isinstance(eos, bool):
        eos = -1
    return Config(dim=dim, layers=int(need("num_hidden_layers")), heads=heads,
                  kv_heads=int(opt("num_key_value_heads", heads)), head_dim=int(opt("head_dim", dim // heads)),
                  ffn=int(need("intermediate_size")), vocab=int(need("vocab_size")),
                  eps=float(opt("rms_norm_eps", 1e-6)),
                  rope_theta=float(opt("rope_theta", 10000.0)),
                  max_pos=min(int(opt("max_position_embeddings", 2048)), 8192), bos=int(opt("bos_token_id", 1)),
                  eos=int(eos))


@dataclass
class _Entry:
    file: str
    dtype: str
    shape: Tuple[int, ...]
    start: int
    end: int


_DTYPES = {"F16": (np.float16, 2), "BF16": (np.uint16, 2), "F32": (np.float32, 4), "F8_E4M3": (np.uint8, 1)}


class Index:
    """Every tensor of a checkpoint directory by name, backed by read-only memory maps."""

    def __init__(self, path: str):
        single = os.path.join(path, "model.safetensors")
        if os.path.exists(single):
            files = [single]
        else:
            p = os.path.join(path, "model.safetensors.index.json")
            try:
                with open(p) as fh:
                    wm = json.load(fh).get("weight_map")
            except OSError as e:
                raise CheckpointError(f"{p}: {e}") from None
            if not isinstance(wm, dict):
                raise CheckpointError("index: no weight_map")
            files = sorted({os.path.join(path, v) for v in wm.values() if isinstance(v, str)})
        self.entries: Dict[str, _Entry] = {}
        self._maps: Dict[str, np.memmap] = {}
        for f in files:
            try:
                with open(f, "rb") as fh:
                    raw = fh.read(8)
                    if len(raw) != 8:
                        raise CheckpointError(f"{f}: shorter than its own header")
                    (n,) = struct.unpack("<Q", raw)
                    size = os.fstat(fh.fileno()).st_size
                    if n > size - 8:
                        raise CheckpointError(f"{f}: header of {n} bytes in a file of {size}")
                    head = json.loads(fh.read(n).decode("utf-8"))
            except OSError as e:
                raise CheckpointError(f"{f}: {e}") from None
            except (UnicodeDecodeError, json.JSONDecodeError) as e:
                raise CheckpointError(f"{f}: bad header: {e}") from None
            if not isinstance(head, dict):
                raise CheckpointError("safetensors: bad header")
            for name, v in head.items():
                if name == "__metadata__":
                    continue
                off = v.get("data_offsets") if isinstance(v, dict) else None
                if not (isinstance(off, list) and len(off) == 2):
                    raise CheckpointError(f"{name}: no data_offsets")
                start, end = 8 + n + int(off[0]), 8 + n + int(off[1])
                if not (8 + n <= start <= end <= size):
                    raise CheckpointError(f"{name}: data outside {f}")
                self.entries[name] = _Entry(f, str(v.get("dtype", "")), tuple(int(x) for x in v.get("shape", [])),
                                            start, end)

    def __contains__(self, name: str) -> bool:
        return name in self.entries

    def names(self) -> List[str]:
        return list(self.entries)

    def raw(self, name: str, shape: Sequence[int]) -> np.ndarray:
        """The stored tensor, checked against the expected shape, as a view of the mapped file
        (``uint16`` for BF16)."""
        e = self.entries.get(name)
        if e is None:
            raise CheckpointError(f"checkpoint has no {name}")
        if e.shape != tuple(shape):
            raise CheckpointError(f"{name}: shape {list(e.shape)}, expected {list(shape)}")
        if e.dtype not in _DTYPES:
            raise CheckpointError(f"{name}: dtype {e.dtype} not supported")
        dt, size = _DTYPES[e.dtype]
        n = int(np.prod(shape)) if len(shape) else 1
        if e.end - e.start != n * size:
            raise CheckpointError(f"{name}: dtype {e.dtype} not supported")
        m = self._maps.get(e.file)
        if m is None:
            m = self._maps[e.file] = np.memmap(e.file, np.uint8, "r")
        return m[e.start:e.end].view(dt).reshape(shape)

    def f16(self, name: str, shape: Sequence[int], rows: Optional[slice] = None,
            cols: Optional[slice] = None) -> np.ndarray:
        """Rows ``rows`` and columns ``cols`` of the tensor as f16 (BF16 and F32 rounded to
        nearest even), in memory of its own."""
        a = self.raw(name, shape)
        dtype = self.entries[name].dtype
        if rows is not None:
            a = a[rows]
        if cols is not None:
            a = a[:, cols]
        if dtype == "BF16":
            a = (a.astype(np.uint32) << 16).view(np.float32)
        elif dtype == "F8_E4M3":
            # E4M3 bytes, with the scale tensor FP8 checkpoints store beside a weight
            # ("....weight_scale": one f32 for the tensor, or one per output row).
            from . import fp8
            a = fp8.decode(a)
            sname = name + "_scale"
            if sname in self.entries:
                e = self.entries[sname]
                sc = self.raw(sname, e.shape).astype(np.float32).reshape(-1)
                if sc.size == 1:
                    a = a * sc[0]
                elif sc.size == shape[0]:
                    a = a * (sc[rows] if rows is not None else sc)[:, None]
                else:
                    raise CheckpointError(f"{sname}: {sc.size} scales for a tensor of {shape[0]} rows")
        with np.errstate(over="ignore"):
            return np.ascontiguousarray(a.astype(np.float16))


def load(path: str, rank: int = 0, nranks: int = 1) -> Weights:
    """A Llama-family checkpoint directory as ``Weights``. With ``nranks > 1`` the result is rank
    ``rank``'s tensor-parallel shard, sliced as ``engine.shard_weights`` slices a whole model
    (``Engine(..., sharded=True)`` takes it as is): its query heads, KV heads and MLP columns;
    norms, embedding and LM head whole."""
    cfg = config(path)
    ix = Index(path)
    for name in ix.names():
        if name.endswith(".bias"):
            raise CheckpointError(f"{name}: models with biases are not supported")
    if not 0 <= rank < nranks:
        raise CheckpointError(f"rank {rank} of {nranks}")
    if cfg.heads % nranks or cfg.kv_heads % nranks or cfg.ffn % nranks:
        raise CheckpointError(f"heads {cfg.heads}, kv_heads {cfg.kv_heads} and ffn {cfg.ffn} must divide by {nranks}")
    dm, hd = cfg.dim, cfg.head_dim
    hl, gl, fl = cfg.heads // nranks, cfg.kv_heads // nranks, cfg.ffn // nranks
    qs = slice(rank * hl * hd, (rank + 1) * hl * hd)
    ks = slice(rank * gl * hd, (rank + 1) * gl * hd)
    fs = slice(rank * fl, (rank + 1) * fl)
    layers = []
    for i in range(cfg.layers):
        p = f"model.layers.{i}."
        wqkv = np.concatenate([ix.f16(p + "self_attn.q_proj.weight", (cfg.heads * hd, dm), rows=qs),
                               ix.f16(p + "self_attn.k_proj.weight", (cfg.kv_heads * hd, dm), rows=ks),
                               ix.f16(p + "self_attn.v_proj.weight", (cfg.kv_heads * hd, dm), rows=ks)], 0)
        layers.append(Layer(
            attn_norm=ix.f16(p + "input_layernorm.weight", (dm,)), wqkv=wqkv,
            wo=ix.f16(p + "self_attn.o_proj.weight", (dm, cfg.heads * hd), cols=qs),
            mlp_norm=ix.f16(p + "post_attention_layernorm.weight", (dm,)),
            wg=ix.f16(p + "mlp.gate_proj.weight", (cfg.ffn, dm), rows=fs),
            wu=ix.f16(p + "mlp.up_proj.weight", (cfg.ffn, dm), rows=fs),
            wd=ix.f16(p + "mlp.down_proj.weight", (dm, cfg.ffn), cols=fs)))
    head = ix.f16("lm_head.weight", (cfg.vocab, dm)) if "lm_head.weight" in ix else None
    local = Config(**{**cfg.__dict__, "heads": hl, "kv_heads": gl, "ffn": fl})
    return Weights(local, ix.f16("model.embed_tokens.weight", (cfg.vocab, dm)), layers,
                   ix.f16("model.norm.weight", (dm,)), head)


def save(w: Weights, path: str, dtype: str = "F16") -> None:
    """Writes ``w`` (a whole model) as a checkpoint directory laid out as Hugging Face lays out a
    Llama model: ``config.json`` and one ``model.safetensors``. ``dtype`` "F16" (what the
    reference writes), "BF16" or "F32" choose the stored type (the latter two for tests of the
    conversions); "F8_E4M3" stores the projection matrices as E4M3 bytes with one f32 scale per
    output row in "<name>_scale" (tessel_b200/fp8.py) and everything else as F16."""
    if dtype not in _DTYPES:
        raise CheckpointError(f"dtype {dtype} not supported")
    c = w.cfg
    os.makedirs(path, exist_ok=True)
    cfg = {"model_type": "llama", "hidden_size": c.dim, "num_hidden_layers": c.layers,
           "num_attention_heads": c.heads, "num_key_value_heads": c.kv_heads, "head_dim": c.head_dim,
           "intermediate_size": c.ffn, "vocab_size": c.vocab, "rms_norm_eps": c.eps, "rope_theta": c.rope_theta,
           "max_position_embeddings": c.max_pos, "bos_token_id": c.bos, "eos_token_id": c.eos, "rope_scaling": None,
           "tie_word_embeddings": w.lm_head is None}
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump(cfg, fh)
    hd, H, G = c.head_dim, c.heads, c.kv_heads
    tensors: List[Tuple[str, np.ndarray]] = [("model.embed_tokens.weight", w.embed), ("model.norm.weight", w.norm)]
    if w.lm_head is not None:
        tensors.append(("lm_head.weight", w.lm_head))
    for i, l in enumerate(w.layers):
        p = f"model.layers.{i}."
        tensors += [(p + "input_layernorm.weight", l.attn_norm),
                    (p + "self_attn.q_proj.weight", l.wqkv[:H * hd]),
                    (p + "self_attn.k_proj.weight", l.wqkv[H * hd:(H + G) * hd]),
                    (p + "self_attn.v_proj.weight", l.wqkv[(H + G) * hd:]),
                    (p + "self_attn.o_proj.weight", l.wo),
                    (p + "post_attention_layernorm.weight", l.mlp_norm),
                    (p + "mlp.gate_proj.weight", l.wg), (p + "mlp.up_proj.weight", l.wu),
                    (p + "mlp.down_proj.weight", l.wd)]

    def stored(a: np.ndarray) -> np.ndarray:
        a = np.ascontiguousarray(a, np.float16)
        if dtype == "F16":
            return a
        if dtype == "F32":
            return a.astype(np.float32)
        return (a.astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)  # truncated to bf16's 8 significant bits

    blobs: List[Tuple[str, str, tuple, bytes]] = []  # name, dtype, shape, bytes
    for name, a in tensors:
        if dtype == "F8_E4M3":
            if "_proj.weight" in name:
                from . import fp8
                q, sc = fp8.quantize_rows(np.asarray(a, np.float32))
                blobs.append((name, "F8_E4M3", a.shape, q.tobytes()))
                blobs.append((name + "_scale", "F32", sc.shape, sc.tobytes()))
            else:
                blobs.append((name, "F16", a.shape, np.ascontiguousarray(a, np.float16).tobytes()))
        else:
            blobs.append((name, dtype, a.shape, stored(a).tobytes()))
    head, off = {}, 0
    for name, dt, shape, raw in blobs:
        head[name] = {"dtype": dt, "shape": list(shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
    hb = json.dumps(head).encode("utf-8")
    hb += b" " * (-len(hb) % 8)
    with open(os.path.join(path, "model.safetensors"), "wb") as fh:
        fh.write(struct.pack("<Q", len(hb)))
        fh.write(hb)
        for _, _, _, raw in blobs:
            fh.write(raw)
