"""A CPU stand-in for ``tessel_b200.gpu.Gpu`` whose kernels are the oracle's.

It plays the role tessel's ``Device::Emu`` plays in the reference's tests
(src/gpu.rs:70-107 with host buffers): the engine and the scheduler run
unchanged on it, so their host logic (padding, slots, block tables, graph
keying, tensor-parallel sharding) is tested without a GPU, and a GPU run of the
same engine can be compared with it. Test infrastructure only.
"""
from __future__ import annotations

import bisect
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np

import oracle
from tessel_b200.gpu import Buf, F32, GpuError, I32, K


class EmuGpu:
    def __init__(self, allreduce=None):
        self._bases: List[int] = []
        self._bufs: Dict[int, np.ndarray] = {}
        self._next = 1 << 20
        self._kernels: List[tuple] = []
        self.launches = 0
        self.profile = None
        self.phase = ""
        self.replays = 0
        self.captures = 0
        self._capturing = False
        self._recorded: List[list] = []
        # allreduce(np.ndarray f32) -> summed array, for tensor-parallel tests.
        self._allreduce = allreduce

    # -- buffers -----------------------------------------------------------------
    def alloc(self, nbytes: int) -> Buf:
        base = self._next
        self._next += (max(nbytes, 1) + 4095) // 4096 * 4096 + 4096
        self._bases.append(base)
        self._bufs[base] = np.zeros(max(nbytes, 1), np.uint8)
        return Buf(base, nbytes)

    def _view(self, ptr: int, nbytes: int) -> np.ndarray:
        i = bisect.bisect_right(self._bases, ptr) - 1
        base = self._bases[i]
        a = self._bufs[base]
        off = ptr - base
        assert off + nbytes <= a.size, "kernel argument runs past its buffer"
        return a[off:off + nbytes]

    def arr(self, b: Buf, dtype, shape) -> np.ndarray:
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        return self._view(b.ptr, n).view(dtype).reshape(shape)

    def write(self, b: Buf, offset: int, data) -> None:
        a = np.ascontiguousarray(data) if isinstance(data, np.ndarray) else np.frombuffer(bytes(data), np.uint8)
        if offset + a.nbytes > b.bytes:
            raise GpuError(f"write of {a.nbytes} bytes at {offset} into a buffer of {b.bytes}")
        self._view(b.ptr + offset, a.nbytes)[:] = a.reshape(-1).view(np.uint8)

    write_async = write

    def read(self, b: Buf, offset: int, out: np.ndarray) -> np.ndarray:
        if offset + out.nbytes > b.bytes:
            raise GpuError(f"read of {out.nbytes} bytes at {offset} from a buffer of {b.bytes}")
        out.reshape(-1).view(np.uint8)[:] = self._view(b.ptr + offset, out.nbytes)
        return out

    def read_f32(self, b, offset_elems, n):
        return self.read(b, offset_elems * 4, np.empty(n, np.float32))

    def host_array(self, shape, dtype):
        return np.zeros(shape, dtype)

    def tensor(self, t: np.ndarray) -> Buf:
        t = np.ascontiguousarray(t)
        b = self.alloc(max(t.nbytes, 1))
        if t.nbytes:
            self.write(b, 0, t)
        return b

    def fetch(self, b, dtype, shape):
        return self.read(b, 0, np.empty(shape, dtype))

    # -- kernels -----------------------------------------------------------------
    def kernel(self, name: str, shapes: Sequence[Sequence[int]]) -> K:
        key = (name, tuple(tuple(s) for s in shapes))
        for i, k in enumerate(self._kernels):
            if k == key:
                return K(i, name)
        self._kernels.append(key)
        return K(len(self._kernels) - 1, name)

    def launch(self, k: K, args) -> None:
        self.launches += 1
        if self._capturing:
            self._recorded[-1].append((k, list(args)))
            return
        name, sh = self._kernels[k.id]
        h, f, i = np.float16, np.float32, np.int32
        A = lambda n, dt: self.arr(args[n], dt, sh[n])
        sc = lambda n: args[n].value
        if name == "embed":
            A(2, f)[:] = oracle.embed(A(0, i), A(1, h))
        elif name == "rmsnorm":
            A(2, h)[:] = oracle.rmsnorm(A(0, f), A(1, h), sc(3))
        elif name == "rmsnorm_rows":
            A(3, h)[:] = oracle.rmsnorm_rows(A(0, f), A(1, i), A(2, h), sc(4))
        elif name == "linear":
            A(2, h)[:] = oracle.linear(A(0, h), A(1, h))
        elif name == "linear_residual":
            A(2, f)[:] = oracle.linear_residual(A(0, h), A(1, h), A(2, f))
        elif name in ("logits", "linear_f32"):
            A(2, f)[:] = oracle.logits(A(0, h), A(1, h))
        elif name == "gate_up":
            A(3, h)[:] = oracle.gate_up(A(0, h), A(1, h), A(2, h))
        elif name == "matmul":
            A(2, h)[:] = oracle.matmul(A(0, h), A(1, h))
        elif name == "rope_q":
            A(4, h)[:] = oracle.rope_q(A(0, h), A(1, i), A(2, f), A(3, f), sh[4][1], sh[4][2])
        elif name == "kv_write":
            kc, vc, kd, vd = oracle.kv_write(A(0, h), A(1, i), A(2, i), A(3, f), A(4, f), A(5, h), A(6, h), sh[5][1],
                                             sh[5][2])
            A(5, h)[:], A(6, h)[:], A(7, h)[:], A(8, h)[:] = kc, vc, kd, vd
        elif name == "rope_kv":
            A(5, h)[:] = oracle.rope_q(A(0, h), A(1, i), A(3, f), A(4, f), sh[5][1], sh[5][2])
            kc, vc, kd, vd = oracle.kv_write(A(0, h), A(1, i), A(2, i), A(3, f), A(4, f), A(6, h), A(7, h), sh[6][1],
                                             sh[6][2])
            A(6, h)[:], A(7, h)[:], A(8, h)[:], A(9, h)[:] = kc, vc, kd, vd
        elif name == "linear_rope_kv":
            # X, W, pos, slot, C, S, QKV, Q, Kc, Vc, K, V: linear, rope_q and kv_write in a row.
            qkv = oracle.linear(A(0, h), A(1, h))
            A(6, h)[:] = qkv
            A(7, h)[:] = oracle.rope_q(qkv, A(2, i), A(4, f), A(5, f), sh[7][1], sh[7][2])
            kc, vc, kd, vd = oracle.kv_write(qkv, A(2, i), A(3, i), A(4, f), A(5, f), A(8, h), A(9, h), sh[8][1],
                                             sh[8][2])
            A(8, h)[:], A(9, h)[:], A(10, h)[:], A(11, h)[:] = kc, vc, kd, vd
        elif name in ("quant_rows", "rmsnorm_q8", "linear_q8", "linear_residual_q8", "gate_up_q8"):
            self._q8(name, A, sc)
        elif name == "prefill_attention":
            A(4, h)[:] = oracle.prefill_attention(A(0, h), A(1, h), A(2, h), A(3, i), sc(5))
        elif name == "flash_attention":
            A(3, h)[:] = oracle.flash_attention(A(0, h), A(1, h), A(2, h), sc(4))
        elif name in ("decode_attention", "paged_attention"):
            A(5, h)[:] = oracle.decode_attention(A(0, h), A(1, h), A(2, h), A(3, i), A(4, i), sc(6))
        elif name == "chunk_attention":
            # Row r of a chunk is a decode query with r + 1 more cached tokens than the chunk's start.
            q, o, meta, table = A(0, h), A(5, h), A(4, i), A(3, i)
            for row0, nrows, pos0, _ in meta:
                if nrows <= 0:
                    continue
                rows = np.arange(row0, row0 + nrows)
                tb = np.repeat(table[row0:row0 + 1], nrows, axis=0)
                ln = (pos0 + 1 + np.arange(nrows)).astype(np.int32)
                o[rows] = oracle.decode_attention(q[rows], A(1, h), A(2, h), tb, ln, sc(6))
        elif name == "residual_add":
            A(0, f)[:] = A(0, f) + A(1, f)
        elif name == "argmax_rows":
            x = A(0, f)
            A(1, i)[:] = [oracle.argmax(r) for r in x]
        elif name == "argmax_partial":
            x, pr = A(0, f), A(1, f)
            rank, base = sc(2), sc(3)
            pr[:] = 0
            for m, row in enumerate(x):
                ok = ~np.isnan(row)
                if base == 0 and not ok[0]:
                    pr[rank, m] = (np.nan, 0)
                elif not ok.any():
                    pr[rank, m] = (-np.inf, -1)
                else:
                    at = int(np.argmax(np.where(ok, row, -np.inf)))
                    pr[rank, m] = (row[at], base + at)
        elif name == "argmax_merge":
            pr, out = A(0, f), A(1, i)
            for m in range(pr.shape[1]):
                best = pr[0, m]
                if not np.isnan(best[0]):
                    for r in range(1, pr.shape[0]):
                        v = pr[r, m]
                        if v[1] >= 0 and (v[0] > best[0] or best[1] < 0):
                            best = v
                out[m] = 0 if best[1] < 0 else int(best[1])
        else:
            raise GpuError(f"no kernel {name}")

    @staticmethod
    def _q8(name, A, sc) -> None:
        """The FP8 mode's kernels in numpy: the device's quantiser rule (tessel_b200/fp8.py), exact
        products of the decoded bytes summed in f64, scaled back in f32 as the epilogue does."""
        from tessel_b200 import fp8
        h, f, u8 = np.float16, np.float32, np.uint8

        def product(xq, sx, wq, sw):
            acc = (fp8.decode(xq).astype(np.float64) @ fp8.decode(wq).astype(np.float64).T).astype(f)
            return acc * (sx[:, None] * sw[None, :])

        if name == "quant_rows":
            A(1, u8)[:], A(2, f)[:] = fp8.quantize_rows(A(0, h).astype(f))
        elif name == "rmsnorm_q8":
            A(2, u8)[:], A(3, f)[:] = fp8.quantize_rows(oracle.rmsnorm(A(0, f), A(1, h), sc(4)).astype(f))
        elif name == "linear_q8":
            A(4, h)[:] = product(A(0, u8), A(1, f), A(2, u8), A(3, f)).astype(h)
        elif name == "linear_residual_q8":
            A(4, f)[:] = A(4, f) + product(A(0, u8), A(1, f), A(2, u8), A(3, f))
        else:
            g = product(A(0, u8), A(1, f), A(2, u8), A(3, f))
            u = product(A(0, u8), A(1, f), A(4, u8), A(5, f))
            A(6, h)[:] = ((g / (f(1) + np.exp(-g))) * u).astype(h)

    def allreduce(self, b: Buf, count: int, dtype: int = 0) -> None:
        if self._capturing:
            self._recorded[-1].append(("allreduce", b, count))
            return
        if self._allreduce is None:
            return
        a = self.arr(b, np.float32, (count,))
        a[:] = self._allreduce(a.copy())

    # -- graphs ------------------------------------------------------------------
    def capture_begin(self):
        self._capturing = True
        self.captures += 1
        self._recorded.append([])

    def capture_end(self) -> int:
        self._capturing = False
        return len(self._recorded) - 1

    def replay(self, g: int) -> None:
        self.replays += 1
        for item in self._recorded[g]:
            if item[0] == "allreduce":
                self.allreduce(item[1], item[2])
            else:
                self.launch(item[0], item[1])

    def sync(self):
        pass
