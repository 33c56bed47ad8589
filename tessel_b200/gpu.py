"""Buffers that outlive a kernel launch, and launches that take them.

The host-side mirror of tessel's ``Gpu`` (src/gpu.rs:28-263), with the same
methods, argument meaning and error behaviour, over the C ABI of
``libtessel_b200``: ``alloc`` (zero-filled), ``write`` / ``read`` (bounds
checked, synchronous), ``kernel`` (cached by name and shapes), ``launch``
(asynchronous; buffers, f32 and i32 scalars), ``capture_begin`` /
``capture_end`` / ``replay``, ``sync`` and the per-kernel ``profile``. Errors
are raised as :class:`GpuError` carrying the library's message, where the
reference returns ``Err(String)``.
"""
from __future__ import annotations

import ctypes as C
import struct
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple, Union

import numpy as np

from . import _lib


class GpuError(RuntimeError):
    pass


@dataclass(frozen=True)
class Buf:
    """A device buffer: its address and size in bytes (src/gpu.rs:14-19)."""
    ptr: int
    bytes: int


@dataclass(frozen=True)
class F32:
    value: float


@dataclass(frozen=True)
class I32:
    value: int


Arg = Union[Buf, F32, I32]


@dataclass(frozen=True)
class K:
    """A kernel made for its shapes (src/gpu.rs:47-48)."""
    id: int
    name: str


def _bits(a: Arg) -> int:
    if isinstance(a, Buf):
        return a.ptr
    if isinstance(a, F32):
        return struct.unpack("<I", struct.pack("<f", a.value))[0]
    if isinstance(a, I32):
        return a.value & 0xFFFFFFFF
    raise TypeError(f"not a kernel argument: {a!r}")


class Gpu:
    def __init__(self, device: int = 0):
        self._l = _lib.lib()
        h = C.c_void_p()
        if self._l.tb200_init(device, C.byref(h)) != 0:
            raise GpuError(self._l.tb200_last_error(None).decode())
        self._h = h
        self.device = device
        self.launches = 0
        self._profiling = False
        self._phase = ""
        # Kernels whose tiles were chosen by timing (``tune``): id -> ((MT, BN, splits), microseconds).
        self.tuned: Dict[int, tuple] = {}
        self.fusion: Dict[int, bool] = {}   # fused-kernel id -> whether the engine's timing preferred it

    # -- plumbing --------------------------------------------------------------
    def _check(self, rc: int) -> None:
        if rc != 0:
            raise GpuError(self._l.tb200_last_error(self._h).decode())

    def close(self) -> None:
        if self._h:
            self._l.tb200_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- buffers ---------------------------------------------------------------
    def alloc(self, nbytes: int) -> Buf:
        """A zeroed buffer of ``nbytes`` bytes."""
        p = C.c_uint64()
        self._check(self._l.tb200_alloc(self._h, nbytes, C.byref(p)))
        return Buf(p.value, nbytes)

    def wrap(self, ptr: int, nbytes: int) -> Buf:
        """A buffer over device memory allocated elsewhere in this process."""
        return Buf(int(ptr), int(nbytes))

    def free(self, b: Buf) -> None:
        self._check(self._l.tb200_free(self._h, b.ptr))

    def write(self, b: Buf, offset: int, data) -> None:
        """Copies ``data`` (bytes or a contiguous numpy array) into ``b`` at byte ``offset``."""
        a = np.ascontiguousarray(data) if isinstance(data, np.ndarray) else np.frombuffer(bytes(data), np.uint8)
        n = a.nbytes
        if offset + n > b.bytes:
            raise GpuError(f"write of {n} bytes at {offset} into a buffer of {b.bytes}")
        self._check(self._l.tb200_write(self._h, b.ptr, offset, a.ctypes.data_as(C.c_void_p), n))

    def write_async(self, b: Buf, offset: int, a: np.ndarray) -> None:
        """As ``write`` without waiting; ``a`` must stay alive and unchanged until the next ``sync``."""
        n = a.nbytes
        if offset + n > b.bytes:
            raise GpuError(f"write of {n} bytes at {offset} into a buffer of {b.bytes}")
        self._check(self._l.tb200_write_async(self._h, b.ptr, offset, a.ctypes.data_as(C.c_void_p), n))

    def read(self, b: Buf, offset: int, out: np.ndarray) -> np.ndarray:
        """Reads ``out.nbytes`` bytes of ``b`` from byte ``offset`` (waiting for the GPU)."""
        assert out.flags["C_CONTIGUOUS"]
        if offset + out.nbytes > b.bytes:
            raise GpuError(f"read of {out.nbytes} bytes at {offset} from a buffer of {b.bytes}")
        self._check(self._l.tb200_read(self._h, b.ptr, offset, out.ctypes.data_as(C.c_void_p), out.nbytes))
        return out

    def read_f32(self, b: Buf, offset_elems: int, n: int) -> np.ndarray:
        return self.read(b, offset_elems * 4, np.empty(n, np.float32))

    def host_array(self, shape, dtype) -> np.ndarray:
        """A page-locked numpy array (lives until the context is closed)."""
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        p = C.c_void_p()
        self._check(self._l.tb200_host_alloc(self._h, max(n, 1), C.byref(p)))
        raw = (C.c_uint8 * max(n, 1)).from_address(p.value)
        return np.frombuffer(raw, dtype=dtype, count=int(np.prod(shape))).reshape(shape)

    def tensor(self, t: np.ndarray) -> Buf:
        """A buffer holding ``t`` as the kernels read it (src/gpu.rs:257-262). A tensor that is
        already on the device (``model.DevArray``) is used where it lies."""
        if hasattr(t, "ptr") and hasattr(t, "nbytes") and not isinstance(t, np.ndarray):
            return Buf(int(t.ptr), int(t.nbytes))
        t = np.ascontiguousarray(t)
        b = self.alloc(max(t.nbytes, 1))
        if t.nbytes:
            self.write(b, 0, t)
        return b

    def fetch(self, b: Buf, dtype, shape) -> np.ndarray:
        out = np.empty(shape, dtype)
        return self.read(b, 0, out)

    # -- kernels ---------------------------------------------------------------
    def kernel(self, name: str, shapes: Sequence[Sequence[int]]) -> K:
        """Kernel ``name`` for these array shapes, made once and then reused.

        The reference's ``file``, ``meta`` and ``warps`` arguments
        (src/gpu.rs:148-155) have no equivalent: tile shapes are chosen in the
        library.
        """
        flat = [int(d) for s in shapes for d in s]
        ranks = [len(s) for s in shapes]
        fa = (C.c_int64 * max(len(flat), 1))(*flat)
        ra = (C.c_int32 * max(len(ranks), 1))(*ranks)
        out = C.c_int32()
        self._check(self._l.tb200_kernel(self._h, name.encode(), fa, ra, len(ranks), C.byref(out)))
        return K(out.value, name)

    def launch(self, k: K, args: Sequence[Arg]) -> None:
        """Launches ``k`` (asynchronously)."""
        raw = (C.c_uint64 * max(len(args), 1))(*[_bits(a) for a in args])
        self.launches += 1
        self._check(self._l.tb200_launch(self._h, k.id, raw, len(args)))

    # -- the per-kernel profile (src/gpu.rs:38-42, :198-222), kept by the library ------------
    @property
    def profile(self):
        """None, or (while profiling) the table so far as {(phase, kernel): [launches, ms]}.
        Assigning anything but None clears the table and starts profiling: every launch then
        waits for its kernel and adds its device time; assigning None stops it."""
        if not self._profiling:
            return None
        return {(p, k): [n, ms] for p, k, n, ms in self.profile_rows()}

    @profile.setter
    def profile(self, value) -> None:
        self._profiling = value is not None
        self._check(self._l.tb200_profile(self._h, 1 if self._profiling else 0))

    @property
    def phase(self) -> str:
        return self._phase

    @phase.setter
    def phase(self, value: str) -> None:
        if value != self._phase:
            self._phase = value
            self._check(self._l.tb200_phase(self._h, value.encode()))

    def tune(self, k: K, args: Sequence[Arg]):
        """Times the candidate tiles of projection kernel ``k`` on ``args`` and keeps the fastest
        (``tb200_tune``; the reference's ``Engine::mm``, src/llm/engine.rs:233-270). Returns
        ((MT, BN, splits), microseconds); whatever ``k`` writes is clobbered."""
        raw = (C.c_uint64 * max(len(args), 1))(*[_bits(a) for a in args])
        plan = (C.c_int32 * 3)()
        us = C.c_float()
        self._check(self._l.tb200_tune(self._h, k.id, raw, len(args), plan, C.byref(us)))
        return tuple(plan), us.value

    def decode_attention_static(self, dims: Sequence[int], q: Buf, kc: Buf, vc: Buf, table: Buf, lens: Buf, o: Buf,
                                scale: float) -> None:
        """Paged decode attention without any device allocation (``tb200_decode_attention_static``):
        for hosts that handed all device memory to their own pool, or that may not allocate where
        they run. ``dims`` = (B, H, G, D, NP, P, MP). The split-KV scratch is a 16 MiB array inside
        the library; B*H*(D+2)*4 bytes must fit it. Make the first call on a device outside any
        stream capture, and keep calls on one stream: they share the array."""
        d = (C.c_int32 * 7)(*[int(x) for x in dims])
        self.launches += 1
        self._check(self._l.tb200_decode_attention_static(self._h, d, q.ptr, kc.ptr, vc.ptr, table.ptr, lens.ptr,
                                                          o.ptr, scale))

    def profile_rows(self):
        """The profile, largest first: (phase, kernel, launches, milliseconds)."""
        n = C.c_int()
        self._check(self._l.tb200_profile_rows(self._h, C.byref(n)))
        rows = []
        for i in range(n.value):
            ph, kn, cnt, ms = C.c_char_p(), C.c_char_p(), C.c_uint64(), C.c_double()
            self._check(self._l.tb200_profile_row(self._h, i, C.byref(ph), C.byref(kn), C.byref(cnt), C.byref(ms)))
            rows.append((ph.value.decode(), kn.value.decode(), int(cnt.value), float(ms.value)))
        return rows

    # -- graphs, sync, timing ----------------------------------------------------
    def capture_begin(self) -> None:
        self._check(self._l.tb200_capture_begin(self._h))

    def capture_end(self) -> int:
        g = C.c_int32()
        self._check(self._l.tb200_capture_end(self._h, C.byref(g)))
        return g.value

    def replay(self, g: int) -> None:
        self.launches += 1
        self._check(self._l.tb200_replay(self._h, g))

    def sync(self) -> None:
        self._check(self._l.tb200_sync(self._h))

    def time_begin(self) -> None:
        self._check(self._l.tb200_time_begin(self._h))

    def time_end(self) -> float:
        ms = C.c_float()
        self._check(self._l.tb200_time_end(self._h, C.byref(ms)))
        return ms.value

    def kernel_launches(self) -> int:
        """Kernels launched by the library on this context."""
        n = C.c_uint64()
        self._check(self._l.tb200_launch_count(self._h, C.byref(n)))
        return n.value

    def set_stream(self, stream_ptr: Optional[int]) -> None:
        self._check(self._l.tb200_set_stream(self._h, C.c_void_p(stream_ptr) if stream_ptr else None))

    # -- tensor parallelism ------------------------------------------------------
    def comm_id(self) -> bytes:
        buf = C.create_string_buffer(_lib.COMM_ID_BYTES)
        self._check(self._l.tb200_comm_id(self._h, buf))
        return buf.raw

    def comm_init(self, rank: int, nranks: int, comm_id: bytes) -> None:
        buf = C.create_string_buffer(comm_id, _lib.COMM_ID_BYTES)
        self._check(self._l.tb200_comm_init(self._h, rank, nranks, buf))

    def ipc_export(self, b: Buf) -> bytes:
        buf = C.create_string_buffer(64)
        self._check(self._l.tb200_ipc_export(self._h, b.ptr, buf))
        return buf.raw

    def ipc_import(self, handle: bytes, nbytes: int) -> Buf:
        p = C.c_uint64()
        self._check(self._l.tb200_ipc_import(self._h, C.create_string_buffer(handle, 64), C.byref(p)))
        return Buf(p.value, nbytes)

    def tp_sizes(self):
        """(table, trace) byte sizes of the fused cross-rank reduction's bookkeeping."""
        a, b = C.c_size_t(), C.c_size_t()
        self._check(self._l.tb200_tp_sizes(C.byref(a), C.byref(b)))
        return a.value, b.value

    def tp_table(self, rank: int, nranks: int, inbox0, inbox1, landing, x: Buf, h: Buf,
                 trace: Optional[Buf] = None) -> bytes:
        """The table ``linear_scatter`` and ``tp_reduce_norm`` read. ``inbox0``, ``inbox1`` and
        ``landing`` are lists of Buf indexed by rank (filled with 0xff bytes by their owners:
        :meth:`fill`), ``x`` and ``h`` this rank's own buffers."""
        n = self.tp_sizes()[0]
        out = C.create_string_buffer(n)
        arr = lambda bs: (C.c_uint64 * 8)(*[b.ptr for b in bs])
        self._check(self._l.tb200_tp_table(self._h, out, n, rank, nranks, arr(inbox0), arr(inbox1), arr(landing),
                                           x.ptr, h.ptr, trace.ptr if trace else 0))
        return out.raw

    def fill(self, b: Buf, value: int) -> None:
        """Every byte of ``b`` set to ``value`` (``tb200_memset``, on the stream)."""
        self._check(self._l.tb200_memset(self._h, b.ptr, value, b.bytes))

    def allreduce(self, b: Buf, count: int, dtype: int = 0) -> None:
        self._check(self._l.tb200_allreduce(self._h, b.ptr, count, dtype))
