"""``CudaCompute``: the backend seam of the reference, served by the CUDA library.

Method names, argument meaning and refusals follow the reference's ``CpuCompute``
(crates/cpu-compute/src/cpu.rs:246-339, 506-655) and its ``KvCache``
(crates/attention/src/cache.rs), with one addition the device makes natural: a backend
holds ``n_slots`` resident sequences, so most calls name a ``slot``.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np

from . import _lib


class KvDtype(enum.IntEnum):
    F32 = _lib.KV_F32
    F16 = _lib.KV_F16


class CudaComputeError(Exception):
    """A named refusal: ``code`` is an ``itk_status``, ``msg`` the backend's text."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"[{code}] {msg}")
        self.code = code
        self.msg = msg


class PositionCache:
    """The forward loop's position contract (crates/muse-glimmer/src/cache.rs:18-74)."""

    def __init__(self):
        self._p = 0

    def position(self) -> int:
        return self._p

    def advance(self, tokens: int):
        self._p += tokens

    def rewind_to(self, position: int):
        self._p = position


@dataclass
class Checkpoint:
    id: int
    serial: int
    base_: int
    max_round_tokens_: int

    def base(self) -> int:
        return self.base_

    def max_round_tokens(self) -> int:
        return self.max_round_tokens_

    def _c(self):
        return _lib.Checkpoint(self.id, self.serial, self.base_, self.max_round_tokens_)


def _host_f32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


def _ptr(a: np.ndarray):
    return C.c_void_p(a.ctypes.data)


class DeviceSnapshot:
    """A device-resident prefix snapshot (one sequence prefix, position-ordered rows)."""

    def __init__(self, owner: "CudaCompute", handle):
        self._owner = owner
        self._h = handle

    def __del__(self):
        if getattr(self, "_h", None):
            _lib.load().itk_snapshot_free(self._h)
            self._h = None

    @property
    def token_count(self) -> int:
        return _lib.load().itk_snapshot_token_count(self._h)

    @property
    def payload_bytes(self) -> int:
        return _lib.load().itk_snapshot_payload_bytes(self._h)

    def to_itkv(self, model_fingerprint: str, version: int = 1) -> bytes:
        """The snapshot in the versioned ``ITKV`` byte format with its FNV-1a-64 checksum: version 1 is the
        reference's (f32 rows), version 2 stores the rows in the cache's own element type (half the bytes for f16)."""
        b = self._owner
        size = C.c_size_t()
        fp = model_fingerprint.encode()
        b._check(b._lib.itk_snapshot_to_itkv_version(b._h, self._h, fp, version, None, 0, C.byref(size)))
        buf = (C.c_uint8 * size.value)()
        b._check(b._lib.itk_snapshot_to_itkv_version(b._h, self._h, fp, version, buf, size.value, C.byref(size)))
        return bytes(buf)

    def layer(self, layer: int):
        """(first_position, keys, values): the layer block ``[rows][Hkv][D]`` in the cache's element type
        (``float32`` or raw ``uint16`` half bits)."""
        b = self._owner
        first, rows = C.c_uint64(), C.c_uint64()
        b._check(b._lib.itk_snapshot_layer_to_host(b._h, self._h, layer, None, None, C.byref(first), C.byref(rows)))
        dt = np.uint16 if b.kv_dtype == KvDtype.F16 else np.float32
        k = np.empty((rows.value, b.kv_heads, b.head_dim), dtype=dt)
        v = np.empty_like(k)
        if rows.value:
            b._check(b._lib.itk_snapshot_layer_to_host(b._h, self._h, layer, _ptr(k), _ptr(v), C.byref(first), C.byref(rows)))
        return first.value, k, v


class CudaCompute:
    """The CUDA backend: owns the resident KV of ``n_slots`` sequences on one B200."""

    def __init__(self, n_layers: int, q_heads: int, kv_heads: int, head_dim: int, *, n_slots: int = 1,
                 max_context: int = 4096, chunk_cap: int = 64, kv_dtype: KvDtype = KvDtype.F16,
                 layer_window: Optional[Sequence[int]] = None, device: int = 0,
                 options: Optional[dict] = None):
        self._lib = _lib.load()
        self._h = None
        self.n_layers, self.q_heads, self.kv_heads, self.head_dim = n_layers, q_heads, kv_heads, head_dim
        self.n_slots, self.max_context, self.chunk_cap = n_slots, max_context, chunk_cap
        self.kv_dtype = KvDtype(kv_dtype)
        self.layer_window = list(layer_window) if layer_window is not None else None
        win = None
        if self.layer_window is not None:
            win = (C.c_uint32 * max(len(self.layer_window), 1))(*self.layer_window)
        cfg = _lib.Config(n_layers, C.cast(win, C.POINTER(C.c_uint32)) if win is not None else None, q_heads, kv_heads,
                          head_dim, n_slots, max_context, chunk_cap, int(self.kv_dtype), device)
        h = C.c_void_p()
        rc = self._lib.itk_backend_create(C.byref(cfg), C.byref(h))
        if rc != _lib.OK:
            raise CudaComputeError(rc, self._lib.itk_last_error(None).decode("utf-8", "replace"))
        self._h = h
        for name, value in (options or {}).items():
            self.set_option(name, value)

    def set_option(self, name: str, value: int):
        """A tuning or A/B switch of this backend (``itk_set_option``): e.g. ``decode_ctas``, ``verify_tc``."""
        self._check(self._lib.itk_set_option(self._h, name.encode(), int(value)))

    def close(self):
        if self._h is not None:
            self._lib.itk_backend_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- plumbing -----------------------------------------------------------------------
    def _check(self, rc: int):
        if rc != _lib.OK:
            raise CudaComputeError(rc, self._lib.itk_last_error(self._h).decode("utf-8", "replace"))

    @property
    def q_width(self) -> int:
        return self.q_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.kv_heads * self.head_dim

    def set_stream(self, cuda_stream: int):
        """Issue work on a caller-owned ``cudaStream_t`` (e.g. ``torch.cuda.current_stream().cuda_stream``)."""
        self._check(self._lib.itk_set_stream(self._h, C.c_void_p(cuda_stream)))

    def synchronize(self):
        self._check(self._lib.itk_synchronize(self._h))

    def stats(self) -> dict:
        s = _lib.Stats()
        self._check(self._lib.itk_get_stats(self._h, C.byref(s)))
        return {name: getattr(s, name) for name, _ in s._fields_}

    def profile_enable(self, capacity: int):
        """Bracket up to ``capacity`` kernel launches with CUDA events (0 disables)."""
        self._check(self._lib.itk_profile_enable(self._h, capacity))

    def profile_read(self) -> dict:
        a_ms, p_ms = C.c_double(), C.c_double()
        a_n, p_n = C.c_uint64(), C.c_uint64()
        self._check(self._lib.itk_profile_read(self._h, C.byref(a_ms), C.byref(a_n), C.byref(p_ms), C.byref(p_n)))
        c_ms, c_n = C.c_double(), C.c_uint64()
        self._check(self._lib.itk_profile_read_copy(self._h, C.byref(c_ms), C.byref(c_n)))
        return {"attention_ms": a_ms.value, "attention_launches": a_n.value, "append_ms": p_ms.value,
                "append_launches": p_n.value, "copy_ms": c_ms.value, "copy_launches": c_n.value}

    # -- Compute::attention ---------------------------------------------------------------
    def attention(self, layer: int, q, k, v, cache: PositionCache, slot: int = 0) -> np.ndarray:
        """One sequence's attention step: append the RoPE'd rows at ``cache.position()``.., then attend.

        ``q`` is ``[rows][q_heads*D]``, ``k`` and ``v`` are ``[rows][kv_heads*D]``; returns ``[rows][q_heads*D]``.
        The caller advances ``cache`` afterwards, as the reference's forward does."""
        q, k, v = _host_f32(q).reshape(-1), _host_f32(k).reshape(-1), _host_f32(v).reshape(-1)
        out = np.empty(max(q.size, 1), dtype=np.float32)
        self._check(self._lib.itk_attention(self._h, slot, layer, _ptr(q), q.size, _ptr(k), k.size, _ptr(v), v.size,
                                            cache.position(), _ptr(out)))
        return out[: q.size]

    def attention_batch(self, layer: int, slots: Sequence[int], positions: Sequence[int], rows: int, q, k, v,
                        out: Optional[np.ndarray] = None) -> np.ndarray:
        """The same step for several slots at once; host arrays ``[n][rows][...]``."""
        n = len(slots)
        q, k, v = _host_f32(q), _host_f32(k), _host_f32(v)
        if out is None:
            out = np.empty(n * rows * self.q_width, dtype=np.float32)
        sl = (C.c_uint32 * n)(*slots)
        ps = (C.c_uint64 * n)(*positions)
        self._check(self._lib.itk_attention_batch(self._h, layer, n, sl, ps, rows, _ptr(q), _ptr(k), _ptr(v), _ptr(out)))
        return out

    def attention_batch_ptrs(self, layer: int, slots_c, positions_c, n: int, rows: int, q_ptr: int, k_ptr: int,
                             v_ptr: int, out_ptr: int, device: bool):
        """Raw-pointer form for callers that manage their own (pinned host or device) buffers."""
        fn = self._lib.itk_attention_batch_device if device else self._lib.itk_attention_batch
        self._check(fn(self._h, layer, n, slots_c, positions_c, rows, C.c_void_p(q_ptr), C.c_void_p(k_ptr),
                       C.c_void_p(v_ptr), C.c_void_p(out_ptr)))

    def attention_layers_host_ptrs(self, slots_c, positions_c, n: int, rows: int, q_ptr: int, k_ptr: int, v_ptr: int,
                                   out_ptr: int):
        """Every layer's attention step of one forward from host buffers ``[layers][n][rows][...]`` in one call;
        uploads, kernels and downloads of consecutive layers overlap.  Raw-pointer form."""
        self._check(self._lib.itk_attention_layers_host(self._h, n, slots_c, positions_c, rows, C.c_void_p(q_ptr),
                                                        C.c_void_p(k_ptr), C.c_void_p(v_ptr), C.c_void_p(out_ptr)))

    def attention_layers_host(self, slots: Sequence[int], positions: Sequence[int], rows: int, q, k, v) -> np.ndarray:
        n = len(slots)
        q, k, v = _host_f32(q), _host_f32(k), _host_f32(v)
        out = np.empty(self.n_layers * n * rows * self.q_width, dtype=np.float32)
        sl = (C.c_uint32 * n)(*slots)
        ps = (C.c_uint64 * n)(*positions)
        self.attention_layers_host_ptrs(sl, ps, n, rows, q.ctypes.data, k.ctypes.data, v.ctypes.data, out.ctypes.data)
        return out

    # -- attention preparation on the device (RMSNorm + RoPE ahead of the append) -----------------------------
    def set_layer_prep(self, layer: int, *, q_norm_weight=None, k_norm_weight=None, norm_eps: float = 1e-6,
                       rope_base: Optional[float] = None, rotary_dim: Optional[int] = None, pairing: int = 0):
        """Configure what the ``*_prep`` calls do to a layer's raw Q and K rows: per-head RMSNorm (a ``[head_dim]``
        weight each, or ``None`` to skip) and the rotation (``rope_base`` ``None`` skips it; ``pairing`` 0 joins
        channels (2i, 2i+1) as ``rope_interleaved`` does, 1 joins (i, i + rotary_dim/2) as ``rope`` does)."""
        qw = _host_f32(q_norm_weight).reshape(-1) if q_norm_weight is not None else None
        kw = _host_f32(k_norm_weight).reshape(-1) if k_norm_weight is not None else None
        for w in (qw, kw):
            if w is not None and w.size != self.head_dim:
                raise CudaComputeError(_lib.ERR_SHAPE_MISMATCH, f"rms_norm: got {w.size}, expected {self.head_dim}")
        rot = 0 if rope_base is None else (self.head_dim if rotary_dim is None else rotary_dim)
        cfg = _lib.PrepConfig(C.cast(_ptr(qw), C.POINTER(C.c_float)) if qw is not None else None,
                              C.cast(_ptr(kw), C.POINTER(C.c_float)) if kw is not None else None,
                              norm_eps, 0.0 if rope_base is None else rope_base, rot, pairing)
        self._check(self._lib.itk_layer_prep_set(self._h, layer, C.byref(cfg)))

    def attention_prep(self, layer: int, q, k, v, cache: PositionCache, slot: int = 0) -> np.ndarray:
        """``attention`` taking the projections' raw rows: the backend normalises and rotates Q and K on the device
        as ``set_layer_prep`` configured, then appends and attends (crates/cpu-compute/src/cpu.rs:592-646 does the
        rotation inside its attention step too)."""
        q, k, v = _host_f32(q).reshape(-1), _host_f32(k).reshape(-1), _host_f32(v).reshape(-1)
        rows = q.size // self.q_width
        out = np.empty(max(q.size, 1), dtype=np.float32)
        sl, ps = (C.c_uint32 * 1)(slot), (C.c_uint64 * 1)(cache.position())
        self._check(self._lib.itk_attention_batch_prep(self._h, layer, 1, sl, ps, rows, _ptr(q), _ptr(k), _ptr(v),
                                                       _ptr(out)))
        return out[: q.size]

    def attention_batch_prep(self, layer: int, slots: Sequence[int], positions: Sequence[int], rows: int, q, k, v
                             ) -> np.ndarray:
        n = len(slots)
        q, k, v = _host_f32(q), _host_f32(k), _host_f32(v)
        out = np.empty(n * rows * self.q_width, dtype=np.float32)
        sl = (C.c_uint32 * n)(*slots)
        ps = (C.c_uint64 * n)(*positions)
        self._check(self._lib.itk_attention_batch_prep(self._h, layer, n, sl, ps, rows, _ptr(q), _ptr(k), _ptr(v),
                                                       _ptr(out)))
        return out

    def attention_batch_prep_ptrs(self, layer: int, slots_c, positions_c, n: int, rows: int, q_ptr: int, k_ptr: int,
                                  v_ptr: int, out_ptr: int):
        """Device-pointer form of ``attention_batch_prep``; only queues work."""
        self._check(self._lib.itk_attention_batch_prep_device(self._h, layer, n, slots_c, positions_c, rows,
                                                              C.c_void_p(q_ptr), C.c_void_p(k_ptr), C.c_void_p(v_ptr),
                                                              C.c_void_p(out_ptr)))

    # -- replayable decode loop ------------------------------------------------------------------
    def resident_begin(self, slots: Sequence[int], max_steps: int):
        """Reserve ``max_steps`` decode steps for ``slots`` and move their positions to device memory; the step's
        launches (``resident_layer`` per layer, then ``resident_advance``) can then be captured once and replayed."""
        n = len(slots)
        sl = (C.c_uint32 * n)(*slots)
        self._check(self._lib.itk_resident_begin(self._h, n, sl, max_steps))

    def resident_layer(self, layer: int, q_ptr: int, k_ptr: int, v_ptr: int, out_ptr: int):
        self._check(self._lib.itk_resident_layer(self._h, layer, C.c_void_p(q_ptr), C.c_void_p(k_ptr), C.c_void_p(v_ptr),
                                                 C.c_void_p(out_ptr)))

    def resident_advance(self):
        self._check(self._lib.itk_resident_advance(self._h))

    def resident_end(self, steps_done: int):
        self._check(self._lib.itk_resident_end(self._h, steps_done))

    # -- gather fused into the decode kernel (multi-GPU) ------------------------------------------
    def gather_create(self, world: int, rank: int, data_bytes: int):
        """Allocate this rank's gather buffer; returns (device pointer of its data, 64-byte handle to send to peers)."""
        ptr = C.c_void_p()
        handle = (C.c_uint8 * 64)()
        self._check(self._lib.itk_gather_create(self._h, world, rank, data_bytes, C.byref(ptr), handle))
        return ptr.value, bytes(handle)

    def gather_open(self, peer_rank: int, handle: bytes):
        buf = (C.c_uint8 * 64).from_buffer_copy(handle)
        self._check(self._lib.itk_gather_open(self._h, peer_rank, buf))

    def gather_attach(self, peer_rank: int, peer_data_ptr: int):
        """Open a peer whose gather buffer this process already addresses (``peer_data_ptr`` = what ``gather_create``
        returned on that peer)."""
        self._check(self._lib.itk_gather_attach(self._h, peer_rank, C.c_void_p(peer_data_ptr)))

    def gather_close_peers(self):
        """Unmap the peers' gather buffers (every rank does this, then the ranks synchronise, then ``close``)."""
        self._check(self._lib.itk_gather_close_peers(self._h))

    def gather_reset(self):
        self._check(self._lib.itk_gather_reset(self._h))

    def gather_status(self) -> int:
        bits = C.c_uint32()
        self._check(self._lib.itk_gather_status(self._h, C.byref(bits)))
        return bits.value

    def resident_layer_gather(self, layer: int, q_ptr: int, k_ptr: int, v_ptr: int, gather_offset_bytes: int):
        self._check(self._lib.itk_resident_layer_gather(self._h, layer, C.c_void_p(q_ptr), C.c_void_p(k_ptr),
                                                        C.c_void_p(v_ptr), gather_offset_bytes))

    def gqa_attention(self, layer: int, q, query_positions: Sequence[int], slot: int = 0) -> np.ndarray:
        """``gqa_attention`` over what the slot already holds; one query row per listed position."""
        q = _host_f32(q).reshape(-1)
        rows = len(query_positions)
        out = np.empty(max(q.size, 1), dtype=np.float32)
        ps = (C.c_uint64 * max(rows, 1))(*query_positions)
        self._check(self._lib.itk_gqa_attention(self._h, slot, layer, _ptr(q), q.size, rows, ps, _ptr(out)))
        return out[: q.size] if rows else np.zeros(0, dtype=np.float32)

    # -- KvCache-level operations -----------------------------------------------------------
    def append(self, layer: int, k, v, position: int, slot: int = 0):
        k, v = _host_f32(k).reshape(-1), _host_f32(v).reshape(-1)
        self._check(self._lib.itk_append(self._h, slot, layer, _ptr(k), k.size, _ptr(v), v.size, position))

    def append_rows(self, layer: int, k, v, start: int, slot: int = 0):
        k = _host_f32(k).reshape(-1, self.kv_width)
        v = _host_f32(v).reshape(-1, self.kv_width)
        assert k.shape == v.shape
        self._check(self._lib.itk_append_rows(self._h, slot, layer, _ptr(k), _ptr(v), k.shape[0], start))

    def append_rows_device(self, layer: int, slots: Sequence[int], starts: Sequence[int], rows: int, k_ptr: int,
                           v_ptr: int):
        """Bulk append from device-resident f32 rows ``[n][rows][Hkv*D]`` (prefill without a host round trip)."""
        n = len(slots)
        sl = (C.c_uint32 * n)(*slots)
        st = (C.c_uint64 * n)(*starts)
        self._check(self._lib.itk_append_rows_device(self._h, layer, n, sl, st, rows, C.c_void_p(k_ptr),
                                                     C.c_void_p(v_ptr)))

    def next_position(self, layer: int, slot: int = 0) -> int:
        out = C.c_uint64()
        self._check(self._lib.itk_next_position(self._h, slot, layer, C.byref(out)))
        return out.value

    def stored_len(self, layer: int, slot: int = 0) -> int:
        out = C.c_uint64()
        self._check(self._lib.itk_stored_len(self._h, slot, layer, C.byref(out)))
        return out.value

    def view(self, layer: int, slot: int = 0):
        """(first_position, keys, values): the visible rows oldest first, ``[rows][Hkv][D]`` in the cache's
        element type (``float32``, or raw ``uint16`` half bits for an f16 cache)."""
        first, rows = C.c_uint64(), C.c_uint64()
        self._check(self._lib.itk_view_gather(self._h, slot, layer, None, None, C.byref(first), C.byref(rows)))
        dt = np.uint16 if self.kv_dtype == KvDtype.F16 else np.float32
        k = np.empty((rows.value, self.kv_heads, self.head_dim), dtype=dt)
        v = np.empty_like(k)
        if rows.value:
            self._check(self._lib.itk_view_gather(self._h, slot, layer, _ptr(k), _ptr(v), C.byref(first), C.byref(rows)))
        return first.value, k, v

    def restore_bulk(self, layer: int, first_position: int, keys, values, slot: int = 0):
        keys, values = _host_f32(keys).reshape(-1), _host_f32(values).reshape(-1)
        self._check(self._lib.itk_restore_bulk(self._h, slot, layer, first_position, _ptr(keys), keys.size,
                                               _ptr(values), values.size))

    def reset(self, slot: int = 0):
        self._check(self._lib.itk_reset(self._h, slot))

    # -- speculation seam ---------------------------------------------------------------------
    def cache_checkpoint(self, max_round_tokens: int, slot: int = 0) -> Checkpoint:
        cp = _lib.Checkpoint()
        self._check(self._lib.itk_cache_checkpoint(self._h, slot, max_round_tokens, C.byref(cp)))
        return Checkpoint(cp.id, cp.serial, cp.base, cp.max_round_tokens)

    def cache_rewind(self, checkpoint: Checkpoint, target: int, slot: int = 0):
        c = checkpoint._c()
        self._check(self._lib.itk_cache_rewind(self._h, slot, C.byref(c), target))

    def cache_release(self, checkpoint: Checkpoint, slot: int = 0):
        c = checkpoint._c()
        self._check(self._lib.itk_cache_release(self._h, slot, C.byref(c)))

    # -- prefix-KV seam --------------------------------------------------------------------------
    def capture_prefix_snapshot(self, slot: int = 0) -> DeviceSnapshot:
        h = C.c_void_p()
        self._check(self._lib.itk_snapshot_capture(self._h, slot, C.byref(h)))
        return DeviceSnapshot(self, h)

    def install_prefix_snapshot(self, snapshot: DeviceSnapshot, slot: int = 0) -> int:
        self._check(self._lib.itk_snapshot_restore(self._h, slot, snapshot._h))
        return snapshot.token_count

    def snapshot_from_itkv(self, data: bytes, expected_fingerprint: Optional[str] = None) -> DeviceSnapshot:
        """Decode ``ITKV`` bytes (strictly), check geometry and fingerprint, and upload the rows."""
        h = C.c_void_p()
        fp = expected_fingerprint.encode() if expected_fingerprint is not None else None
        self._check(self._lib.itk_snapshot_from_itkv(self._h, data, len(data), fp, C.byref(h)))
        return DeviceSnapshot(self, h)

    def snapshot_from_host(self, token_count: int, blocks) -> DeviceSnapshot:
        """Build a device snapshot from f32 layer blocks ``[(first_position, keys, values)]`` laid out like the
        ITKV format's layer blocks; values are cast to the cache's element type as an append would."""
        n = len(blocks)
        firsts = (C.c_uint64 * n)(*[b[0] for b in blocks])
        ks = [_host_f32(b[1]).reshape(-1) for b in blocks]
        vs = [_host_f32(b[2]).reshape(-1) for b in blocks]
        rows = (C.c_uint64 * n)(*[k.size // self.kv_width for k in ks])
        kp = (C.c_void_p * n)(*[k.ctypes.data for k in ks])
        vp = (C.c_void_p * n)(*[v.ctypes.data for v in vs])
        h = C.c_void_p()
        self._check(self._lib.itk_snapshot_from_host_f32(self._h, token_count, firsts, rows, kp, vp, C.byref(h)))
        return DeviceSnapshot(self, h)
