"""ctypes face of the CPU oracle (``kv_oracle.hpp``). TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the bench's CPU-baseline / reference legs
import this module; the shipped package never does.  The wrapper keeps the
reference's vocabulary: ``KvCache.append``, ``view``, ``restore_bulk``,
``checkpoint`` / ``rewind_to`` / ``release``, ``gqa_attention``,
``KvSnapshot.capture`` / ``restore`` / ``to_bytes`` / ``from_bytes``,
``CpuCompute.attention`` and friends, so a test reads like the reference's own.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

# Refusal codes (one per variant of the reference's error enums).
OK = 0
ZERO_DIMENSION = 1
INVALID_WINDOW = 2
SIZE_OVERFLOW = 3
SHAPE_MISMATCH = 4
INVALID_LAYER = 5
OUT_OF_ORDER_POSITION = 6
NON_DIVISIBLE_HEADS = 7
NO_VISIBLE_KEYS = 8
CHECKPOINT_BUSY = 9
STALE_CHECKPOINT = 10
CHECKPOINT_TOO_DEEP = 11
CHECKPOINT_RANGE_EXCEEDED = 12
BULK_RESTORE_NOT_FRESH = 13
REWIND_OUT_OF_RANGE = 14
INCOHERENT_CACHE = 32
INCONSISTENT_SNAPSHOT = 33
BAD_MAGIC = 34
UNSUPPORTED_VERSION = 35
TRUNCATED = 36
CHECKSUM_MISMATCH = 37
GEOMETRY_MISMATCH = 38
FINGERPRINT_MISMATCH = 39
EMPTY_PREFIX = 40  # the prefix store's refusals (crates/itak-kv/src/error.rs), raised by oracle/prefix_store.py by name
TOKEN_COUNT_MISMATCH = 41
PREFIX_HASH_MISMATCH = 42
SNAPSHOT_TOKEN_MISMATCH = 43
ENTRY_TOO_LARGE = 44
INVALID_CONFIG = 45
IO = 46
STEP_FAILED = 64


class OracleError(Exception):
    def __init__(self, code: int, msg: str):
        super().__init__(f"[{code}] {msg}")
        self.code = code
        self.msg = msg


def build(force: bool = False) -> str:
    """Compile ``liboracle.so`` with the Makefile beside this file."""
    src = [os.path.join(_HERE, f) for f in ("oracle_capi.cpp", "kv_oracle.hpp")]
    stale = not os.path.exists(_LIB_PATH) or any(
        os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in src
    )
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


class _Checkpoint(C.Structure):
    _fields_ = [
        ("cache_id", C.c_uint64),
        ("serial", C.c_uint64),
        ("max_round_tokens", C.c_uint64),
        ("saved_bytes", C.c_uint64),
    ]


class _BackendConfig(C.Structure):
    _fields_ = [
        ("sliding", C.POINTER(C.c_int32)),
        ("n_layers", C.c_uint64),
        ("q_heads", C.c_uint64),
        ("kv_heads", C.c_uint64),
        ("key_length", C.c_uint64),
        ("value_length", C.c_uint64),
        ("sliding_window", C.c_uint64),
        ("rope_freq_base_swa", C.c_float),
    ]


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        L.orc_last_error.restype = C.c_char_p
        L.orc_default_scale.restype = C.c_float
        L.orc_default_scale.argtypes = [C.c_size_t]
        for name in ("orc_cache_id", "orc_checksum", "orc_prefix_hash", "orc_prefix_discriminator",
                     "orc_geometry_bytes_per_token", "orc_geometry_stored_bytes_for"):
            getattr(L, name).restype = C.c_uint64
        for name in ("orc_view_len", "orc_view_position_at", "orc_view_window"):
            getattr(L, name).restype = C.c_int64
        for name in ("orc_cache_layer_count", "orc_view_dump", "orc_snapshot_token_count",
                     "orc_snapshot_layer_count", "orc_snapshot_layer_first", "orc_snapshot_layer_floats",
                     "orc_prefix_slot_runs"):
            getattr(L, name).restype = C.c_size_t
        for name in ("orc_snapshot_new", "orc_backend_new", "orc_backend_cache"):
            getattr(L, name).restype = C.c_void_p
        _lib = L
    return _lib


def _check(code: int):
    if code != OK:
        raise OracleError(code, lib().orc_last_error().decode("utf-8", "replace"))


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


def _fp(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _sz(v) -> C.c_size_t:
    # usize::MAX and friends must survive the trip
    return C.c_size_t(int(v) & 0xFFFFFFFFFFFFFFFF)


# --- layer kinds ---------------------------------------------------------------
@dataclass(frozen=True)
class LayerKind:
    windowed: bool = False
    window_size: int = 0

    @staticmethod
    def Global() -> "LayerKind":
        return LayerKind(False, 0)

    @staticmethod
    def Windowed(window: int) -> "LayerKind":
        """Struct-literal construction: no zero check (the cache constructor has one)."""
        return LayerKind(True, int(window))

    @staticmethod
    def windowed_checked(window: int) -> "LayerKind":
        """``LayerKind::windowed``: refuses a zero window by name."""
        if window == 0:
            raise OracleError(INVALID_WINDOW, "sliding window must be positive, got 0")
        return LayerKind(True, int(window))

    def window(self) -> Optional[int]:
        return self.window_size if self.windowed else None


GLOBAL = LayerKind.Global()


def glimmer_layer_pattern():
    return [GLOBAL if i % 4 == 3 else LayerKind.Windowed(2048) for i in range(52)]


def _pattern_arrays(pattern: Sequence[LayerKind]):
    n = len(pattern)
    w = (C.c_int32 * max(n, 1))(*[1 if k.windowed else 0 for k in pattern])
    s = (C.c_uint64 * max(n, 1))(*[(k.window_size & 0xFFFFFFFFFFFFFFFF) if k.windowed else 0 for k in pattern])
    return w, s, n


# --- conversions -----------------------------------------------------------------
def f32_to_f16_bits(x) -> np.ndarray:
    a = _f32(x).reshape(-1)
    out = np.empty(a.size, dtype=np.uint16)
    lib().orc_f32_to_f16_bits(_fp(a), out.ctypes.data_as(C.POINTER(C.c_uint16)), _sz(a.size))
    return out.reshape(np.shape(x))


def f16_bits_to_f32(bits) -> np.ndarray:
    a = np.ascontiguousarray(np.asarray(bits, dtype=np.uint16)).reshape(-1)
    out = np.empty(a.size, dtype=np.float32)
    lib().orc_f16_bits_to_f32(a.ctypes.data_as(C.POINTER(C.c_uint16)), _fp(out), _sz(a.size))
    return out.reshape(np.shape(bits))


def round_through_f16(x) -> np.ndarray:
    a = _f32(x)
    out = np.empty_like(a)
    lib().orc_round_through_f16(_fp(a.reshape(-1)), _fp(out.reshape(-1)), _sz(a.size))
    return out


def rope_interleaved(x, position: int, base: float, head_dim: int, rotary_dim: Optional[int] = None) -> np.ndarray:
    a = _f32(x)
    out = np.empty(max(head_dim, 1), dtype=np.float32)
    _check(lib().orc_rope(0, _fp(a), _sz(a.size), _sz(position), C.c_float(base), _sz(head_dim),
                          _sz(head_dim if rotary_dim is None else rotary_dim), _fp(out)))
    return out[:head_dim]


def rope(x, position: int, base: float, head_dim: int, rotary_dim: Optional[int] = None) -> np.ndarray:
    a = _f32(x)
    out = np.empty(max(head_dim, 1), dtype=np.float32)
    _check(lib().orc_rope(1, _fp(a), _sz(a.size), _sz(position), C.c_float(base), _sz(head_dim),
                          _sz(head_dim if rotary_dim is None else rotary_dim), _fp(out)))
    return out[:head_dim]


def rope_rows(x, heads: int, head_dim: int, start_position: int, base: float, pairing: int = 0) -> np.ndarray:
    """Rotate ``[rows][heads][head_dim]`` at positions start, start+1, ..."""
    a = _f32(x).reshape(-1, heads, head_dim)
    out = np.empty_like(a)
    _check(lib().orc_rope_rows(pairing, _fp(a), _sz(a.shape[0]), _sz(heads), _sz(head_dim), _sz(start_position),
                               C.c_float(base), _fp(out)))
    return out


def rms_norm(x, weight, eps: float) -> np.ndarray:
    """torch_math::rms_norm (crates/torch-math/src/norm.rs:21-53) over one row."""
    a, w = _f32(x).reshape(-1), _f32(weight).reshape(-1)
    out = np.empty(max(a.size, 1), dtype=np.float32)
    _check(lib().orc_rms_norm(_fp(a), _sz(a.size), _fp(w), _sz(w.size), C.c_float(eps), _fp(out)))
    return out[:a.size]


def prepare_rows(x, heads: int, head_dim: int, start_position: int, weight=None, eps: float = 1e-6,
                 rope_base: Optional[float] = None, rotary_dim: Optional[int] = None, pairing: int = 0) -> np.ndarray:
    """The attention preparation of ``[rows][heads][head_dim]`` rows as the reference composes it: per-head
    rms_norm (when a weight is given), then the rotation of each head row at its position (when a base is given;
    crates/wgpu-compute/src/kernels/k9_attn_prep.rs:1-40 states the composition, the CPU functions do the math)."""
    a = _f32(x).reshape(-1, heads, head_dim).copy()
    for r in range(a.shape[0]):
        for h in range(heads):
            row = a[r, h]
            if weight is not None:
                row = rms_norm(row, weight, eps)
            if rope_base is not None:
                fn = rope_interleaved if pairing == 0 else rope
                row = fn(row, start_position + r, rope_base, head_dim, rotary_dim)
            a[r, h] = row
    return a


def draft_attention(q, positions, committed_positions, committed_k, committed_v, block_k, block_v, q_heads: int,
                    kv_heads: int, key_len: int, value_len: int, causal: bool = False, sliding: bool = False,
                    window: int = 0) -> np.ndarray:
    """The draft model's attention over committed + block rows (crates/dflash/src/model.rs:388-466).
    ``committed_k`` / ``committed_v`` are compact ``[committed][kv_heads*len]`` in the order of
    ``committed_positions``; returns ``[rows][q_heads*value_len]``."""
    q = _f32(q).reshape(-1)
    rows = len(positions)
    ck, cv = _f32(committed_k).reshape(-1), _f32(committed_v).reshape(-1)
    bk, bv = _f32(block_k).reshape(-1), _f32(block_v).reshape(-1)
    pos = np.ascontiguousarray(positions, dtype=np.uint64)
    cpos = np.ascontiguousarray(committed_positions, dtype=np.uint64)
    out = np.zeros(max(rows * q_heads * value_len, 1), dtype=np.float32)
    u64p = C.POINTER(C.c_uint64)
    _check(lib().orc_draft_attention(_fp(q), _sz(rows), _sz(q_heads), _sz(kv_heads), _sz(key_len), _sz(value_len),
                                     pos.ctypes.data_as(u64p), cpos.ctypes.data_as(u64p), _sz(len(cpos)), _fp(ck), _fp(cv),
                                     _fp(bk), _fp(bv), int(causal), int(sliding), C.c_uint64(window), _fp(out)))
    return out[: rows * q_heads * value_len].reshape(rows, q_heads * value_len)


def default_scale(head_dim: int) -> float:
    return float(lib().orc_default_scale(_sz(head_dim)))


def kv_head_for_query_head(q_head: int, num_q_heads: int, num_kv_heads: int) -> int:
    out = C.c_size_t()
    _check(lib().orc_kv_head_for_query_head(_sz(q_head), _sz(num_q_heads), _sz(num_kv_heads), C.byref(out)))
    return out.value


# --- hashes ----------------------------------------------------------------------
def checksum(data: bytes) -> int:
    return lib().orc_checksum(data, _sz(len(data)))


def prefix_hash(tokens) -> int:
    a = np.ascontiguousarray(np.asarray(tokens, dtype=np.uint32))
    return lib().orc_prefix_hash(a.ctypes.data_as(C.POINTER(C.c_uint32)), _sz(a.size))


def prefix_discriminator(tokens) -> int:
    a = np.ascontiguousarray(np.asarray(tokens, dtype=np.uint32))
    return lib().orc_prefix_discriminator(a.ctypes.data_as(C.POINTER(C.c_uint32)), _sz(a.size))


# --- cache -------------------------------------------------------------------------
@dataclass
class Checkpoint:
    cache_id: int
    serial: int
    max_round_tokens_: int
    saved_bytes_: int
    bases_: list

    def base(self, layer: int) -> Optional[int]:
        return self.bases_[layer] if 0 <= layer < len(self.bases_) else None

    def bases(self):
        return list(self.bases_)

    def max_round_tokens(self) -> int:
        return self.max_round_tokens_

    def saved_bytes(self) -> int:
        return self.saved_bytes_

    def _c(self) -> _Checkpoint:
        return _Checkpoint(self.cache_id, self.serial, self.max_round_tokens_, self.saved_bytes_)


@dataclass
class LayerStats:
    layer: int
    appended: int
    stored: int


class CacheView:
    def __init__(self, cache: "KvCache", layer: int):
        self._c = cache
        self._layer = layer

    def __len__(self) -> int:
        return int(lib().orc_view_len(self._c._h, _sz(self._layer)))

    def len(self) -> int:
        return len(self)

    def is_empty(self) -> bool:
        return len(self) == 0

    def window(self) -> Optional[int]:
        w = lib().orc_view_window(self._c._h, _sz(self._layer))
        return None if w < 0 else int(w)

    def num_kv_heads(self) -> int:
        return self._c.num_kv_heads

    def head_dim(self) -> int:
        return self._c.head_dim

    def position_at(self, vi: int) -> Optional[int]:
        p = lib().orc_view_position_at(self._c._h, _sz(self._layer), _sz(vi))
        return None if p < 0 else int(p)

    def key(self, vi: int, head: int) -> Optional[np.ndarray]:
        out = np.empty(self._c.head_dim, dtype=np.float32)
        ok = lib().orc_view_key(self._c._h, _sz(self._layer), _sz(vi), _sz(head), _fp(out))
        return out if ok else None

    def value(self, vi: int, head: int) -> Optional[np.ndarray]:
        out = np.empty(self._c.head_dim, dtype=np.float32)
        ok = lib().orc_view_value(self._c._h, _sz(self._layer), _sz(vi), _sz(head), _fp(out))
        return out if ok else None

    def dump(self):
        """(positions, keys[visible][Hkv][D], values[visible][Hkv][D]) oldest first."""
        n = len(self)
        shape = (n, self._c.num_kv_heads, self._c.head_dim)
        k = np.empty(shape, dtype=np.float32)
        v = np.empty(shape, dtype=np.float32)
        if n:
            lib().orc_view_dump(self._c._h, _sz(self._layer), _fp(k), _fp(v))
        pos = [self.position_at(i) for i in range(n)]
        return pos, k, v


class KvCache:
    def __init__(self, pattern: Sequence[LayerKind], num_kv_heads: int, head_dim: int, _handle=None, _owned=True):
        self._owned = _owned
        self.pattern = list(pattern)
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        if _handle is not None:
            self._h = C.c_void_p(_handle)
            return
        w, s, n = _pattern_arrays(pattern)
        h = C.c_void_p()
        self._h = None
        _check(lib().orc_cache_new(w, s, _sz(n), _sz(num_kv_heads), _sz(head_dim), C.byref(h)))
        self._h = h

    def __del__(self):
        if getattr(self, "_h", None) is not None and self._owned:
            lib().orc_cache_free(self._h)
            self._h = None

    def id(self) -> int:
        return lib().orc_cache_id(self._h)

    def layer_count(self) -> int:
        return lib().orc_cache_layer_count(self._h)

    def layer_kind(self, layer: int) -> LayerKind:
        w, s = C.c_int32(), C.c_uint64()
        _check(lib().orc_cache_layer_kind(self._h, _sz(layer), C.byref(w), C.byref(s)))
        return LayerKind(bool(w.value), s.value)

    def append(self, layer: int, k, v, position: int):
        k, v = _f32(k).reshape(-1), _f32(v).reshape(-1)
        _check(lib().orc_cache_append(self._h, _sz(layer), _fp(k), _sz(k.size), _fp(v), _sz(v.size), _sz(position)))

    def append_rows(self, layer: int, k, v, start: int):
        """Append consecutive positions start.. from ``[rows][Hkv*D]`` arrays."""
        row = self.num_kv_heads * self.head_dim
        k, v = _f32(k).reshape(-1, row), _f32(v).reshape(-1, row)
        _check(lib().orc_cache_append_rows(self._h, _sz(layer), _fp(k), _fp(v), _sz(k.shape[0]), _sz(start)))

    def restore_bulk(self, layer: int, first_position: int, keys, values):
        keys, values = _f32(keys).reshape(-1), _f32(values).reshape(-1)
        _check(lib().orc_cache_restore_bulk(self._h, _sz(layer), _sz(first_position), _fp(keys), _sz(keys.size),
                                            _fp(values), _sz(values.size)))

    def stored_len(self, layer: int) -> int:
        out = C.c_size_t()
        _check(lib().orc_cache_stored_len(self._h, _sz(layer), C.byref(out)))
        return out.value

    def next_position(self, layer: int) -> int:
        out = C.c_size_t()
        _check(lib().orc_cache_next_position(self._h, _sz(layer), C.byref(out)))
        return out.value

    def view(self, layer: int) -> CacheView:
        if not 0 <= layer < self.layer_count():
            raise OracleError(INVALID_LAYER, f"layer {layer} out of range, cache has {self.layer_count()} layers")
        return CacheView(self, layer)

    def stats(self):
        n = self.layer_count()
        a = (C.c_uint64 * n)()
        s = (C.c_uint64 * n)()
        lib().orc_cache_stats(self._h, a, s)
        return [LayerStats(i, a[i], s[i]) for i in range(n)]

    def checkpoint_active(self) -> bool:
        return bool(lib().orc_cache_checkpoint_active(self._h))

    def checkpoint(self, max_round_tokens: int) -> Checkpoint:
        n = self.layer_count()
        cp = _Checkpoint()
        bases = (C.c_uint64 * n)()
        _check(lib().orc_cache_checkpoint(self._h, _sz(max_round_tokens), C.byref(cp), bases))
        return Checkpoint(cp.cache_id, cp.serial, cp.max_round_tokens, cp.saved_bytes, list(bases))

    def rewind_to(self, cp: Checkpoint, target: int):
        c = cp._c()
        _check(lib().orc_cache_rewind(self._h, C.byref(c), _sz(target)))

    def release(self, cp: Checkpoint):
        c = cp._c()
        _check(lib().orc_cache_release(self._h, C.byref(c)))


def gqa_attention(q, num_queries: int, num_q_heads: int, query_positions, view: CacheView,
                  scale: Optional[float] = None) -> np.ndarray:
    q = _f32(q).reshape(-1)
    pos = (C.c_uint64 * max(len(query_positions), 1))(*query_positions)
    out = np.zeros(max(q.size, 1), dtype=np.float32)
    _check(lib().orc_gqa_attention(view._c._h, _sz(view._layer), _fp(q), _sz(q.size), _sz(num_queries),
                                   _sz(num_q_heads), pos, _sz(len(query_positions)),
                                   0 if scale is None else 1, C.c_float(0.0 if scale is None else scale), _fp(out)))
    if num_queries == 0:
        return np.zeros(0, dtype=np.float32)
    return out[: q.size]


def attention_units(caches: Sequence[KvCache], layers, q: np.ndarray, positions, num_q_heads: int, threads: int):
    """One single-query attention per unit over ``threads`` host threads.

    Returns (outputs ``[units][Hq*D]``, wall seconds)."""
    n = len(caches)
    q = _f32(q).reshape(n, -1)
    out = np.zeros_like(q)
    hs = (C.c_void_p * n)(*[c._h.value for c in caches])
    ls = (C.c_uint64 * n)(*layers)
    ps = (C.c_uint64 * n)(*positions)
    secs = C.c_double()
    _check(lib().orc_attention_units(_sz(n), hs, ls, _fp(q), _sz(q.shape[1]), ps, _sz(num_q_heads), _sz(threads),
                                     _fp(out), C.byref(secs)))
    return out, secs.value


# --- snapshots ---------------------------------------------------------------------
@dataclass
class KvGeometry:
    layers: list
    num_kv_heads: int
    head_dim: int

    def row_floats(self) -> int:
        return self.num_kv_heads * self.head_dim

    def bytes_per_token(self) -> int:
        w, s, n = _pattern_arrays(self.layers)
        return lib().orc_geometry_bytes_per_token(w, s, _sz(n), _sz(self.num_kv_heads), _sz(self.head_dim))

    def stored_bytes_for(self, tokens: int) -> int:
        w, s, n = _pattern_arrays(self.layers)
        return lib().orc_geometry_stored_bytes_for(w, s, _sz(n), _sz(self.num_kv_heads), _sz(self.head_dim),
                                                   _sz(tokens))


class KvSnapshot:
    def __init__(self, handle, geometry: Optional[KvGeometry] = None):
        self._h = C.c_void_p(handle) if not isinstance(handle, C.c_void_p) else handle
        self.geometry = geometry

    def __del__(self):
        if getattr(self, "_h", None) is not None:
            lib().orc_snapshot_free(self._h)
            self._h = None

    @staticmethod
    def capture(cache: KvCache, fingerprint: str) -> "KvSnapshot":
        h = C.c_void_p()
        _check(lib().orc_snapshot_capture(cache._h, fingerprint.encode(), C.byref(h)))
        return KvSnapshot(h, KvGeometry(list(cache.pattern), cache.num_kv_heads, cache.head_dim))

    @staticmethod
    def build(geometry: KvGeometry, fingerprint: str, token_count: int, blocks) -> "KvSnapshot":
        """A snapshot value from public fields; ``blocks`` = [(first_position, keys, values)]."""
        w, s, n = _pattern_arrays(geometry.layers)
        h = lib().orc_snapshot_new(w, s, _sz(n), _sz(geometry.num_kv_heads), _sz(geometry.head_dim),
                                   fingerprint.encode(), _sz(token_count), _sz(len(blocks)))
        snap = KvSnapshot(h, geometry)
        for i, (first, keys, values) in enumerate(blocks):
            snap.set_layer(i, first, keys, values)
        return snap

    def set_layer(self, layer: int, first_position: int, keys, values):
        keys, values = _f32(keys).reshape(-1), _f32(values).reshape(-1)
        lib().orc_snapshot_set_layer(self._h, _sz(layer), _sz(first_position), _fp(keys), _sz(keys.size),
                                     _fp(values), _sz(values.size))

    def validate(self):
        _check(lib().orc_snapshot_validate(self._h))

    @property
    def token_count(self) -> int:
        return lib().orc_snapshot_token_count(self._h)

    def layer_count(self) -> int:
        return lib().orc_snapshot_layer_count(self._h)

    def layer(self, i: int):
        """(first_position, keys, values) of one layer block, flat f32."""
        n = lib().orc_snapshot_layer_floats(self._h, _sz(i))
        k = np.empty(n, dtype=np.float32)
        v = np.empty(n, dtype=np.float32)
        lib().orc_snapshot_layer_copy(self._h, _sz(i), _fp(k), _fp(v))
        return lib().orc_snapshot_layer_first(self._h, _sz(i)), k, v

    def __eq__(self, other) -> bool:
        return bool(lib().orc_snapshot_equal(self._h, other._h))

    def restore(self) -> KvCache:
        h = C.c_void_p()
        _check(lib().orc_snapshot_restore(self._h, C.byref(h)))
        g = self.geometry
        return KvCache(g.layers, g.num_kv_heads, g.head_dim, _handle=h.value)

    def restore_checked(self, geometry: KvGeometry, fingerprint: str) -> KvCache:
        w, s, n = _pattern_arrays(geometry.layers)
        h = C.c_void_p()
        _check(lib().orc_snapshot_restore_checked(self._h, w, s, _sz(n), _sz(geometry.num_kv_heads),
                                                  _sz(geometry.head_dim), fingerprint.encode(), C.byref(h)))
        return KvCache(geometry.layers, geometry.num_kv_heads, geometry.head_dim, _handle=h.value)

    def to_bytes(self) -> bytes:
        size = C.c_size_t()
        _check(lib().orc_snapshot_to_bytes(self._h, None, _sz(0), C.byref(size)))
        buf = (C.c_uint8 * size.value)()
        _check(lib().orc_snapshot_to_bytes(self._h, buf, _sz(size.value), C.byref(size)))
        return bytes(buf)

    @staticmethod
    def from_bytes(data: bytes, geometry: Optional[KvGeometry] = None) -> "KvSnapshot":
        h = C.c_void_p()
        _check(lib().orc_snapshot_from_bytes(data, _sz(len(data)), C.byref(h)))
        return KvSnapshot(h, geometry)


# --- slot/ring laws -------------------------------------------------------------------
def prefix_visible_range(sliding: bool, window: int, position: int):
    f, r = C.c_size_t(), C.c_size_t()
    lib().orc_prefix_visible_range(1 if sliding else 0, _sz(window), _sz(position), C.byref(f), C.byref(r))
    return f.value, r.value


def prefix_slot_runs(sliding: bool, first_position: int, rows: int, ring: int):
    cap = 8
    buf = (C.c_uint64 * (3 * cap))()
    n = lib().orc_prefix_slot_runs(1 if sliding else 0, _sz(first_position), _sz(rows), _sz(ring), buf, _sz(cap))
    return [(buf[3 * i], buf[3 * i + 1], buf[3 * i + 2]) for i in range(min(n, cap))], n


# --- CPU backend step --------------------------------------------------------------------
@dataclass
class BackendConfig:
    sliding: list  # per layer: True = sliding-window layer
    q_heads: int
    kv_heads: int
    key_length: int
    value_length: int
    sliding_window: int
    rope_freq_base_swa: float = 10000.0

    def _c(self):
        n = len(self.sliding)
        arr = (C.c_int32 * max(n, 1))(*[1 if s else 0 for s in self.sliding])
        cfg = _BackendConfig(C.cast(arr, C.POINTER(C.c_int32)), n, self.q_heads, self.kv_heads, self.key_length,
                             self.value_length, self.sliding_window, self.rope_freq_base_swa)
        cfg._keep = arr
        return cfg


class PositionCache:
    """The position contract of the forward loop (``Cache`` trait)."""

    def __init__(self):
        self._p = 0

    def position(self) -> int:
        return self._p

    def advance(self, tokens: int):
        self._p += tokens

    def rewind_to(self, position: int):
        self._p = position


class CpuCompute:
    """The CPU backend's attention step and speculation seam."""

    def __init__(self):
        self._h = C.c_void_p(lib().orc_backend_new())

    def __del__(self):
        if getattr(self, "_h", None) is not None:
            lib().orc_backend_free(self._h)
            self._h = None

    def reset(self):
        lib().orc_backend_reset(self._h)

    def kv_cache(self, cfg: BackendConfig) -> Optional[KvCache]:
        h = lib().orc_backend_cache(self._h)
        if not h:
            return None
        pattern = [LayerKind.Windowed(cfg.sliding_window) if s else GLOBAL for s in cfg.sliding]
        return KvCache(pattern, cfg.kv_heads, cfg.key_length, _handle=h, _owned=False)

    def attention(self, cfg: BackendConfig, layer: int, sliding: bool, q, k, v, cache: PositionCache) -> np.ndarray:
        q, k, v = _f32(q).reshape(-1), _f32(k).reshape(-1), _f32(v).reshape(-1)
        out = np.zeros(max(q.size, 1), dtype=np.float32)
        c = cfg._c()
        _check(lib().orc_backend_attention(self._h, C.byref(c), _sz(layer), 1 if sliding else 0, _fp(q), _sz(q.size),
                                           _fp(k), _sz(k.size), _fp(v), _sz(v.size), _sz(cache.position()),
                                           _fp(out)))
        return out[: q.size]

    def cache_checkpoint(self, max_round_tokens: int, n_layers: int = 64) -> Checkpoint:
        cp = _Checkpoint()
        bases = (C.c_uint64 * 4096)()
        _check(lib().orc_backend_checkpoint(self._h, _sz(max_round_tokens), C.byref(cp), bases))
        cache_h = lib().orc_backend_cache(self._h)
        n = lib().orc_cache_layer_count(C.c_void_p(cache_h))
        return Checkpoint(cp.cache_id, cp.serial, cp.max_round_tokens, cp.saved_bytes, list(bases[:n]))

    def cache_rewind(self, cp: Checkpoint, target: int):
        c = cp._c()
        _check(lib().orc_backend_rewind(self._h, C.byref(c), _sz(target)))

    def cache_release(self, cp: Checkpoint):
        c = cp._c()
        _check(lib().orc_backend_release(self._h, C.byref(c)))


# --- deterministic generators used by the reference's fixtures ---------------------------
def lcg(seed: int, count: int) -> np.ndarray:
    """f32 in [-0.5, 0.5): state = max(seed, 1); state = state*A + C; (state >> 40) / 2^24 - 0.5.

    The generator of crates/wgpu-compute/tests/fused_kernels.rs:45-55 and
    crates/itak-kv/tests/restore_fixture.rs:22-30.
    """
    out = np.empty(count, dtype=np.float32)
    lib().orc_lcg(C.c_uint64(seed & 0xFFFFFFFFFFFFFFFF), _sz(count), _fp(out))
    return out
