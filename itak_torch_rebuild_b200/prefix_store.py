"""Python mirror of the persistent prefix store (``crates/itak-kv/src/store.rs``): the same method names over the
C ABI's ``itk_prefix_store_*`` entry points.  Entries carry ITKV snapshot bytes (``DeviceSnapshot.to_itkv`` /
``CudaCompute.snapshot_from_itkv``)."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Sequence

from . import _lib
from .backend import CudaComputeError


@dataclass
class EntryMeta:
    """store.rs:72-87"""
    file_name: str
    prefix_hash: int
    token_count: int
    bytes: int
    created_unix: int
    last_used_unix: int


@dataclass
class PrefixHit:
    """store.rs:89-102, with the snapshot as its ITKV bytes."""
    token_count: int
    tokens: List[int]
    snapshot_bytes: bytes


class PrefixStore:
    def __init__(self, root: str, max_bytes: int):
        """PrefixStore::open (store.rs:147-170)."""
        self._lib = _lib.load()
        self._h = None
        h = C.c_void_p()
        rc = self._lib.itk_prefix_store_open(str(root).encode(), max_bytes, C.byref(h))
        if rc != _lib.OK:
            raise CudaComputeError(rc, self._lib.itk_prefix_store_last_error(None).decode("utf-8", "replace"))
        self._h = h

    def close(self):
        if self._h is not None:
            self._lib.itk_prefix_store_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int):
        if rc != _lib.OK:
            raise CudaComputeError(rc, self._lib.itk_prefix_store_last_error(self._h).decode("utf-8", "replace"))

    @property
    def last_refusal(self) -> str:
        """The last entry refused by name (the reference writes this line to its diag log)."""
        return self._lib.itk_prefix_store_last_refusal(self._h).decode("utf-8", "replace")

    def rescan(self):
        self._check(self._lib.itk_prefix_store_rescan(self._h))

    def put(self, tokens: Sequence[int], snapshot_bytes: bytes, now: int):
        n = len(tokens)
        ids = (C.c_uint32 * max(n, 1))(*tokens)
        buf = (C.c_uint8 * max(len(snapshot_bytes), 1)).from_buffer_copy(snapshot_bytes or b"\0")
        self._check(self._lib.itk_prefix_store_put(self._h, ids, n, C.cast(buf, C.c_void_p), len(snapshot_bytes), now))

    def lookup(self, query: Sequence[int], expected_geometry=None, expected_fingerprint: Optional[str] = None,
               now: int = 0) -> Optional[PrefixHit]:
        """``expected_geometry``: ``(layer_windows, kv_heads, head_dim)`` with 0 for a global layer, or None."""
        n = len(query)
        ids = (C.c_uint32 * max(n, 1))(*query)
        cfg_ref, keep = None, None
        if expected_geometry is not None:
            windows, hkv, d = expected_geometry
            keep = (C.c_uint32 * max(len(windows), 1))(*windows)
            cfg = _lib.Config(len(windows), C.cast(keep, C.POINTER(C.c_uint32)), hkv, hkv, d, 1, 1, 1, 0, 0)
            cfg_ref = C.byref(cfg)
        count, ptr, size = C.c_uint64(), C.c_void_p(), C.c_size_t()
        fp = expected_fingerprint.encode() if expected_fingerprint is not None else None
        self._check(self._lib.itk_prefix_store_lookup(self._h, ids, n, cfg_ref, fp, now, C.byref(count), C.byref(ptr),
                                                      C.byref(size)))
        if count.value == 0:
            return None
        data = C.string_at(ptr.value, size.value)
        return PrefixHit(count.value, list(query[: count.value]), data)

    def stats(self) -> dict:
        e, t, m = C.c_uint64(), C.c_uint64(), C.c_uint64()
        self._check(self._lib.itk_prefix_store_stats(self._h, C.byref(e), C.byref(t), C.byref(m)))
        return {"entries": e.value, "total_bytes": t.value, "max_bytes": m.value}

    def entries(self) -> List[EntryMeta]:
        """Indexed entries, longest prefix first."""
        out = []
        for i in range(self.stats()["entries"]):
            name = C.create_string_buffer(256)
            h, n, b, c, u = (C.c_uint64() for _ in range(5))
            self._check(self._lib.itk_prefix_store_entry(self._h, i, name, 256, C.byref(h), C.byref(n), C.byref(b),
                                                         C.byref(c), C.byref(u)))
            out.append(EntryMeta(name.value.decode(), h.value, n.value, b.value, c.value, u.value))
        return out


def check_itkv(data: bytes):
    """Strictly decode ITKV bytes on the host (no device): returns (version, token_count, bytes per stored element)
    or raises the named refusal."""
    lib = _lib.load()
    version, tokens, elem = C.c_uint32(), C.c_uint64(), C.c_uint32()
    why = C.create_string_buffer(512)
    rc = lib.itk_itkv_check(data, len(data), C.byref(version), C.byref(tokens), C.byref(elem), why, len(why))
    if rc != _lib.OK:
        raise CudaComputeError(rc, why.value.decode("utf-8", "replace"))
    return version.value, tokens.value, elem.value
