"""CPU restatement of the reference's persistent prefix store (crates/itak-kv/src/store.rs) for the parity tests:
entry encoding, file naming, trust checks of a lookup, last-used stamping and LRU eviction, in plain Python over the
oracle's snapshot codec.  Test infrastructure only: nothing in the product imports it."""
from __future__ import annotations

import os
import struct
from typing import List, Optional, Sequence, Tuple

from . import oracle as orc

ENTRY_MAGIC = b"ITKVPENT"  # store.rs:63
ENTRY_FORMAT_VERSION = 1   # store.rs:65
PREAMBLE_LEN = 72          # store.rs:67
LAST_USED_OFFSET = 24      # store.rs:69


class StoreRefusal(Exception):
    def __init__(self, kind: str, text: str):
        super().__init__(text)
        self.kind = kind


def encode_preamble(created: int, last_used: int, prefix_hash: int, token_count: int, payload_bytes: int) -> bytes:
    """store.rs:556-567"""
    return (ENTRY_MAGIC + struct.pack("<II", ENTRY_FORMAT_VERSION, 0) +
            struct.pack("<QQQQQQQ", created, last_used, prefix_hash, token_count, token_count * 4, payload_bytes, 0))


def parse_preamble(data: bytes) -> Tuple[int, int, int, int, int]:
    """store.rs:569-609 -> (created, last_used, prefix_hash, token_count, payload_bytes)"""
    if len(data) < PREAMBLE_LEN:
        raise StoreRefusal("Truncated", f"entry: truncated, needs {PREAMBLE_LEN} bytes, has {len(data)}")
    if data[:8] != ENTRY_MAGIC:
        raise StoreRefusal("BadMagic", "entry: bad magic")
    (version,) = struct.unpack_from("<I", data, 8)
    if version != ENTRY_FORMAT_VERSION:
        raise StoreRefusal("UnsupportedVersion", f"entry: unsupported format version {version}")
    created, last_used, key, count, tokens_bytes, payload = struct.unpack_from("<QQQQQQ", data, 16)
    expected = min(count * 4, 2 ** 64 - 1)
    if tokens_bytes != expected:
        raise StoreRefusal("InconsistentSnapshot", f"inconsistent snapshot: entry tokens_bytes is {tokens_bytes} but token "
                                                   f"count {count} implies {expected}")
    return created, last_used, key, count, payload


def entry_bytes(tokens: Sequence[int], payload: bytes, now: int) -> bytes:
    """What PrefixStore::put writes (store.rs:262-283)."""
    key = orc.prefix_hash(tokens)
    return (encode_preamble(now, now, key, len(tokens), len(payload)) +
            b"".join(struct.pack("<I", t) for t in tokens) + payload)


def file_name_for(tokens: Sequence[int], counter: int = 0) -> str:
    """store.rs:459-468"""
    base = f"{orc.prefix_hash(tokens):016x}-{len(tokens)}-{orc.prefix_discriminator(tokens):016x}"
    return base + (".kv" if counter == 0 else f"-c{counter}.kv")


class PrefixStore:
    """The index and policy of store.rs:128-546 over a directory."""

    def __init__(self, root: str, max_bytes: int):
        if max_bytes == 0:
            raise StoreRefusal("InvalidConfig", "invalid config: the store byte cap is zero")
        os.makedirs(root, exist_ok=True)
        self.root, self.max_bytes = root, max_bytes
        self.entries: List[dict] = []
        self.rescan()

    def rescan(self):
        found = []
        for name in os.listdir(self.root):
            if name.startswith(".tmp-") or not name.endswith(".kv"):
                continue
            path = os.path.join(self.root, name)
            try:
                with open(path, "rb") as f:
                    head = f.read(PREAMBLE_LEN)
                created, last_used, key, count, _ = parse_preamble(head)
            except StoreRefusal:
                continue
            found.append({"file_name": name, "prefix_hash": key, "token_count": count, "bytes": os.path.getsize(path),
                          "created_unix": created, "last_used_unix": last_used})
        self.entries = found

    def total_bytes(self) -> int:
        return sum(e["bytes"] for e in self.entries)

    def sorted_entries(self) -> List[dict]:
        return sorted(self.entries, key=lambda e: -e["token_count"])

    def put(self, tokens: Sequence[int], snapshot: "orc.KvSnapshot", now: int):
        if len(tokens) == 0:
            raise StoreRefusal("EmptyPrefix", "empty token prefix refused")
        if snapshot.token_count != len(tokens):
            raise StoreRefusal("TokenCountMismatch", f"snapshot covers {snapshot.token_count} tokens but was offered under "
                                                     f"{len(tokens)} token ids")
        data = entry_bytes(tokens, snapshot.to_bytes(), now)
        if len(data) > self.max_bytes:
            raise StoreRefusal("EntryTooLarge", f"entry of {len(data)} bytes exceeds the store cap of {self.max_bytes} bytes")
        name = file_name_for(tokens)  # (the collision counter is exercised by the product's own test)
        with open(os.path.join(self.root, name), "wb") as f:
            f.write(data)
        self.entries = [e for e in self.entries if e["file_name"] != name]
        self.entries.append({"file_name": name, "prefix_hash": orc.prefix_hash(tokens), "token_count": len(tokens),
                             "bytes": len(data), "created_unix": now, "last_used_unix": now})
        while self.total_bytes() > self.max_bytes:  # store.rs:518-546
            victims = [e for e in self.entries if e["file_name"] != name]
            if not victims:
                break
            v = min(victims, key=lambda e: (e["last_used_unix"], e["file_name"]))
            os.remove(os.path.join(self.root, v["file_name"]))
            self.entries = [e for e in self.entries if e["file_name"] != v["file_name"]]

    def lookup(self, query: Sequence[int], now: int) -> Optional[Tuple[int, bytes]]:
        """store.rs:314-452 without the optional geometry / fingerprint requirements -> (token_count, payload)."""
        for cand in [e for e in self.sorted_entries() if e["token_count"] <= len(query)]:
            path = os.path.join(self.root, cand["file_name"])
            data = open(path, "rb").read()
            try:
                _, _, key, count, payload_len = parse_preamble(data)
                end = PREAMBLE_LEN + count * 4
                if len(data) < end:
                    continue
                tokens = list(struct.unpack_from(f"<{count}I", data, PREAMBLE_LEN))
                if orc.prefix_hash(tokens) != key:
                    continue
                if tokens != list(query[:count]):
                    continue
                payload = data[end:]
                if len(payload) != payload_len:
                    continue
                snap = orc.KvSnapshot.from_bytes(payload)
                if snap.token_count != count:
                    continue
            except (StoreRefusal, orc.OracleError):
                continue
            with open(path, "r+b") as f:
                f.seek(LAST_USED_OFFSET)
                f.write(struct.pack("<Q", now))
            cand["last_used_unix"] = now
            return count, payload
        return None
