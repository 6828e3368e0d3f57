"""The persistent prefix store (C ABI itk_prefix_store_*, host code only) against the reference's own store tests
(crates/itak-kv/src/store.rs:655-810) and, byte for byte, against the oracle's restatement of its entry format
(oracle/prefix_store.py).  Snapshots are the oracle's ITKV bytes, the same bytes the device codec writes
(tests/test_gpu_snapshot.py::test_itkv_* pin that equality), so no GPU is needed here."""
import os
import struct

import numpy as np
import pytest

from itak_torch_rebuild_b200 import CudaComputeError, _lib
from itak_torch_rebuild_b200.prefix_store import PrefixStore
from oracle import oracle as orc
from oracle import prefix_store as ops

GEOMETRY = orc.KvGeometry([orc.LayerKind.Windowed(4), orc.GLOBAL], 2, 3)  # store.rs:666-672


def snapshot_for(tokens, fingerprint):
    """store.rs:674-691"""
    cache = orc.KvCache(GEOMETRY.layers, GEOMETRY.num_kv_heads, GEOMETRY.head_dim)
    row = GEOMETRY.row_floats()
    for position, token in enumerate(tokens):
        for layer in range(len(GEOMETRY.layers)):
            k = [np.float32(token) + np.float32(position * 10 + layer + i) / np.float32(11.0) for i in range(row)]
            v = [-(np.float32(token) + np.float32(position + layer * 3 + i) / np.float32(5.0)) for i in range(row)]
            cache.append(layer, k, v, position)
    return orc.KvSnapshot.capture(cache, fingerprint)


def test_open_refuses_a_planted_garbage_entry_by_name(tmp_path):
    """store.rs:701-723: a 72-byte entry whose token count is u64::MAX and whose tokens_bytes disagrees is refused by
    name (the message formats the saturating product) and the store opens with it unindexed."""
    data = bytearray(72)
    data[0:8] = b"ITKVPENT"
    data[8:12] = struct.pack("<I", 1)
    data[40:48] = struct.pack("<Q", 2 ** 64 - 1)
    (tmp_path / "planted.kv").write_bytes(bytes(data))
    store = PrefixStore(str(tmp_path), 1 << 30)
    assert store.entries() == []
    assert "planted.kv" in store.last_refusal and "implies 18446744073709551615" in store.last_refusal


def test_put_lookup_round_trip(tmp_path):
    """store.rs:725-744"""
    store = PrefixStore(str(tmp_path), 1 << 30)
    tokens = [10, 20, 30, 40, 50]
    snap = snapshot_for(tokens, "model-a")
    store.put(tokens, snap.to_bytes(), 100)
    hit = store.lookup([10, 20, 30, 40, 50, 60, 70], now=200)
    assert hit is not None and hit.token_count == 5 and hit.tokens == tokens
    assert orc.KvSnapshot.from_bytes(hit.snapshot_bytes) == snap
    assert store.entries()[0].last_used_unix == 200  # restamped in the index ...
    assert PrefixStore(str(tmp_path), 1 << 30).entries()[0].last_used_unix == 200  # ... and on disk


def test_longest_prefix_wins_among_nested_entries(tmp_path):
    """store.rs:746-786"""
    store = PrefixStore(str(tmp_path), 1 << 30)
    for now, toks in enumerate(([1, 2], [1, 2, 3, 4], [1, 2, 3, 4, 5, 6]), start=1):
        store.put(toks, snapshot_for(toks, "model-a").to_bytes(), now)
    assert store.lookup([1, 2, 3, 4, 5, 6, 7, 8], now=10).token_count == 6
    assert store.lookup([1, 2, 3, 4, 99], now=11).token_count == 4
    assert store.lookup([1, 2, 77], now=12).token_count == 2
    assert store.lookup([9, 9], now=13) is None
    assert [e.token_count for e in store.entries()] == [6, 4, 2]


def test_put_refuses_mismatched_and_oversize(tmp_path):
    """store.rs:788-808"""
    store = PrefixStore(str(tmp_path / "a"), 1 << 30)
    other = snapshot_for([7, 8], "model-a").to_bytes()
    with pytest.raises(CudaComputeError) as e:
        store.put([1, 2, 3], other, 1)
    assert e.value.code == _lib.ERR_TOKEN_COUNT_MISMATCH
    assert e.value.msg == "snapshot covers 2 tokens but was offered under 3 token ids"
    with pytest.raises(CudaComputeError) as e:
        store.put([], other, 1)
    assert e.value.code == _lib.ERR_EMPTY_PREFIX and e.value.msg == "empty token prefix refused"
    small = PrefixStore(str(tmp_path / "b"), 128)
    snap = snapshot_for([1, 2, 3], "model-a").to_bytes()
    with pytest.raises(CudaComputeError) as e:
        small.put([1, 2, 3], snap, 1)
    assert e.value.code == _lib.ERR_ENTRY_TOO_LARGE
    assert e.value.msg == f"entry of {72 + 12 + len(snap)} bytes exceeds the store cap of 128 bytes"
    with pytest.raises(CudaComputeError) as e:
        PrefixStore(str(tmp_path / "c"), 0)
    assert e.value.code == _lib.ERR_INVALID_CONFIG and e.value.msg == "invalid config: the store byte cap is zero"


def test_entry_files_are_byte_identical_to_the_reference_layout(tmp_path):
    """Entry layout store.rs:5-21 and file naming store.rs:459-468: what the library writes equals the oracle's
    encoding, and a directory written by one side is served by the other."""
    tokens = [5, 6, 7, 0xFFFFFFFF]
    snap = snapshot_for(tokens, "fp")
    store = PrefixStore(str(tmp_path / "ours"), 1 << 30)
    store.put(tokens, snap.to_bytes(), 1234)
    name = ops.file_name_for(tokens)
    assert [e.file_name for e in store.entries()] == [name]
    assert (tmp_path / "ours" / name).read_bytes() == ops.entry_bytes(tokens, snap.to_bytes(), 1234)
    assert store.entries()[0].prefix_hash == orc.prefix_hash(tokens)
    assert store.stats() == {"entries": 1, "total_bytes": 72 + 16 + len(snap.to_bytes()), "max_bytes": 1 << 30}
    # the oracle's store reads our directory ...
    theirs = ops.PrefixStore(str(tmp_path / "ours"), 1 << 30)
    assert theirs.lookup(tokens + [9], now=5) == (4, snap.to_bytes())
    # ... and ours reads a directory the oracle wrote
    ref = ops.PrefixStore(str(tmp_path / "ref"), 1 << 30)
    ref.put(tokens, snap, 77)
    mine = PrefixStore(str(tmp_path / "ref"), 1 << 30)
    hit = mine.lookup(tokens, now=78)
    assert hit.token_count == 4 and hit.snapshot_bytes == snap.to_bytes()
    assert mine.entries()[0].created_unix == 77 and mine.entries()[0].last_used_unix == 78


def test_lru_eviction_matches_the_oracle_policy(tmp_path):
    """store.rs:41-46, 518-546: after every put, the least recently used entry other than the new one goes while
    the store is over its cap; ties fall to the smaller file name."""
    prefixes = [[1], [1, 2], [1, 2, 3], [4, 5], [6, 7, 8, 9]]
    snaps = [snapshot_for(p, "m") for p in prefixes]
    sizes = [72 + 4 * len(p) + len(s.to_bytes()) for p, s in zip(prefixes, snaps)]
    cap = sizes[0] + sizes[1] + sizes[2] + 10
    ours, ref = PrefixStore(str(tmp_path / "o"), cap), ops.PrefixStore(str(tmp_path / "r"), cap)
    for now, (p, s) in enumerate(zip(prefixes[:3], snaps[:3]), start=1):
        ours.put(p, s.to_bytes(), now)
        ref.put(p, s, now)
    assert ours.lookup([1, 9], now=50).token_count == 1  # [1] becomes the most recently used
    assert ref.lookup([1, 9], now=50)[0] == 1
    for now, (p, s) in enumerate(zip(prefixes[3:], snaps[3:]), start=60):
        ours.put(p, s.to_bytes(), now)
        ref.put(p, s, now)
        assert sorted(e.file_name for e in ours.entries()) == sorted(e["file_name"] for e in ref.entries)
        assert sorted(os.listdir(tmp_path / "o")) == sorted(os.listdir(tmp_path / "r"))
        assert ours.stats()["total_bytes"] <= cap
        if now == 60:  # [1, 2] (last used at 2) went first; [1] (used at 50) stayed
            names = [e.file_name for e in ours.entries()]
            assert ops.file_name_for([1]) in names and ops.file_name_for([1, 2]) not in names


def test_forged_and_corrupt_entries_are_refused_and_shorter_prefixes_still_serve(tmp_path):
    """Trust model store.rs:23-33: ids must hash back to the key, the payload must decode and cover the preamble's
    token count; a failing candidate is refused by name and never stops a shorter honest prefix."""
    store = PrefixStore(str(tmp_path), 1 << 30)
    short, long = [1, 2], [1, 2, 3, 4]
    store.put(short, snapshot_for(short, "m").to_bytes(), 1)
    store.put(long, snapshot_for(long, "m").to_bytes(), 2)
    path = tmp_path / ops.file_name_for(long)
    honest = path.read_bytes()
    # (a) flipped payload byte: the snapshot checksum refuses it
    bad = bytearray(honest)
    bad[-20] ^= 0x40
    path.write_bytes(bytes(bad))
    assert store.lookup([1, 2, 3, 4, 5], now=10).token_count == 2
    assert ops.file_name_for(long) in store.last_refusal and "checksum mismatch" in store.last_refusal
    # (b) stored ids edited: they no longer hash to the entry key
    bad = bytearray(honest)
    bad[72:76] = struct.pack("<I", 9)
    path.write_bytes(bytes(bad))
    assert store.lookup([1, 2, 3, 4, 5], now=11).token_count == 2
    want = f"stored token ids hash to {orc.prefix_hash([9, 2, 3, 4]):#018x}, not the entry key {orc.prefix_hash(long):#018x}"
    assert want in store.last_refusal
    # (c) torn final file
    path.write_bytes(honest[:100])
    assert store.lookup([1, 2, 3, 4, 5], now=12).token_count == 2
    assert "truncated" in store.last_refusal
    # (d) a snapshot of another prefix length under this entry's preamble
    other = snapshot_for([1, 2, 3], "m").to_bytes()
    forged = ops.encode_preamble(2, 2, orc.prefix_hash(long), 4, len(other)) + honest[72:88] + other
    path.write_bytes(forged)
    assert store.lookup([1, 2, 3, 4, 5], now=13).token_count == 2
    assert "entry preamble covers 4 tokens but its snapshot covers 3" in store.last_refusal
    # restored: the long entry serves again
    path.write_bytes(honest)
    assert store.lookup([1, 2, 3, 4, 5], now=14).token_count == 4
    # temp files and foreign names are never indexed (store.rs:35-39)
    (tmp_path / ".tmp-whatever.kv").write_bytes(honest)
    (tmp_path / "notes.txt").write_bytes(b"x")
    store.rescan()
    assert len(store.entries()) == 2


def test_required_geometry_and_fingerprint(tmp_path):
    """Trust check 3 (store.rs:424-445)."""
    store = PrefixStore(str(tmp_path), 1 << 30)
    toks = [3, 1, 4, 1, 5]
    store.put(toks, snapshot_for(toks, "model-a").to_bytes(), 1)
    good = ([4, 0], 2, 3)
    assert store.lookup(toks, expected_geometry=good, expected_fingerprint="model-a", now=2).token_count == 5
    assert store.lookup(toks, expected_geometry=([0, 0], 2, 3), now=3) is None
    assert "snapshot geometry differs from the required geometry" in store.last_refusal
    assert store.lookup(toks, expected_geometry=good, expected_fingerprint="model-b", now=4) is None
    assert "model fingerprint mismatch: need model-b, snapshot carries model-a" in store.last_refusal


def test_put_replaces_an_entry_with_the_same_tokens(tmp_path):
    store = PrefixStore(str(tmp_path), 1 << 30)
    toks = [8, 8, 8]
    store.put(toks, snapshot_for(toks, "old").to_bytes(), 1)
    store.put(toks, snapshot_for(toks, "new").to_bytes(), 2)
    assert len(store.entries()) == 1 and store.entries()[0].created_unix == 2
    assert store.lookup(toks, expected_fingerprint="new", now=3).token_count == 3


def test_a_taken_file_name_gets_a_counter_suffix(tmp_path):
    """store.rs:459-502: when another token list already owns the hash/length/discriminator name (a double hash
    collision, here planted), the put takes `-c1` and both entries serve their own prefix."""
    tokens, squatter = [7, 7, 7], [1, 2, 3]
    name = ops.file_name_for(tokens)
    snap_s = snapshot_for(squatter, "m").to_bytes()
    # a well-formed entry for `squatter` sitting under the name `tokens` would get
    (tmp_path / name).write_bytes(ops.entry_bytes(squatter, snap_s, 5))
    store = PrefixStore(str(tmp_path), 1 << 30)
    assert [e.file_name for e in store.entries()] == [name]
    store.put(tokens, snapshot_for(tokens, "m").to_bytes(), 6)
    names = sorted(e.file_name for e in store.entries())
    assert names == sorted([name, ops.file_name_for(tokens, counter=1)])
    assert store.lookup(tokens, now=7).snapshot_bytes == snapshot_for(tokens, "m").to_bytes()
    assert store.lookup(squatter, now=8).snapshot_bytes == snap_s
    # putting the same tokens again reuses the suffixed name instead of taking `-c2`
    store.put(tokens, snapshot_for(tokens, "m2").to_bytes(), 9)
    assert sorted(e.file_name for e in store.entries()) == names


def test_typed_snapshots_are_stored_and_served_and_forged_ones_refused(tmp_path):
    """The store's payload check reads both format versions: a version-2 snapshot (half rows, this library's
    extension for f16 caches) is put, found and returned byte for byte; one whose element type tag is unknown, or
    whose rows stop short, is refused at the door by name."""
    from kvparity import typed_itkv_bytes

    tokens = [3, 1, 4, 1, 5]
    snap = snapshot_for(tokens, "model-h")
    window = [4, 0]
    typed = typed_itkv_bytes(snap, "model-h", GEOMETRY.num_kv_heads, GEOMETRY.head_dim, window, half=True)
    assert len(typed) < len(snap.to_bytes())
    store = PrefixStore(str(tmp_path), 1 << 30)
    store.put(tokens, typed, 7)
    hit = store.lookup(tokens + [9, 2], now=8)
    assert hit is not None and hit.token_count == 5 and hit.snapshot_bytes == typed

    def resum(data):
        return bytes(data[:-8]) + struct.pack("<Q", orc.checksum(bytes(data[:-8])))

    bad_tag = bytearray(typed)
    bad_tag[8] = 9
    with pytest.raises(CudaComputeError) as e:
        store.put([8, 8, 8, 8, 8], resum(bad_tag), 9)
    assert e.value.code == _lib.ERR_INCONSISTENT_SNAPSHOT and "element type" in e.value.msg
    with pytest.raises(CudaComputeError) as e:
        store.put(tokens, typed[:-30], 9)
    assert e.value.code == _lib.ERR_TRUNCATED
