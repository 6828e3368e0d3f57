"""The oracle against the reference's prefix-snapshot known-answer tests:
crates/itak-kv/src/snapshot.rs:646-861 (unit tests), crates/itak-kv/src/hash.rs:67-87,
crates/itak-kv/tests/restore_fixture.rs:116-189 (cold vs restored continuation)."""
import struct

import numpy as np
import pytest

from oracle import oracle as orc
from oracle.oracle import GLOBAL, KvCache, KvGeometry, KvSnapshot, LayerKind, OracleError, gqa_attention, lcg

FNV_OFFSET = 0xCBF29CE484222325


def geometry():
    return KvGeometry([LayerKind.Windowed(4), GLOBAL, LayerKind.Windowed(4)], 2, 3)


def filled_cache(tokens):
    g = geometry()
    cache = KvCache(g.layers, g.num_kv_heads, g.head_dim)
    row = g.row_floats()
    for position in range(tokens):
        for layer in range(3):
            k = np.array([np.float32(position * 100 + layer * 10 + i) / np.float32(7) for i in range(row)], np.float32)
            v = np.array([-np.float32(position * 50 + layer * 5 + i) / np.float32(3) for i in range(row)], np.float32)
            cache.append(layer, k, v, position)
    return cache


def test_bytes_round_trip():
    """snapshot.rs:646-653"""
    snap = KvSnapshot.capture(filled_cache(10), "model-a")
    decoded = KvSnapshot.from_bytes(snap.to_bytes(), geometry())
    assert decoded == snap


def test_byte_layout_is_the_documented_one():
    """snapshot.rs:13-29: header fields, per-layer 28-byte headers, f32 LE payload, FNV-1a-64 trailer."""
    snap = KvSnapshot.capture(filled_cache(10), "model-a")
    b = snap.to_bytes()
    assert b[:4] == b"ITKV"
    assert struct.unpack_from("<I", b, 4)[0] == 1
    assert struct.unpack_from("<I", b, 8)[0] == 7 and b[12:19] == b"model-a"
    token_count, hkv, d, layers = struct.unpack_from("<QIII", b, 19)
    assert (token_count, hkv, d, layers) == (10, 2, 3, 3)
    at = 19 + 20
    want = [(1, 4, 6, 4), (0, 0, 0, 10), (1, 4, 6, 4)]
    for tag, window, first, rows in want:
        assert b[at] == tag and b[at + 1:at + 4] == b"\0\0\0"
        assert struct.unpack_from("<QQQ", b, at + 4) == (window, first, rows)
        at += 28
    payload = (4 + 10 + 4) * 6 * 2 * 4
    assert len(b) == at + payload + 8
    assert struct.unpack_from("<Q", b, len(b) - 8)[0] == orc.checksum(b[:-8])
    first, k, _ = snap.layer(1)
    assert first == 0
    assert np.frombuffer(b, dtype="<f4", count=60, offset=at + 4 * 6 * 2 * 4).tobytes() == k.tobytes()


def test_restore_rebuilds_the_same_views():
    """snapshot.rs:656-676"""
    cache = filled_cache(10)
    restored = KvSnapshot.capture(cache, "model-a").restore()
    for layer in range(3):
        assert restored.next_position(layer) == cache.next_position(layer)
        wp, wk, wv = cache.view(layer).dump()
        gp, gk, gv = restored.view(layer).dump()
        assert gp == wp and gk.tobytes() == wk.tobytes() and gv.tobytes() == wv.tobytes()


def test_restore_can_continue_appending():
    """snapshot.rs:679-690"""
    restored = KvSnapshot.capture(filled_cache(6), "model-a").restore()
    for layer in range(3):
        restored.append(layer, np.full(6, 1.5), np.full(6, -2.5), 6)
    assert restored.next_position(0) == 7


def test_capture_refuses_a_divergent_cache():
    """snapshot.rs:693-706"""
    g = geometry()
    cache = KvCache(g.layers, g.num_kv_heads, g.head_dim)
    cache.append(0, np.zeros(6), np.zeros(6), 0)
    with pytest.raises(OracleError) as e:
        KvSnapshot.capture(cache, "model-a")
    assert e.value.code == orc.INCOHERENT_CACHE


def test_decode_refuses_corruption():
    """snapshot.rs:709-726"""
    snap = KvSnapshot.capture(filled_cache(5), "model-a")
    b = bytearray(snap.to_bytes())
    b[len(b) - 12] ^= 0xFF
    with pytest.raises(OracleError) as e:
        KvSnapshot.from_bytes(bytes(b))
    assert e.value.code == orc.CHECKSUM_MISMATCH
    with pytest.raises(OracleError) as e:
        KvSnapshot.from_bytes(bytes(b[:8]))
    assert e.value.code == orc.TRUNCATED
    bad = bytearray(snap.to_bytes())
    bad[0] = ord("X")
    with pytest.raises(OracleError) as e:
        KvSnapshot.from_bytes(bytes(bad))
    assert e.value.code == orc.BAD_MAGIC
    # trailing bytes after the checksum (snapshot.rs:518-523)
    with pytest.raises(OracleError) as e:
        KvSnapshot.from_bytes(snap.to_bytes() + b"\0")
    assert e.value.code == orc.INCONSISTENT_SNAPSHOT and "trailing" in e.value.msg
    # unknown version (snapshot.rs:430-436)
    v2 = bytearray(snap.to_bytes())
    v2[4] = 2
    with pytest.raises(OracleError) as e:
        KvSnapshot.from_bytes(bytes(v2))
    assert e.value.code == orc.UNSUPPORTED_VERSION


def test_restore_checked_refuses_geometry_and_fingerprint():
    """snapshot.rs:729-748"""
    snap = KvSnapshot.capture(filled_cache(4), "model-a")
    other = geometry()
    other.head_dim = 9
    with pytest.raises(OracleError) as e:
        snap.restore_checked(other, "model-a")
    assert e.value.code == orc.GEOMETRY_MISMATCH
    with pytest.raises(OracleError) as e:
        snap.restore_checked(geometry(), "model-b")
    assert e.value.code == orc.FINGERPRINT_MISMATCH
    snap.restore_checked(geometry(), "model-a")


def test_decode_refuses_a_layer_count_that_cannot_fit_the_buffer():
    """snapshot.rs:751-774: 32-byte header declaring u32::MAX layers."""
    b = b"ITKV" + struct.pack("<IIQIII", 1, 0, 0, 1, 1, 0xFFFFFFFF)
    assert len(b) == 32
    with pytest.raises(OracleError) as e:
        KvSnapshot.from_bytes(b)
    assert e.value.code == orc.INCONSISTENT_SNAPSHOT


def test_decode_refuses_geometry_whose_row_products_overflow():
    """snapshot.rs:777-813: 2^32 tokens x (65536 x 65536) row floats with zero stored rows."""
    b = b"ITKV" + struct.pack("<II", 1, 1) + b"x" + struct.pack("<QIII", 1 << 32, 65536, 65536, 1)
    b += bytes([0, 0, 0, 0]) + struct.pack("<QQQ", 0, 0, 0)
    b += struct.pack("<Q", orc.checksum(b))
    with pytest.raises(OracleError) as e:
        KvSnapshot.from_bytes(b)
    assert e.value.code == orc.INCONSISTENT_SNAPSHOT


def test_validate_refuses_geometry_whose_row_width_overflows():
    """snapshot.rs:816-842"""
    g = KvGeometry([GLOBAL], 1 << 32, 1 << 32)
    snap = KvSnapshot.build(g, "x", 0, [(0, [], [])])
    with pytest.raises(OracleError) as e:
        snap.validate()
    assert e.value.code == orc.INCONSISTENT_SNAPSHOT


def test_validate_refuses_a_layer_cut_short():
    """wgpu-compute/src/session.rs:6325-6331: a truncated layer block is inconsistent."""
    snap = KvSnapshot.capture(filled_cache(10), "model-a")
    first, k, v = snap.layer(1)
    snap.set_layer(1, first, k[:4], v)
    with pytest.raises(OracleError) as e:
        snap.validate()
    assert e.value.code == orc.INCONSISTENT_SNAPSHOT and "inconsistent" in e.value.msg


def test_glimmer_sizing_math():
    """snapshot.rs:845-861: 106,496 B/token; 272,629,760 B at 4096; 3,653,238,784 B at 131,072."""
    g = KvGeometry(orc.glimmer_layer_pattern(), 2, 128)
    assert g.bytes_per_token() == 106_496
    assert g.stored_bytes_for(4096) == 272_629_760
    assert g.stored_bytes_for(131_072) == 3_653_238_784
    # the f16 halves of crates/wgpu-compute/tests/kv_f16.rs:229-239
    assert g.stored_bytes_for(131_072) // 2 == 1_826_619_392


def test_hashes():
    """hash.rs:67-87: the empty hash is the FNV offset basis; order and value sensitive."""
    assert orc.prefix_hash([]) == FNV_OFFSET
    assert orc.checksum(b"") == FNV_OFFSET
    assert orc.prefix_hash([1, 2, 3]) != orc.prefix_hash([3, 2, 1])
    assert orc.prefix_hash([1, 2, 3]) != orc.prefix_hash([1, 2, 4])
    assert orc.prefix_hash([1, 2]) != orc.prefix_hash([1, 2, 0])
    assert orc.prefix_hash([7, 8, 9, 10]) != orc.prefix_discriminator([7, 8, 9, 10])
    assert orc.checksum(b"itkv") != orc.checksum(b"itkw")
    # FNV-1a-64 published test vector for "a"
    assert orc.checksum(b"a") == 0xAF63DC4C8601EC8C
    # prefix_hash folds each token's 4 little-endian bytes
    assert orc.prefix_hash([0x04030201]) == orc.checksum(bytes([1, 2, 3, 4]))


# --- restore_fixture.rs -------------------------------------------------------------
Q_HEADS, LOGITS = 4, 16


def fixture_geometry():
    return KvGeometry([LayerKind.Windowed(4), GLOBAL, GLOBAL, LayerKind.Windowed(4)], 2, 8)


def fixture_rows(g, layer, position, token):
    row = g.row_floats()
    s = lcg((layer << 40) | (position << 16) | token, 2 * row)
    return s[:row], s[row:]


def append_token(cache, g, position, token):
    for layer in range(len(g.layers)):
        cache.append(layer, *fixture_rows(g, layer, position, token), position)


def logits_for(cache, g, position, token):
    q = lcg(0x5EED ^ (position << 20) ^ token, Q_HEADS * g.head_dim)
    logits = np.zeros(LOGITS, dtype=np.float32)
    for layer in range(len(g.layers)):
        out = gqa_attention(q, 1, Q_HEADS, [position], cache.view(layer))
        for o in range(LOGITS):
            acc = logits[o]
            for i, value in enumerate(out):
                w = np.float32(np.float32((o * 31 + i * 7 + layer * 3) % 13) / np.float32(7.0)) - np.float32(0.8)
                acc = np.float32(acc + np.float32(w * value))
            logits[o] = acc
    return logits


def continue_run(cache, g, start, continuation):
    all_logits, stream = [], []
    for step, token in enumerate(continuation):
        append_token(cache, g, start + step, token)
        logits = logits_for(cache, g, start + step, token)
        stream.append(int(np.argmax(logits)))
        all_logits.append(logits)
    return all_logits, stream


def test_restored_cache_continues_bitwise_identically():
    """restore_fixture.rs:116-189 (the store hop is the byte round trip here)."""
    g = fixture_geometry()
    prefix = [11, 22, 33, 44, 55, 66, 77, 88, 99]
    continuation = [5, 4, 3, 2, 1]
    cold = KvCache(g.layers, g.num_kv_heads, g.head_dim)
    for position, token in enumerate(prefix):
        append_token(cold, g, position, token)
    cold_logits, cold_stream = continue_run(cold, g, len(prefix), continuation)

    warm = KvCache(g.layers, g.num_kv_heads, g.head_dim)
    for position, token in enumerate(prefix):
        append_token(warm, g, position, token)
    snap = KvSnapshot.from_bytes(KvSnapshot.capture(warm, "fixture-model").to_bytes(), g)
    assert snap.token_count == len(prefix)
    restored = snap.restore_checked(g, "fixture-model")
    for layer in range(len(g.layers)):
        wp, wk, wv = warm.view(layer).dump()
        gp, gk, gv = restored.view(layer).dump()
        assert gp == wp and gk.tobytes() == wk.tobytes() and gv.tobytes() == wv.tobytes()
        assert restored.next_position(layer) == len(prefix)
    restored_logits, restored_stream = continue_run(restored, g, len(prefix), continuation)
    assert restored_stream == cold_stream
    for a, b in zip(restored_logits, cold_logits):
        assert a.tobytes() == b.tobytes()
