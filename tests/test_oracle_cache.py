"""The oracle against the reference's KV-cache known-answer tests
(crates/attention/tests/cache_tests.rs; line ranges per test)."""
import numpy as np
import pytest

from oracle import oracle as orc
from oracle.oracle import GLOBAL, KvCache, LayerKind, OracleError

USIZE_MAX = (1 << 64) - 1


def row(kv_heads, head_dim, fill):
    return np.full(kv_heads * head_dim, fill, dtype=np.float32)


def test_glimmer_pattern_is_39_windowed_13_global():
    """cache_tests.rs:12-35"""
    pattern = orc.glimmer_layer_pattern()
    assert len(pattern) == 52
    assert [i for i, k in enumerate(pattern) if not k.windowed] == [3, 7, 11, 15, 19, 23, 27, 31, 35, 39, 43, 47, 51]
    assert sum(1 for k in pattern if k.windowed) == 39
    assert all(k.window_size == 2048 for k in pattern if k.windowed)


def test_ring_buffer_wraps_and_evicts_oldest():
    """cache_tests.rs:38-62: window 4, positions 0..=6 leave 3,4,5,6."""
    cache = KvCache([LayerKind.windowed_checked(4)], 1, 1)
    for pos in range(7):
        cache.append(0, row(1, 1, pos), row(1, 1, pos), pos)
    assert cache.stored_len(0) == 4
    assert cache.next_position(0) == 7
    view = cache.view(0)
    assert len(view) == 4 and not view.is_empty()
    for vi, want in enumerate([3, 4, 5, 6]):
        assert view.position_at(vi) == want
        assert view.value(vi, 0).tolist() == [float(want)]
        assert view.key(vi, 0).tolist() == [float(want)]
    assert view.position_at(4) is None
    stats = cache.stats()
    assert stats[0].appended == 7 and stats[0].stored == 4


def test_ring_buffer_holds_exactly_the_glimmer_window():
    """cache_tests.rs:65-79: 2050 appends at window 2048 -> first visible position 2."""
    cache = KvCache([LayerKind.windowed_checked(2048)], 2, 4)
    rows = np.repeat(np.arange(2050, dtype=np.float32)[:, None], 8, axis=1)
    cache.append_rows(0, rows, rows, 0)
    assert cache.stored_len(0) == 2048
    view = cache.view(0)
    assert view.position_at(0) == 2
    assert view.position_at(2047) == 2049
    assert view.value(0, 0)[0] == 2.0
    assert view.value(2047, 1)[0] == 2049.0


def test_global_layer_keeps_everything():
    """cache_tests.rs:82-96"""
    cache = KvCache([GLOBAL], 2, 2)
    for pos in range(10):
        cache.append(0, row(2, 2, pos), row(2, 2, pos), pos)
    assert cache.stored_len(0) == 10
    view = cache.view(0)
    assert len(view) == 10 and view.window() is None
    for pos in range(10):
        assert view.position_at(pos) == pos
        assert view.value(pos, 1)[0] == float(pos)


def test_append_rejects_bad_shapes_and_out_of_order_positions():
    """cache_tests.rs:99-131"""
    cache = KvCache([GLOBAL], 2, 4)
    with pytest.raises(OracleError) as e:
        cache.append(0, row(1, 4, 0.0), row(2, 4, 0.0), 0)
    assert e.value.code == orc.SHAPE_MISMATCH and e.value.msg == "k: got 4, expected 8"
    with pytest.raises(OracleError) as e:
        cache.append(0, row(2, 4, 0.0), row(2, 4, 0.0), 1)
    assert e.value.code == orc.OUT_OF_ORDER_POSITION
    assert e.value.msg == "layer 0 appends must be in order: expected position 0, got 1"
    assert cache.stored_len(0) == 0
    cache.append(0, row(2, 4, 0.0), row(2, 4, 0.0), 0)
    assert cache.stored_len(0) == 1


def test_construction_rejects_zero_dimensions_and_window():
    """cache_tests.rs:134-161"""
    for args, code, text in [
        (([], 2, 128), orc.ZERO_DIMENSION, "layer pattern must be positive, got 0"),
        (([GLOBAL], 0, 128), orc.ZERO_DIMENSION, "num_kv_heads must be positive, got 0"),
        (([GLOBAL], 2, 0), orc.ZERO_DIMENSION, "head_dim must be positive, got 0"),
        (([LayerKind.Windowed(0)], 2, 128), orc.INVALID_WINDOW, "sliding window must be positive, got 0"),
    ]:
        with pytest.raises(OracleError) as e:
            KvCache(*args)
        assert e.value.code == code and e.value.msg == text
    with pytest.raises(OracleError) as e:
        LayerKind.windowed_checked(0)
    assert e.value.code == orc.INVALID_WINDOW


def test_construction_refuses_sizes_that_overflow():
    """cache_tests.rs:164-183"""
    with pytest.raises(OracleError) as e:
        KvCache([LayerKind.Windowed(USIZE_MAX)], 2, 128)
    assert e.value.code == orc.SIZE_OVERFLOW and e.value.msg.startswith("windowed layer storage")
    with pytest.raises(OracleError) as e:
        KvCache([GLOBAL], USIZE_MAX, 2)
    assert e.value.code == orc.SIZE_OVERFLOW and e.value.msg.startswith("kv row length")


def test_invalid_layer_is_an_error_not_a_panic():
    """cache_tests.rs:186-205"""
    cache = KvCache([GLOBAL], 1, 1)
    with pytest.raises(OracleError) as e:
        cache.view(5)
    assert e.value.code == orc.INVALID_LAYER and e.value.msg == "layer 5 out of range, cache has 1 layers"
    with pytest.raises(OracleError) as e:
        cache.append(5, row(1, 1, 0.0), row(1, 1, 0.0), 0)
    assert e.value.code == orc.INVALID_LAYER
    assert cache.layer_kind(0) == GLOBAL


def test_empty_view_is_empty_and_indexes_to_none():
    """cache_tests.rs:208-216"""
    cache = KvCache([LayerKind.windowed_checked(8)], 1, 2)
    view = cache.view(0)
    assert view.is_empty() and len(view) == 0
    assert view.position_at(0) is None
    assert view.key(0, 0) is None
    assert view.window() == 8


def rows_for(layer, position, row_len):
    k = np.array([np.float32(position * 100 + layer * 10 + i) / np.float32(7.0) for i in range(row_len)], np.float32)
    v = np.array([-np.float32(position * 50 + layer * 5 + i) / np.float32(3.0) for i in range(row_len)], np.float32)
    return k, v


def test_bulk_restore_matches_append_replay_bitwise():
    """cache_tests.rs:218-283"""
    pattern = [LayerKind.windowed_checked(4), GLOBAL, LayerKind.windowed_checked(4)]
    kv_heads, head_dim, tokens = 2, 3, 9
    row_len = kv_heads * head_dim
    replay = KvCache(pattern, kv_heads, head_dim)
    for position in range(tokens):
        for layer in range(3):
            replay.append(layer, *rows_for(layer, position, row_len), position)
    bulk = KvCache(pattern, kv_heads, head_dim)
    for layer, kind in enumerate(pattern):
        first, count = (0, tokens) if not kind.windowed else (tokens - min(tokens, kind.window_size), min(tokens, kind.window_size))
        keys = np.concatenate([rows_for(layer, p, row_len)[0] for p in range(first, first + count)])
        values = np.concatenate([rows_for(layer, p, row_len)[1] for p in range(first, first + count)])
        bulk.restore_bulk(layer, first, keys, values)
    for layer in range(3):
        assert bulk.next_position(layer) == tokens
        wp, wk, wv = replay.view(layer).dump()
        gp, gk, gv = bulk.view(layer).dump()
        assert gp == wp
        assert gk.tobytes() == wk.tobytes() and gv.tobytes() == wv.tobytes()
        k, v = rows_for(layer, tokens, row_len)
        replay.append(layer, k, v, tokens)
        bulk.append(layer, k, v, tokens)


def test_bulk_restore_refusals_are_named():
    """cache_tests.rs:286-322"""
    pattern = [LayerKind.windowed_checked(4), GLOBAL]
    cache = KvCache(pattern, 1, 2)
    with pytest.raises(OracleError) as e:
        cache.restore_bulk(0, 0, np.zeros(10), np.zeros(10))
    assert e.value.code == orc.SHAPE_MISMATCH and "bulk restore rows (windowed layer)" in e.value.msg
    with pytest.raises(OracleError) as e:
        cache.restore_bulk(1, 3, np.zeros(4), np.zeros(4))
    assert e.value.code == orc.SHAPE_MISMATCH and "first position (global layer)" in e.value.msg
    cache.append(0, row(1, 2, 1.0), row(1, 2, 1.0), 0)
    with pytest.raises(OracleError) as e:
        cache.restore_bulk(0, 0, np.zeros(2), np.zeros(2))
    assert e.value.code == orc.BULK_RESTORE_NOT_FRESH
    assert e.value.msg.startswith("layer 0 already holds 1 appended positions")
    fresh = KvCache(pattern, 1, 2)
    with pytest.raises(OracleError) as e:
        fresh.restore_bulk(0, 0, np.zeros(4), np.zeros(2))
    assert e.value.code == orc.SHAPE_MISMATCH and e.value.msg == "bulk restore rows: got 4, expected 2"
