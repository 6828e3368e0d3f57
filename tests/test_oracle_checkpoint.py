"""The oracle against the reference's checkpoint / rewind known-answer tests
(crates/attention/tests/checkpoint_tests.rs; line ranges per test).

Rows carry exactly representable values encoding (position, head, dim), so
"restored" is exact equality.
"""
import numpy as np
import pytest

from oracle import oracle as orc
from oracle.oracle import GLOBAL, KvCache, LayerKind, OracleError, gqa_attention


def k_row(kv_heads, head_dim, position):
    return np.array([position * 1000 + (e // head_dim) * 100 + (e % head_dim) for e in range(kv_heads * head_dim)],
                    dtype=np.float32)


def v_row(kv_heads, head_dim, position):
    return k_row(kv_heads, head_dim, position) + np.float32(500)


def append(cache, layer, kv_heads, head_dim, position):
    cache.append(layer, k_row(kv_heads, head_dim, position), v_row(kv_heads, head_dim, position), position)


def append_all(cache, kv_heads, head_dim, positions):
    for layer in range(cache.layer_count()):
        for p in positions:
            append(cache, layer, kv_heads, head_dim, p)


def view_snapshot(cache, layer):
    pos, k, v = cache.view(layer).dump()
    return pos, k.tobytes(), v.tobytes()


def reference_cache(pattern, kv_heads, head_dim, positions):
    cache = KvCache(pattern, kv_heads, head_dim)
    append_all(cache, kv_heads, head_dim, positions)
    return cache


W4 = LayerKind.windowed_checked(4)


def test_windowed_rewind_restores_rows_evicted_by_speculative_appends():
    """checkpoint_tests.rs:80-117"""
    cache = reference_cache([W4], 1, 2, range(6))
    committed = view_snapshot(cache, 0)
    cp = cache.checkpoint(3)
    assert cache.checkpoint_active()
    assert cp.base(0) == 6
    for p in (6, 7, 8):
        append(cache, 0, 1, 2, p)
    assert view_snapshot(cache, 0) != committed
    cache.rewind_to(cp, 6)
    cache.release(cp)
    assert not cache.checkpoint_active()
    assert view_snapshot(cache, 0) == committed
    st = cache.stats()
    assert st[0].appended == 6 and st[0].stored == 4
    fresh = reference_cache([W4], 1, 2, range(6))
    q = [0.5, -0.25]
    after = gqa_attention(q, 1, 1, [5], cache.view(0))
    never = gqa_attention(q, 1, 1, [5], fresh.view(0))
    assert after.tobytes() == never.tobytes()


def test_windowed_rewind_to_mid_block_keeps_exactly_the_committed_prefix():
    """checkpoint_tests.rs:120-144"""
    cache = reference_cache([W4], 2, 2, range(6))
    cp = cache.checkpoint(3)
    for p in (6, 7, 8):
        append(cache, 0, 2, 2, p)
    cache.rewind_to(cp, 7)
    cache.release(cp)
    assert view_snapshot(cache, 0) == view_snapshot(reference_cache([W4], 2, 2, range(7)), 0)
    assert cache.stats()[0].appended == 7
    append(cache, 0, 2, 2, 7)
    assert view_snapshot(cache, 0) == view_snapshot(reference_cache([W4], 2, 2, range(8)), 0)


def test_windowed_checkpoint_saved_slots_wrap_the_ring():
    """checkpoint_tests.rs:147-161: base 7, window 4 saves slots 3 and 0."""
    cache = reference_cache([W4], 1, 2, range(7))
    cp = cache.checkpoint(2)
    for p in (7, 8):
        append(cache, 0, 1, 2, p)
    cache.rewind_to(cp, 7)
    cache.release(cp)
    assert view_snapshot(cache, 0) == view_snapshot(reference_cache([W4], 1, 2, range(7)), 0)
    assert cache.stats()[0].appended == 7


def test_global_rewind_truncates_and_keeps_the_prefix():
    """checkpoint_tests.rs:164-181"""
    cache = reference_cache([GLOBAL], 2, 2, range(5))
    cp = cache.checkpoint(3)
    assert cp.saved_bytes() == 0
    for p in (5, 6, 7):
        append(cache, 0, 2, 2, p)
    assert cache.stored_len(0) == 8
    cache.rewind_to(cp, 6)
    cache.release(cp)
    assert view_snapshot(cache, 0) == view_snapshot(reference_cache([GLOBAL], 2, 2, range(6)), 0)
    assert cache.stats()[0].appended == 6 and cache.stored_len(0) == 6


def test_rewind_to_a_checkpoint_taken_before_any_append():
    """checkpoint_tests.rs:184-207"""
    pattern = [W4, GLOBAL]
    cache = KvCache(pattern, 1, 2)
    cp = cache.checkpoint(2)
    assert cp.base(0) == 0 and cp.base(1) == 0
    append_all(cache, 1, 2, [0, 1])
    cache.rewind_to(cp, 0)
    cache.release(cp)
    for layer in range(2):
        assert cache.stats()[layer].appended == 0
        assert cache.view(layer).is_empty()
    append_all(cache, 1, 2, [0, 1])
    ref = reference_cache(pattern, 1, 2, [0, 1])
    for layer in range(2):
        assert view_snapshot(cache, layer) == view_snapshot(ref, layer)


def test_second_rewind_restores_the_snapshot_again():
    """checkpoint_tests.rs:210-230"""
    cache = reference_cache([W4], 1, 2, range(6))
    committed = view_snapshot(cache, 0)
    cp = cache.checkpoint(3)
    for p in (6, 7, 8):
        append(cache, 0, 1, 2, p)
    cache.rewind_to(cp, 6)
    append(cache, 0, 1, 2, 6)
    assert view_snapshot(cache, 0) != committed
    cache.rewind_to(cp, 6)
    cache.release(cp)
    assert view_snapshot(cache, 0) == committed


def test_checkpoint_contract_violations_are_named_refusals():
    """checkpoint_tests.rs:233-316"""
    pattern = [W4, GLOBAL]
    cache = reference_cache(pattern, 1, 2, [0, 1])
    with pytest.raises(OracleError) as e:
        cache.checkpoint(0)
    assert e.value.code == orc.ZERO_DIMENSION and e.value.msg == "max_round_tokens must be positive, got 0"
    with pytest.raises(OracleError) as e:
        cache.checkpoint(5)
    assert e.value.code == orc.CHECKPOINT_TOO_DEEP
    assert e.value.msg.startswith("checkpoint round bound 5 exceeds the smallest sliding window 4")
    cp = cache.checkpoint(2)
    with pytest.raises(OracleError) as e:
        cache.checkpoint(1)
    assert e.value.code == orc.CHECKPOINT_BUSY
    append_all(cache, 1, 2, [2, 3])
    with pytest.raises(OracleError) as e:
        cache.append(0, k_row(1, 2, 4), v_row(1, 2, 4), 4)
    assert e.value.code == orc.CHECKPOINT_RANGE_EXCEEDED
    assert "layer 0 append at position 4" in e.value.msg and "first unsaved position 4" in e.value.msg
    with pytest.raises(OracleError) as e:
        cache.rewind_to(cp, 1)
    assert e.value.code == orc.REWIND_OUT_OF_RANGE
    assert e.value.msg == "rewind target 1 is outside layer 0's checkpoint range [2, 4]"
    with pytest.raises(OracleError) as e:
        cache.rewind_to(cp, 5)
    assert e.value.code == orc.REWIND_OUT_OF_RANGE
    assert e.value.msg == "rewind target 5 is outside layer 0's checkpoint range [2, 4]"
    assert cache.stats()[0].appended == 4
    cache.release(cp)
    for op in (lambda: cache.rewind_to(cp, 2), lambda: cache.release(cp)):
        with pytest.raises(OracleError) as e:
            op()
        assert e.value.code == orc.STALE_CHECKPOINT
    other = reference_cache(pattern, 1, 2, [0, 1])
    foreign = other.checkpoint(2)
    mine = cache.checkpoint(2)
    with pytest.raises(OracleError) as e:
        cache.rewind_to(foreign, 2)
    assert e.value.code == orc.STALE_CHECKPOINT
    cache.release(mine)
    other.release(foreign)


def test_checkpoint_memory_bound_at_glimmer_geometry():
    """checkpoint_tests.rs:319-337: 39 * 17 * 2048 = 1,357,824 bytes."""
    cache = KvCache(orc.glimmer_layer_pattern(), 2, 128)
    append_all(cache, 2, 128, [0])
    cp = cache.checkpoint(17)
    assert cp.base(0) == 1 and cp.base(51) == 1
    assert cp.max_round_tokens() == 17
    assert cp.saved_bytes() == 39 * 17 * 2048 == 1_357_824
    cache.release(cp)
