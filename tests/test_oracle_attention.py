"""The oracle against the reference's attention known-answer tests.

Every case restates one test of crates/attention/tests/attention_tests.rs
(line ranges in each docstring); the expected values are the reference's.
"""
import numpy as np
import pytest

from oracle import oracle as orc
from oracle.oracle import GLOBAL, KvCache, LayerKind, OracleError, gqa_attention


def cache_with(kind, kv_heads, head_dim, rows):
    cache = KvCache([kind], kv_heads, head_dim)
    for pos, (k, v) in enumerate(rows):
        cache.append(0, k, v, pos)
    return cache


def test_windowed_layer_provably_cannot_see_beyond_the_window():
    """attention_tests.rs:30-45: window 2 averages (3 + 5) / 2 = 4, not 336."""
    rows = [([1.0], [1000.0]), ([1.0], [3.0]), ([1.0], [5.0])]
    cache = cache_with(LayerKind.windowed_checked(2), 1, 1, rows)
    out = gqa_attention([1.0], 1, 1, [2], cache.view(0))
    assert abs(out[0] - 4.0) <= 1e-6


def test_global_layer_sees_everything():
    """attention_tests.rs:48-61: the same rows on a global layer average to 336."""
    rows = [([1.0], [1000.0]), ([1.0], [3.0]), ([1.0], [5.0])]
    cache = cache_with(GLOBAL, 1, 1, rows)
    out = gqa_attention([1.0], 1, 1, [2], cache.view(0))
    assert abs(out[0] - 336.0) <= 1e-3


def test_causal_mask_blocks_future_positions():
    """attention_tests.rs:64-85: query 0 returns exactly 1; query 1 sits in (99.9, 100)."""
    rows = [([0.0], [1.0]), ([10.0], [100.0]), ([10.0], [1000.0])]
    cache = cache_with(GLOBAL, 1, 1, rows)
    out = gqa_attention([1.0, 1.0], 2, 1, [0, 1], cache.view(0))
    assert abs(out[0] - 1.0) <= 1e-6
    assert 99.9 < out[1] < 100.0


def test_gqa_head_sharing_glimmer_shape_32_to_2():
    """attention_tests.rs:88-114: heads 0..16 read KV head 0 (10), 16..32 read KV head 1 (20)."""
    for h in range(32):
        assert orc.kv_head_for_query_head(h, 32, 2) == (0 if h < 16 else 1)
    cache = cache_with(GLOBAL, 2, 2, [([1.0, 0.0, 1.0, 0.0], [10.0, 0.0, 20.0, 0.0])])
    q = [1.0, 0.0] * 32
    out = gqa_attention(q, 1, 32, [0], cache.view(0))
    for h in range(32):
        assert abs(out[h * 2] - (10.0 if h < 16 else 20.0)) <= 1e-6
        assert abs(out[h * 2 + 1]) <= 1e-6


def test_gqa_head_sharing_smaller_ratio_4_to_2():
    """attention_tests.rs:117-140: 7, 7, 9, 9."""
    for h, want in [(0, 0), (1, 0), (2, 1), (3, 1)]:
        assert orc.kv_head_for_query_head(h, 4, 2) == want
    cache = cache_with(GLOBAL, 2, 1, [([1.0, 1.0], [7.0, 9.0])])
    out = gqa_attention([1.0] * 4, 1, 4, [0], cache.view(0))
    for h, want in [(0, 7.0), (1, 7.0), (2, 9.0), (3, 9.0)]:
        assert abs(out[h] - want) <= 1e-6


def test_scale_defaults_to_one_over_sqrt_head_dim():
    """attention_tests.rs:143-150: scale_for(128) = 0.08838835, scale_for(1) = 1."""
    assert abs(orc.default_scale(128) - 0.08838835) <= 1e-7
    assert abs(orc.default_scale(1) - 1.0) <= 1e-7
    # A pinned scale is honoured: with scale 0 every score ties and the output is the mean.
    cache = cache_with(GLOBAL, 1, 1, [([5.0], [2.0]), ([-3.0], [4.0])])
    out = gqa_attention([1.0], 1, 1, [1], cache.view(0), scale=0.0)
    assert abs(out[0] - 3.0) <= 1e-6


def test_attention_validation_is_named_errors_not_panics():
    """attention_tests.rs:153-212: NoVisibleKeys, NonDivisibleHeads, ShapeMismatch q / query_positions."""
    cache = KvCache([GLOBAL], 2, 2)
    with pytest.raises(OracleError) as e:
        gqa_attention([1.0, 0.0, 1.0, 0.0], 1, 2, [0], cache.view(0))
    assert e.value.code == orc.NO_VISIBLE_KEYS and "position 0" in e.value.msg

    cache = cache_with(GLOBAL, 2, 2, [([1.0, 0.0, 1.0, 0.0], [1.0, 0.0, 1.0, 0.0])])
    with pytest.raises(OracleError) as e:
        gqa_attention([1.0] * 6, 1, 3, [0], cache.view(0))
    assert e.value.code == orc.NON_DIVISIBLE_HEADS
    assert e.value.msg == "3 query heads do not divide evenly across 2 KV heads"

    with pytest.raises(OracleError) as e:
        gqa_attention([1.0], 1, 2, [0], cache.view(0))
    assert e.value.code == orc.SHAPE_MISMATCH and e.value.msg == "q: got 1, expected 4"

    with pytest.raises(OracleError) as e:
        gqa_attention([1.0] * 4, 2, 2, [0], cache.view(0))
    assert e.value.code == orc.SHAPE_MISMATCH and e.value.msg == "query_positions: got 1, expected 2"

    with pytest.raises(OracleError) as e:
        orc.kv_head_for_query_head(0, 3, 2)
    assert e.value.code == orc.NON_DIVISIBLE_HEADS


def test_zero_queries_is_an_empty_result():
    """attention.rs:130-132: zero queries return an empty vector before any other check."""
    cache = cache_with(GLOBAL, 1, 1, [([1.0], [1.0])])
    assert gqa_attention([], 0, 1, [], cache.view(0)).size == 0


def test_softmax_matches_a_float64_restatement():
    """A seeded GQA case against an independent float64 softmax (tolerance 1e-5 of the output)."""
    rng = np.random.default_rng(7)
    hkv, hq, d, n = 2, 8, 16, 37
    cache = KvCache([GLOBAL], hkv, d)
    ks = rng.standard_normal((n, hkv, d)).astype(np.float32)
    vs = rng.standard_normal((n, hkv, d)).astype(np.float32)
    for p in range(n):
        cache.append(0, ks[p], vs[p], p)
    q = rng.standard_normal((hq, d)).astype(np.float32)
    out = gqa_attention(q, 1, hq, [n - 1], cache.view(0)).reshape(hq, d)
    g = hq // hkv
    for h in range(hq):
        s = (ks[:, h // g, :].astype(np.float64) @ q[h].astype(np.float64)) / np.sqrt(d)
        w = np.exp(s - s.max())
        w /= w.sum()
        want = w @ vs[:, h // g, :].astype(np.float64)
        assert np.max(np.abs(out[h] - want)) <= 1e-5
