"""The oracle's slot/ring laws and CPU backend step against the reference's tests:
crates/wgpu-compute/src/session.rs:6184-6269 (visible range, slot-run remap),
crates/cpu-compute/tests/forward_tests.rs:642-719, 780-815, 1098-1181 (incremental decode == prefill,
checkpoint before any forward, speculative round trip, position desync)."""
import numpy as np
import pytest

from oracle import oracle as orc
from oracle.oracle import BackendConfig, CpuCompute, OracleError, PositionCache, lcg


def test_prefix_visible_range_is_the_snapshot_rule():
    """session.rs:6184-6202"""
    assert orc.prefix_visible_range(False, 4, 0) == (0, 0)
    assert orc.prefix_visible_range(False, 4, 70) == (0, 70)
    assert orc.prefix_visible_range(True, 4, 3) == (0, 3)
    assert orc.prefix_visible_range(True, 4, 4) == (0, 4)
    assert orc.prefix_visible_range(True, 4, 70) == (66, 4)


def test_prefix_slot_runs_remap_the_windowed_ring():
    """session.rs:6205-6269: the 70-token / window 4 / ring 67 wrap case and the two-run bound."""
    assert orc.prefix_slot_runs(False, 0, 70, 67)[0] == [(0, 0, 70)]
    assert orc.prefix_slot_runs(True, 10, 4, 67)[0] == [(0, 10, 4)]
    assert orc.prefix_slot_runs(True, 66, 4, 67)[0] == [(0, 66, 1), (1, 0, 3)]
    for cap in (1, 4, 32, 64):
        ring = 4 + cap - 1
        for position in range(300):
            first, rows = orc.prefix_visible_range(True, 4, position)
            runs, n = orc.prefix_slot_runs(True, first, rows, ring)
            assert n <= 2
            assert sum(r[2] for r in runs) == rows
            slots = [r[1] + i for r in runs for i in range(r[2])]
            assert slots == [p % ring for p in range(first, first + rows)]


def cfg(sliding, window, q_heads=4, kv_heads=2, d=8, base=10000.0):
    return BackendConfig(list(sliding), q_heads, kv_heads, d, d, window, base)


def forward(backend, c, pos, rows, seed):
    """One 'forward' over every layer: the same seeded q/k/v go to each layer, then the position advances."""
    outs = []
    qw, kw = c.q_heads * c.key_length, c.kv_heads * c.key_length
    for layer, sliding in enumerate(c.sliding):
        q = lcg(seed * 100 + layer * 3 + 1, rows * qw)
        k = lcg(seed * 100 + layer * 3 + 2, rows * kw)
        v = lcg(seed * 100 + layer * 3 + 3, rows * kw)
        outs.append(backend.attention(c, layer, sliding, q, k, v, pos))
    pos.advance(rows)
    return outs


def test_incremental_decode_matches_prefill_across_window_eviction():
    """forward_tests.rs:642-719: rows one at a time == all rows in one call, window 3 evicting."""
    c = cfg([True, False], 3)
    qw, kw = c.q_heads * c.key_length, c.kv_heads * c.key_length
    rows = 7
    q, k, v = lcg(11, rows * qw), lcg(12, rows * kw), lcg(13, rows * kw)
    for layer, sliding in enumerate(c.sliding):
        whole = CpuCompute().attention(c, layer, sliding, q, k, v, PositionCache())
        step = CpuCompute()
        pos = PositionCache()
        got = []
        for r in range(rows):
            got.append(step.attention(c, layer, sliding, q[r * qw:(r + 1) * qw], k[r * kw:(r + 1) * kw],
                                      v[r * kw:(r + 1) * kw], pos))
            pos.advance(1)
        assert np.concatenate(got).tobytes() == whole.tobytes()


def test_sliding_layers_rotate_and_global_layers_do_not():
    """cpu.rs:598-622: RoPE (adjacent pairs, SWA base) on sliding layers only; global layers are NoPE."""
    c = cfg([True, False], 16, q_heads=2, kv_heads=1, d=4)
    b = CpuCompute()
    pos = PositionCache()
    pos.advance(0)
    k = np.array([1.0, 0.0, 1.0, 0.0, 0.5, 0.25, -1.0, 2.0], dtype=np.float32)  # two rows
    v = np.ones(8, dtype=np.float32)
    q = np.ones(16, dtype=np.float32)
    for layer, sliding in enumerate(c.sliding):
        b.attention(c, layer, sliding, q, k, v, pos)
    cache = b.kv_cache(c)
    rotated = cache.view(0).key(1, 0)
    assert rotated.tobytes() == orc.rope_interleaved(k[4:], 1, 10000.0, 4).tobytes()
    assert cache.view(1).key(1, 0).tobytes() == k[4:].tobytes()


def test_checkpoint_before_any_forward_refuses():
    """forward_tests.rs:780-815 / cpu.rs:281-295"""
    with pytest.raises(OracleError) as e:
        CpuCompute().cache_checkpoint(3)
    assert e.value.code == orc.STEP_FAILED and "no KV state exists yet" in e.value.msg


def test_speculative_round_trip_rewind_restores_exact_continuation():
    """forward_tests.rs:1098-1151: window 3, prompt 4, block 3, keep 2 -> continuation equals the
    never-speculated route (here bit for bit: same rows through the same arithmetic)."""
    c = cfg([True, False], 3)
    ref = CpuCompute()
    rpos = PositionCache()
    forward(ref, c, rpos, 4, 1)
    # the kept two tokens are the first two rows of the block's seeded tensors
    qw, kw = c.q_heads * c.key_length, c.kv_heads * c.key_length
    for layer, sliding in enumerate(c.sliding):
        q = lcg(200 + layer * 3 + 1, 3 * qw)[: 2 * qw]
        k = lcg(200 + layer * 3 + 2, 3 * kw)[: 2 * kw]
        v = lcg(200 + layer * 3 + 3, 3 * kw)[: 2 * kw]
        ref.attention(c, layer, sliding, q, k, v, rpos)
    rpos.advance(2)
    want = forward(ref, c, rpos, 1, 3)

    spec = CpuCompute()
    pos = PositionCache()
    forward(spec, c, pos, 4, 1)
    assert pos.position() == 4
    cp = spec.cache_checkpoint(3)
    forward(spec, c, pos, 3, 2)
    assert pos.position() == 7
    spec.cache_rewind(cp, 6)
    pos.rewind_to(6)
    spec.cache_release(cp)
    got = forward(spec, c, pos, 1, 3)
    assert pos.position() == 7
    for a, b in zip(got, want):
        assert a.tobytes() == b.tobytes()


def test_rewound_kv_with_unrewound_position_cache_refuses():
    """forward_tests.rs:1154-1181: KV at 2, position cache at 4 -> the attention step refuses by name."""
    c = cfg([True, False], 16)
    b = CpuCompute()
    pos = PositionCache()
    forward(b, c, pos, 2, 1)
    cp = b.cache_checkpoint(2)
    forward(b, c, pos, 2, 2)
    b.cache_rewind(cp, 2)
    b.cache_release(cp)
    with pytest.raises(OracleError) as e:
        forward(b, c, pos, 1, 3)
    assert e.value.code == orc.STEP_FAILED
    assert e.value.msg.startswith("attention:") and "position 2" in e.value.msg and "position 4" in e.value.msg


def test_backend_shape_refusals():
    """cpu.rs:514-556: key/value length mismatch, wrong kind, ragged q, wrong k/v length; cpu.rs:233-243 reshape."""
    c = cfg([True, False], 4)
    b = CpuCompute()
    pos = PositionCache()
    qw, kw = c.q_heads * c.key_length, c.kv_heads * c.key_length
    with pytest.raises(OracleError) as e:
        b.attention(c, 0, False, np.zeros(qw), np.zeros(kw), np.zeros(kw), pos)
    assert e.value.code == orc.STEP_FAILED and "does not match the config's kind" in e.value.msg
    with pytest.raises(OracleError) as e:
        b.attention(c, 0, True, np.zeros(qw + 1), np.zeros(kw), np.zeros(kw), pos)
    assert "not a whole number" in e.value.msg
    with pytest.raises(OracleError) as e:
        b.attention(c, 0, True, np.zeros(qw), np.zeros(kw), np.zeros(kw - 1), pos)
    assert "key/value projections hold" in e.value.msg
    bad = cfg([True, False], 4)
    bad.value_length = 4
    with pytest.raises(OracleError) as e:
        b.attention(bad, 0, True, np.zeros(qw), np.zeros(kw), np.zeros(kw), pos)
    assert "key_length 8 != value_length 4" in e.value.msg
    b.attention(c, 0, True, np.zeros(qw), np.zeros(kw), np.zeros(kw), pos)
    other = cfg([True, False], 5)
    with pytest.raises(OracleError) as e:
        b.attention(other, 1, False, np.zeros(qw), np.zeros(kw), np.zeros(kw), pos)
    assert "different shape" in e.value.msg
    b.reset()
    b.attention(other, 1, False, np.zeros(qw), np.zeros(kw), np.zeros(kw), pos)
