"""GPU parity of the speculation seam (checkpoint / rewind / release) and of the backend attention step
against the oracle's restatement of crates/cpu-compute and crates/attention."""
import numpy as np
import pytest

from itak_torch_rebuild_b200 import CudaComputeError, KvDtype, PositionCache, _lib
from oracle import oracle as orc

from kvparity import assert_attention_close, assert_view_equal, make_pair, stored

pytestmark = pytest.mark.gpu

DTYPES = [KvDtype.F32, KvDtype.F16]


def k_row(kv_heads, head_dim, position):
    """crates/attention/tests/checkpoint_tests.rs:17-29: exactly representable markers."""
    return np.array([position * 1000 + (e // head_dim) * 100 + (e % head_dim) for e in range(kv_heads * head_dim)],
                    dtype=np.float32)


def v_row(kv_heads, head_dim, position):
    return k_row(kv_heads, head_dim, position) + np.float32(500)


def append_all(gpu, ref, kv_heads, head_dim, positions, dtype, layers):
    for layer in range(layers):
        for p in positions:
            gpu.append(layer, k_row(kv_heads, head_dim, p), v_row(kv_heads, head_dim, p), p)
            ref.append(layer, stored(k_row(kv_heads, head_dim, p), dtype), stored(v_row(kv_heads, head_dim, p), dtype), p)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("keep", [0, 1, 2, 3])
def test_rewind_leaves_exactly_the_kept_prefix(dtype, keep):
    """crates/attention/tests/checkpoint_tests.rs:80-181 on the device: window 4 next to a global layer,
    prefix 0..=5, a round of 3 appended, rewind to base + keep; the views equal a cache fed only the kept
    prefix, and the sequence continues with no seam."""
    window, hkv, d = [4, 0], 2, 2
    gpu, (ref,) = make_pair(window, hkv, hkv, d, dtype=dtype, max_context=32, chunk_cap=3)
    append_all(gpu, ref, hkv, d, range(6), dtype, 2)
    cp = gpu.cache_checkpoint(3)
    rcp = ref.checkpoint(3)
    assert cp.base() == 6 == rcp.base(0)
    append_all(gpu, ref, hkv, d, [6, 7, 8], dtype, 2)
    gpu.cache_rewind(cp, 6 + keep)
    ref.rewind_to(rcp, 6 + keep)
    gpu.cache_release(cp)
    ref.release(rcp)
    fresh = orc.KvCache([orc.LayerKind.Windowed(4), orc.GLOBAL], hkv, d)
    for layer in range(2):
        for p in range(6 + keep):
            fresh.append(layer, stored(k_row(hkv, d, p), dtype), stored(v_row(hkv, d, p), dtype), p)
    for layer in range(2):
        assert gpu.next_position(layer) == 6 + keep
        assert_view_equal(gpu, ref, layer, dtype)
        assert_view_equal(gpu, fresh, layer, dtype)
    append_all(gpu, ref, hkv, d, [6 + keep], dtype, 2)
    for layer in range(2):
        assert_view_equal(gpu, ref, layer, dtype)


def test_second_rewind_and_divergent_continuation():
    """crates/attention/tests/checkpoint_tests.rs:210-230: rewind, append a divergent row, rewind again."""
    gpu, (ref,) = make_pair([4], 1, 1, 2, dtype=KvDtype.F32, max_context=32, chunk_cap=3)
    append_all(gpu, ref, 1, 2, range(6), KvDtype.F32, 1)
    cp, rcp = gpu.cache_checkpoint(3), ref.checkpoint(3)
    append_all(gpu, ref, 1, 2, [6, 7, 8], KvDtype.F32, 1)
    gpu.cache_rewind(cp, 6)
    ref.rewind_to(rcp, 6)
    gpu.append(0, np.array([9.0, 9.0]), np.array([8.0, 8.0]), 6)
    ref.append(0, np.array([9.0, 9.0]), np.array([8.0, 8.0]), 6)
    assert_view_equal(gpu, ref, 0, KvDtype.F32)
    gpu.cache_rewind(cp, 6)
    ref.rewind_to(rcp, 6)
    gpu.cache_release(cp)
    ref.release(rcp)
    assert_view_equal(gpu, ref, 0, KvDtype.F32)


def test_checkpoint_contract_violations_are_named_refusals():
    """crates/attention/tests/checkpoint_tests.rs:233-316 and crates/cpu-compute/src/cpu.rs:281-295."""
    gpu, refs = make_pair([4, 0], 1, 1, 2, dtype=KvDtype.F32, n_slots=2, max_context=32, chunk_cap=4)
    ref = refs[0]
    with pytest.raises(CudaComputeError) as e:
        gpu.cache_checkpoint(2)
    assert e.value.code == _lib.ERR_STEP_FAILED and "no KV state exists yet" in e.value.msg
    append_all(gpu, ref, 1, 2, [0, 1], KvDtype.F32, 2)
    with pytest.raises(CudaComputeError) as e:
        gpu.cache_checkpoint(0)
    assert e.value.code == _lib.ERR_ZERO_DIMENSION and e.value.msg == "max_round_tokens must be positive, got 0"
    with pytest.raises(CudaComputeError) as e:
        gpu.cache_checkpoint(5)
    assert e.value.code == _lib.ERR_CHECKPOINT_TOO_DEEP
    assert e.value.msg.startswith("checkpoint round bound 5 exceeds the smallest sliding window 4")
    cp = gpu.cache_checkpoint(2)
    with pytest.raises(CudaComputeError) as e:
        gpu.cache_checkpoint(1)
    assert e.value.code == _lib.ERR_CHECKPOINT_BUSY
    append_all(gpu, ref, 1, 2, [2, 3], KvDtype.F32, 2)
    with pytest.raises(CudaComputeError) as e:
        gpu.append(0, k_row(1, 2, 4), v_row(1, 2, 4), 4)
    assert e.value.code == _lib.ERR_CHECKPOINT_RANGE_EXCEEDED
    assert "layer 0 append at position 4" in e.value.msg and "first unsaved position 4" in e.value.msg
    with pytest.raises(CudaComputeError) as e:
        gpu.cache_rewind(cp, 1)
    assert e.value.code == _lib.ERR_REWIND_OUT_OF_RANGE
    assert e.value.msg == "rewind target 1 is outside layer 0's checkpoint range [2, 4]"
    with pytest.raises(CudaComputeError) as e:
        gpu.cache_rewind(cp, 5)
    assert e.value.msg == "rewind target 5 is outside layer 0's checkpoint range [2, 4]"
    assert gpu.next_position(0) == 4
    gpu.cache_release(cp)
    for op in (lambda: gpu.cache_rewind(cp, 2), lambda: gpu.cache_release(cp)):
        with pytest.raises(CudaComputeError) as e:
            op()
        assert e.value.code == _lib.ERR_STALE_CHECKPOINT
    # a handle from another sequence is stale here even with the same serial live
    gpu.append(0, k_row(1, 2, 0), v_row(1, 2, 0), 0, slot=1)
    gpu.append(1, k_row(1, 2, 0), v_row(1, 2, 0), 0, slot=1)
    foreign = gpu.cache_checkpoint(2, slot=1)
    mine = gpu.cache_checkpoint(2, slot=0)
    assert foreign.serial == 1 and mine.serial == 2
    mine2 = type(mine)(foreign.id, mine.serial, mine.base_, mine.max_round_tokens_)
    with pytest.raises(CudaComputeError) as e:
        gpu.cache_rewind(mine2, 4, slot=0)
    assert e.value.code == _lib.ERR_STALE_CHECKPOINT
    gpu.cache_release(mine)
    gpu.cache_release(foreign, slot=1)
    # a reset drops the checkpoint with the sequence
    cp = gpu.cache_checkpoint(2)
    gpu.reset()
    with pytest.raises(CudaComputeError) as e:
        gpu.cache_release(cp)
    assert e.value.code == _lib.ERR_STALE_CHECKPOINT


def cfg_of(sliding, window, hq, hkv, d):
    return orc.BackendConfig(list(sliding), hq, hkv, d, d, window, 10000.0)


def forward_both(gpu, cpu, c, gpos, cpos, rows, seed, dtype):
    """One forward over every layer on both backends.  The CUDA side receives the rows the CPU side
    rotates itself (RoPE is the caller's job on the device path)."""
    qw, kw = c.q_heads * c.key_length, c.kv_heads * c.key_length
    worst = 0.0
    for layer, sliding in enumerate(c.sliding):
        q = orc.lcg(seed * 100 + layer * 3 + 1, rows * qw)
        k = orc.lcg(seed * 100 + layer * 3 + 2, rows * kw)
        v = orc.lcg(seed * 100 + layer * 3 + 3, rows * kw)
        want = cpu.attention(c, layer, sliding, q, k, v, cpos)
        if sliding:
            q_dev = orc.rope_rows(q, c.q_heads, c.key_length, gpos.position(), c.rope_freq_base_swa).reshape(-1)
            k_dev = orc.rope_rows(k, c.kv_heads, c.key_length, gpos.position(), c.rope_freq_base_swa).reshape(-1)
        else:
            q_dev, k_dev = q, k
        got = gpu.attention(layer, q_dev, k_dev, v, gpos)
        worst = max(worst, assert_attention_close(got, want, c.q_heads, c.key_length, dtype, f"layer {layer}"))
    gpos.advance(rows)
    cpos.advance(rows)
    return worst


def test_attention_matches_cpu_step_for_step():
    """crates/wgpu-compute/tests/k4_k8_kernels.rs:296-356: a 3-token prefill then decode steps out to
    position 6 at window 4, every layer compared with the CPU backend step for step (f32 cache)."""
    c = cfg_of([True, False, True], 4, 4, 2, 64)
    gpu, _ = make_pair([4, 0, 4], 4, 2, 64, dtype=KvDtype.F32, max_context=32, chunk_cap=3)
    cpu = orc.CpuCompute()
    gpos, cpos = PositionCache(), orc.PositionCache()
    for i, rows in enumerate([3, 1, 1, 1, 1]):
        forward_both(gpu, cpu, c, gpos, cpos, rows, 10 + i, KvDtype.F32)
    assert gpos.position() == 7
    ref = cpu.kv_cache(c)
    for layer in range(3):
        assert_view_equal(gpu, ref, layer, KvDtype.F32)


def test_speculative_round_trip_rewind_restores_exact_continuation():
    """crates/cpu-compute/tests/forward_tests.rs:1098-1151: window 3, prompt 4, checkpoint(3), block of 3,
    rewind to keep 2, release, continue; the continuation equals the never-speculated route, and equals
    the CPU backend's."""
    c = cfg_of([True, False], 3, 4, 2, 64)
    dtype = KvDtype.F32
    never, _ = make_pair([3, 0], 4, 2, 64, dtype=dtype, max_context=32, chunk_cap=4)
    cpu_never = orc.CpuCompute()
    gp, cp_ = PositionCache(), orc.PositionCache()
    forward_both(never, cpu_never, c, gp, cp_, 4, 1, dtype)
    # keep the first two rows of the block's seeded tensors
    qw, kw = c.q_heads * c.key_length, c.kv_heads * c.key_length
    for layer, sliding in enumerate(c.sliding):
        q = orc.lcg(200 + layer * 3 + 1, 3 * qw)[: 2 * qw]
        k = orc.lcg(200 + layer * 3 + 2, 3 * kw)[: 2 * kw]
        v = orc.lcg(200 + layer * 3 + 3, 3 * kw)[: 2 * kw]
        cpu_never.attention(c, layer, sliding, q, k, v, cp_)
        if sliding:
            q = orc.rope_rows(q, c.q_heads, c.key_length, 4, c.rope_freq_base_swa).reshape(-1)
            k = orc.rope_rows(k, c.kv_heads, c.key_length, 4, c.rope_freq_base_swa).reshape(-1)
        never.attention(layer, q, k, v, gp)
    gp.advance(2)
    cp_.advance(2)

    spec, _ = make_pair([3, 0], 4, 2, 64, dtype=dtype, max_context=32, chunk_cap=4)
    cpu_spec = orc.CpuCompute()
    sp, csp = PositionCache(), orc.PositionCache()
    forward_both(spec, cpu_spec, c, sp, csp, 4, 1, dtype)
    assert sp.position() == 4
    checkpoint = spec.cache_checkpoint(3)
    ccheckpoint = cpu_spec.cache_checkpoint(3)
    forward_both(spec, cpu_spec, c, sp, csp, 3, 2, dtype)
    assert sp.position() == 7
    spec.cache_rewind(checkpoint, 6)
    sp.rewind_to(6)
    spec.cache_release(checkpoint)
    cpu_spec.cache_rewind(ccheckpoint, 6)
    csp.rewind_to(6)
    cpu_spec.cache_release(ccheckpoint)
    for layer in range(2):
        a, b = never.view(layer), spec.view(layer)
        assert a[0] == b[0] and a[1].tobytes() == b[1].tobytes() and a[2].tobytes() == b[2].tobytes()
        assert_view_equal(spec, cpu_spec.kv_cache(c), layer, dtype)
    # the continuation: identical inputs through both device routes give identical bits
    for layer, sliding in enumerate(c.sliding):
        q = orc.lcg(300 + layer * 3 + 1, qw)
        k = orc.lcg(300 + layer * 3 + 2, kw)
        v = orc.lcg(300 + layer * 3 + 3, kw)
        want = cpu_spec.attention(c, layer, sliding, q, k, v, csp)
        if sliding:
            q = orc.rope_rows(q, c.q_heads, c.key_length, 6, c.rope_freq_base_swa).reshape(-1)
            k = orc.rope_rows(k, c.kv_heads, c.key_length, 6, c.rope_freq_base_swa).reshape(-1)
        a = never.attention(layer, q, k, v, gp)
        b = spec.attention(layer, q, k, v, sp)
        assert a.tobytes() == b.tobytes()
        assert_attention_close(b, want, c.q_heads, c.key_length, dtype, f"continuation layer {layer}")


def test_rewound_kv_with_unrewound_position_cache_refuses():
    """crates/cpu-compute/tests/forward_tests.rs:1154-1181: KV at 2, position cache at 4."""
    gpu, _ = make_pair([16, 0], 4, 2, 64, dtype=KvDtype.F16, max_context=32, chunk_cap=2)
    rng = np.random.default_rng(2)
    pos = PositionCache()

    def fwd(rows):
        for layer in range(2):
            gpu.attention(layer, rng.standard_normal(rows * 256), rng.standard_normal(rows * 128),
                          rng.standard_normal(rows * 128), pos)
        pos.advance(rows)

    fwd(2)
    cp = gpu.cache_checkpoint(2)
    fwd(2)
    gpu.cache_rewind(cp, 2)
    gpu.cache_release(cp)
    with pytest.raises(CudaComputeError) as e:
        fwd(1)
    assert e.value.code == _lib.ERR_STEP_FAILED
    assert e.value.msg.startswith("attention:") and "position 2" in e.value.msg and "position 4" in e.value.msg
    assert gpu.next_position(0) == 2


def test_attention_shape_refusals():
    """crates/cpu-compute/src/cpu.rs:532-556."""
    gpu, _ = make_pair([0], 4, 2, 64, dtype=KvDtype.F16, max_context=32, chunk_cap=2)
    pos = PositionCache()
    with pytest.raises(CudaComputeError) as e:
        gpu.attention(0, np.zeros(257), np.zeros(128), np.zeros(128), pos)
    assert e.value.code == _lib.ERR_STEP_FAILED and "not a whole number of 256-wide rows" in e.value.msg
    with pytest.raises(CudaComputeError) as e:
        gpu.attention(0, np.zeros(256), np.zeros(128), np.zeros(127), pos)
    assert "key/value projections hold 128/127 elements for 1 rows, expected 128/128" in e.value.msg
    with pytest.raises(CudaComputeError) as e:
        gpu.attention(0, np.zeros(768), np.zeros(384), np.zeros(384), pos)
    assert e.value.code == _lib.ERR_CAPACITY and "chunk cap" in e.value.msg
    assert gpu.next_position(0) == 0
