"""GPU parity of the copy paths against the oracle: append (f32 copy and the f32 -> f16 cast), the view
gather and bulk restore.  Bit-exact by contract."""
import numpy as np
import pytest

from itak_torch_rebuild_b200 import CudaComputeError, KvDtype, _lib
from oracle import oracle as orc

from kvparity import assert_rows_bit_equal, assert_view_equal, make_pair, stored

pytestmark = pytest.mark.gpu

DTYPES = [KvDtype.F32, KvDtype.F16]


@pytest.mark.parametrize("dtype", DTYPES)
def test_append_rows_land_in_their_slots_bit_equal(dtype):
    """crates/wgpu-compute/tests/k4_k8_kernels.rs:259-292: window 4, positions 6 and 7 land in ring slots 2
    and 3; on a global layer in slots 6 and 7.  Checked through the view (position order)."""
    kv_width = 256
    gpu, (ref,) = make_pair([4, 0], 2, 2, 128, dtype=dtype, max_context=8, chunk_cap=1)
    base_k, base_v = orc.lcg(60, 6 * kv_width).reshape(6, -1), orc.lcg(61, 6 * kv_width).reshape(6, -1)
    k_rows, v_rows = orc.lcg(62, 2 * kv_width).reshape(2, -1), orc.lcg(63, 2 * kv_width).reshape(2, -1)
    for layer in range(2):
        gpu.append_rows(layer, base_k, base_v, 0)
        ref.append_rows(layer, stored(base_k, dtype), stored(base_v, dtype), 0)
        for i in range(2):
            gpu.append(layer, k_rows[i], v_rows[i], 6 + i)
            ref.append(layer, stored(k_rows[i], dtype), stored(v_rows[i], dtype), 6 + i)
        assert gpu.next_position(layer) == 8
    assert gpu.stored_len(0) == 4 and gpu.stored_len(1) == 8
    for layer in range(2):
        assert_view_equal(gpu, ref, layer, dtype)
    first, k, _ = gpu.view(0)
    assert first == 4
    assert_rows_bit_equal(k[2:], np.stack([stored(k_rows[0], dtype), stored(k_rows[1], dtype)]), dtype, "ring tail")


def test_f16_cast_is_round_to_nearest_even_on_every_class_of_value():
    """crates/wgpu-compute/src/kernels/k1_q4k_gemv.rs:285-329 on the device: normals, halfway cases,
    subnormals, overflow to inf, underflow to signed zero, inf, and NaN -> sign|0x7e00."""
    d = 128
    special = np.array([np.inf, -np.inf, np.nan, 65504.0, 65519.99, 65520.0, -65520.0, 1e9, 2.0 ** -24,
                        2.0 ** -25, -(2.0 ** -25), 2.0 ** -26, 6.1e-5, -6.1e-5, 0.0, -0.0, 1.0009765625,
                        1.00048828125, 1.00146484375, 0.333333, -2.7182817], dtype=np.float32)
    neg_nan = np.array([0xFFC12345, 0x7F800001], dtype=np.uint32).view(np.float32)
    rng = np.random.default_rng(3)
    bits = rng.integers(0, 2 ** 32, size=4 * d - special.size - 2, dtype=np.uint64).astype(np.uint32)
    row = np.concatenate([special, neg_nan, bits.view(np.float32)]).astype(np.float32)
    assert row.size == 4 * d
    gpu, _ = make_pair([0], 4, 4, d, dtype=KvDtype.F16, max_context=4, chunk_cap=1)
    gpu.append(0, row, row[::-1].copy(), 0)
    _, k, v = gpu.view(0)
    assert np.array_equal(k.reshape(-1), orc.f32_to_f16_bits(row))
    assert np.array_equal(v.reshape(-1), orc.f32_to_f16_bits(row[::-1].copy()))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hkv,d", [(1, 1), (2, 3), (2, 4), (1, 8), (4, 64), (8, 128)])
def test_ring_eviction_and_global_growth_match_the_oracle(dtype, hkv, d):
    """crates/attention/tests/cache_tests.rs:38-96 shapes and more: appends past a window evict the oldest;
    global layers keep everything; odd head dims take the element-wise path."""
    gpu, (ref,) = make_pair([4, 0, 7], hkv, hkv, d, dtype=dtype, max_context=32, chunk_cap=3)
    rng = np.random.default_rng(hkv * 100 + d)
    pos = 0
    for rows in (1, 3, 2, 1, 3, 3, 1):
        k = rng.standard_normal((rows, hkv * d)).astype(np.float32)
        v = rng.standard_normal((rows, hkv * d)).astype(np.float32)
        for layer in range(3):
            gpu.append_rows(layer, k, v, pos)
            ref.append_rows(layer, stored(k, dtype), stored(v, dtype), pos)
        pos += rows
        for layer in range(3):
            assert gpu.next_position(layer) == ref.next_position(layer)
            assert gpu.stored_len(layer) == ref.stored_len(layer)
            assert_view_equal(gpu, ref, layer, dtype)


def test_append_refusals_are_named_and_leave_state_untouched():
    """crates/attention/tests/cache_tests.rs:99-131, 186-205."""
    gpu, _ = make_pair([0], 2, 2, 4, dtype=KvDtype.F32, max_context=4, chunk_cap=1)
    with pytest.raises(CudaComputeError) as e:
        gpu.append(0, np.zeros(4), np.zeros(8), 0)
    assert e.value.code == _lib.ERR_SHAPE_MISMATCH and e.value.msg == "k: got 4, expected 8"
    with pytest.raises(CudaComputeError) as e:
        gpu.append(0, np.zeros(8), np.zeros(7), 0)
    assert e.value.code == _lib.ERR_SHAPE_MISMATCH and e.value.msg == "v: got 7, expected 8"
    with pytest.raises(CudaComputeError) as e:
        gpu.append(0, np.zeros(8), np.zeros(8), 1)
    assert e.value.code == _lib.ERR_OUT_OF_ORDER_POSITION
    assert e.value.msg == "layer 0 appends must be in order: expected position 0, got 1"
    assert gpu.stored_len(0) == 0
    with pytest.raises(CudaComputeError) as e:
        gpu.append(5, np.zeros(8), np.zeros(8), 0)
    assert e.value.code == _lib.ERR_INVALID_LAYER and e.value.msg == "layer 5 out of range, cache has 1 layers"
    gpu.append(0, np.zeros(8), np.zeros(8), 0)
    assert gpu.stored_len(0) == 1
    # the fixed allocation is a named refusal, not a write past the end
    gpu.append_rows(0, np.zeros((3, 8)), np.zeros((3, 8)), 1)
    with pytest.raises(CudaComputeError) as e:
        gpu.append(0, np.zeros(8), np.zeros(8), 4)
    assert e.value.code == _lib.ERR_CAPACITY


@pytest.mark.parametrize("dtype", DTYPES)
def test_bulk_restore_matches_append_replay_bitwise(dtype):
    """crates/attention/tests/cache_tests.rs:218-283 on the device: bulk-installed state == replayed state,
    and both continue identically."""
    window = [4, 0, 4]
    hkv, d, tokens = 2, 3, 9
    row = hkv * d

    def rows_for(layer, position):
        k = np.array([np.float32(position * 100 + layer * 10 + i) / np.float32(7) for i in range(row)], np.float32)
        v = np.array([-np.float32(position * 50 + layer * 5 + i) / np.float32(3) for i in range(row)], np.float32)
        return k, v

    replay, _ = make_pair(window, hkv, hkv, d, dtype=dtype, max_context=16, chunk_cap=1)
    bulk, (ref,) = make_pair(window, hkv, hkv, d, dtype=dtype, max_context=16, chunk_cap=1)
    for position in range(tokens):
        for layer in range(3):
            k, v = rows_for(layer, position)
            replay.append(layer, k, v, position)
            ref.append(layer, stored(k, dtype), stored(v, dtype), position)
    for layer, w in enumerate(window):
        first, count = (0, tokens) if not w else (tokens - min(tokens, w), min(tokens, w))
        keys = np.concatenate([rows_for(layer, p)[0] for p in range(first, first + count)])
        values = np.concatenate([rows_for(layer, p)[1] for p in range(first, first + count)])
        bulk.restore_bulk(layer, first, keys, values)
    for layer in range(3):
        assert bulk.next_position(layer) == tokens
        a, b = replay.view(layer), bulk.view(layer)
        assert a[0] == b[0] and a[1].tobytes() == b[1].tobytes() and a[2].tobytes() == b[2].tobytes()
        assert_view_equal(bulk, ref, layer, dtype)
        k, v = rows_for(layer, tokens)
        replay.append(layer, k, v, tokens)
        bulk.append(layer, k, v, tokens)
        a, b = replay.view(layer), bulk.view(layer)
        assert a[1].tobytes() == b[1].tobytes() and a[2].tobytes() == b[2].tobytes()


def test_bulk_restore_refusals_are_named():
    """crates/attention/tests/cache_tests.rs:286-322."""
    gpu, _ = make_pair([4, 0], 1, 1, 2, dtype=KvDtype.F32, max_context=16, chunk_cap=1)
    with pytest.raises(CudaComputeError) as e:
        gpu.restore_bulk(0, 0, np.zeros(10), np.zeros(10))
    assert e.value.code == _lib.ERR_SHAPE_MISMATCH and "bulk restore rows (windowed layer)" in e.value.msg
    with pytest.raises(CudaComputeError) as e:
        gpu.restore_bulk(1, 3, np.zeros(4), np.zeros(4))
    assert e.value.code == _lib.ERR_SHAPE_MISMATCH and "first position (global layer)" in e.value.msg
    gpu.append(0, np.ones(2), np.ones(2), 0)
    with pytest.raises(CudaComputeError) as e:
        gpu.restore_bulk(0, 0, np.zeros(2), np.zeros(2))
    assert e.value.code == _lib.ERR_BULK_RESTORE_NOT_FRESH
    assert e.value.msg.startswith("layer 0 already holds 1 appended positions")
    fresh, _ = make_pair([4, 0], 1, 1, 2, dtype=KvDtype.F32, max_context=16, chunk_cap=1)
    with pytest.raises(CudaComputeError) as e:
        fresh.restore_bulk(0, 0, np.zeros(4), np.zeros(2))
    assert e.value.code == _lib.ERR_SHAPE_MISMATCH and e.value.msg == "bulk restore rows: got 4, expected 2"


def test_slots_are_independent_sequences():
    gpu, refs = make_pair([0, 5], 4, 2, 16, dtype=KvDtype.F16, n_slots=3, max_context=32, chunk_cap=2)
    rng = np.random.default_rng(9)
    for slot, n in enumerate((7, 1, 12)):
        k = rng.standard_normal((n, 32)).astype(np.float32)
        v = rng.standard_normal((n, 32)).astype(np.float32)
        for layer in range(2):
            gpu.append_rows(layer, k, v, 0, slot=slot)
            refs[slot].append_rows(layer, stored(k, KvDtype.F16), stored(v, KvDtype.F16), 0)
    for slot in range(3):
        for layer in range(2):
            assert_view_equal(gpu, refs[slot], layer, KvDtype.F16, slot=slot)
    gpu.reset(slot=1)
    assert gpu.next_position(0, slot=1) == 0 and gpu.next_position(0, slot=0) == 7
    assert_view_equal(gpu, refs[2], 1, KvDtype.F16, slot=2)
