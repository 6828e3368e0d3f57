"""GPU parity of GQA attention against the oracle: the reference's hand-computed cases, its seeded kernel
geometries, and sweeps over context length, KV split count, head grouping and cache element type.

Tolerance (stated by the task): max-abs error <= 1e-4 (f32 cache) or 2e-3 (f16 cache) of the output norm."""
import ctypes as C

import numpy as np
import pytest

from itak_torch_rebuild_b200 import CudaCompute, CudaComputeError, KvDtype, PositionCache, _lib
from oracle import oracle as orc

from kvparity import assert_attention_close, assert_view_equal, make_pair, stored

pytestmark = pytest.mark.gpu

DTYPES = [KvDtype.F32, KvDtype.F16]


def fill(gpu, ref, layer, rows, dtype, slot=0):
    for pos, (k, v) in enumerate(rows):
        gpu.append(layer, k, v, pos, slot=slot)
        ref.append(layer, stored(k, dtype), stored(v, dtype), pos)


@pytest.mark.parametrize("dtype", DTYPES)
def test_reference_hand_computed_cases(dtype):
    """crates/attention/tests/attention_tests.rs:30-140 through the CUDA path: the window cannot leak (4.0 vs
    336.0), the causal mask holds (1.0 and ~99.995), GQA 32->2 and 4->2 head sharing."""
    rows = [([1.0], [1000.0]), ([1.0], [3.0]), ([1.0], [5.0])]
    gpu, (ref,) = make_pair([2, 0], 1, 1, 1, dtype=dtype, max_context=8, chunk_cap=1)
    fill(gpu, ref, 0, rows, dtype)
    fill(gpu, ref, 1, rows, dtype)
    assert abs(gpu.gqa_attention(0, [1.0], [2])[0] - 4.0) <= 1e-6
    assert abs(gpu.gqa_attention(1, [1.0], [2])[0] - 336.0) <= 1e-3

    gpu, (ref,) = make_pair([0], 1, 1, 1, dtype=dtype, max_context=8, chunk_cap=1)
    fill(gpu, ref, 0, [([0.0], [1.0]), ([10.0], [100.0]), ([10.0], [1000.0])], dtype)
    out = gpu.gqa_attention(0, [1.0, 1.0], [0, 1])
    assert abs(out[0] - 1.0) <= 1e-6
    assert 99.9 < out[1] < 100.0
    want = orc.gqa_attention([1.0, 1.0], 2, 1, [0, 1], ref.view(0))
    assert abs(out[1] - want[1]) <= 1e-3

    gpu, (ref,) = make_pair([0], 32, 2, 2, dtype=dtype, max_context=8, chunk_cap=1)
    fill(gpu, ref, 0, [([1.0, 0.0, 1.0, 0.0], [10.0, 0.0, 20.0, 0.0])], dtype)
    out = gpu.gqa_attention(0, [1.0, 0.0] * 32, [0])
    for h in range(32):
        assert abs(out[2 * h] - (10.0 if h < 16 else 20.0)) <= 1e-6 and abs(out[2 * h + 1]) <= 1e-6

    gpu, (ref,) = make_pair([0], 4, 2, 1, dtype=dtype, max_context=8, chunk_cap=1)
    fill(gpu, ref, 0, [([1.0, 1.0], [7.0, 9.0])], dtype)
    out = gpu.gqa_attention(0, [1.0] * 4, [0])
    assert np.allclose(out, [7.0, 7.0, 9.0, 9.0], atol=1e-6)


def test_attention_validation_is_named_errors():
    """crates/attention/tests/attention_tests.rs:153-212."""
    gpu, _ = make_pair([0], 2, 2, 2, dtype=KvDtype.F32, max_context=8, chunk_cap=1)
    with pytest.raises(CudaComputeError) as e:
        gpu.gqa_attention(0, [1.0, 0.0, 1.0, 0.0], [0])
    assert e.value.code == _lib.ERR_NO_VISIBLE_KEYS and e.value.msg == "query at position 0 has no visible keys"
    gpu.append(0, [1.0, 0.0, 1.0, 0.0], [1.0, 0.0, 1.0, 0.0], 0)
    with pytest.raises(CudaComputeError) as e:
        gpu.gqa_attention(0, [1.0], [0])
    assert e.value.code == _lib.ERR_SHAPE_MISMATCH and e.value.msg == "q: got 1, expected 4"
    assert gpu.gqa_attention(0, [], []).size == 0
    with pytest.raises(CudaComputeError) as e:
        CudaCompute(1, 3, 2, 2)
    assert e.value.code == _lib.ERR_NON_DIVISIBLE_HEADS


def seeded_case(dtype, hq, hkv, d, n, seed, layer_window=(0,), ctas=None, separate_append=False):
    """Append n seeded N(0,1) rows, then decode steps through the backend's attention call; the outputs and,
    afterwards, the cache contents (the step's rows are stored by the attention launch itself on the f16
    tensor-core path) are compared with the oracle."""
    options = {}
    if ctas is not None:
        options["decode_ctas"] = ctas
    if separate_append:
        options["separate_append"] = 1
    gpu, (ref,) = make_pair(list(layer_window), hq, hkv, d, dtype=dtype, max_context=n + 8, chunk_cap=1, options=options)
    rng = np.random.default_rng(seed)
    worst = 0.0
    for layer in range(len(layer_window)):
        k = rng.standard_normal((n, hkv * d)).astype(np.float32)
        v = rng.standard_normal((n, hkv * d)).astype(np.float32)
        gpu.append_rows(layer, k, v, 0)
        ref.append_rows(layer, stored(k, dtype), stored(v, dtype), 0)
    pos = PositionCache()
    pos.advance(n)
    for step in range(3):
        for layer in range(len(layer_window)):
            q = rng.standard_normal(hq * d).astype(np.float32)
            kn = rng.standard_normal(hkv * d).astype(np.float32)
            vn = rng.standard_normal(hkv * d).astype(np.float32)
            got = gpu.attention(layer, q, kn, vn, pos)
            ref.append(layer, stored(kn, dtype), stored(vn, dtype), pos.position())
            want = orc.gqa_attention(q, 1, hq, [pos.position()], ref.view(layer))
            worst = max(worst, assert_attention_close(got, want, hq, d, dtype, f"n={n} step={step} layer={layer}"))
        pos.advance(1)
    for layer in range(len(layer_window)):
        assert_view_equal(gpu, ref, layer, dtype)
    return worst, gpu.stats()


@pytest.mark.parametrize("n", [1, 2, 15, 16, 17, 63, 64, 65, 127, 128, 129, 300, 1000, 4097])
@pytest.mark.parametrize("d", [64, 128])
def test_f16_decode_kernel_every_tail_length(n, d):
    """The tensor-core decode kernel at every tile-boundary case of the context length."""
    seeded_case(KvDtype.F16, 8, 2, d, n, seed=n * 7 + d)


@pytest.mark.parametrize("ctas", [1, 2, 3, 5, 8, 16, 33, 97, 296])
def test_f16_decode_kernel_every_partition(ctas):
    """The persistent partition and the merge (last CTA combines): any number of CTAs gives the same answer to
    tolerance - one CTA walking every cell in turn, CTAs whose run crosses a cell boundary, and more CTAs
    than tiles."""
    _, st = seeded_case(KvDtype.F16, 8, 2, 128, 700, seed=11, ctas=ctas)
    assert 1 <= st["last_splits"] <= 64


def test_f16_decode_fused_append_equals_the_separate_append():
    """The decode launch that stores the step's new row itself leaves the same cache bits and the same outputs
    as the two-launch form (append kernel, then attention)."""
    a, sa = seeded_case(KvDtype.F16, 32, 8, 128, 515, seed=5)
    b, sb = seeded_case(KvDtype.F16, 32, 8, 128, 515, seed=5, separate_append=True)
    assert sb["kernel_launches"] == sa["kernel_launches"] + 3
    assert abs(a - b) < 1e-6


@pytest.mark.parametrize("hq,hkv", [(1, 1), (2, 1), (4, 1), (8, 1), (16, 1), (32, 8), (64, 8), (32, 2), (12, 4)])
def test_f16_decode_kernel_every_grouping(hq, hkv):
    """GQA groups of 1..16 query heads per KV head (groups above 8 take two head chunks), incl. the
    benchmark shapes 32/8 and 64/8 and the Glimmer shape 32/2."""
    seeded_case(KvDtype.F16, hq, hkv, 128, 333, seed=hq * 31 + hkv)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,d,n", [(4, 2, 8, 40), (32, 4, 64, 520), (8, 8, 32, 129), (6, 3, 24, 77),
                                         (4, 1, 256, 200), (3, 1, 1, 9)])
def test_general_kernel_shapes(dtype, hq, hkv, d, n):
    """The CUDA-core kernel: the TinyLlama shape (32/4, D 64, f32 cache) and head dims the tensor-core
    kernel does not take."""
    if dtype == KvDtype.F16 and d in (64, 128):
        pytest.skip("served by the decode kernel")
    seeded_case(dtype, hq, hkv, d, n, seed=d + n)


@pytest.mark.parametrize("dtype", DTYPES)
def test_sliding_layers_mask_and_wrap(dtype):
    """Window 16 with a ring that wraps many times, next to a global layer: decode steps far past the
    window (crates/attention/src/attention.rs:77-85)."""
    d, hq, hkv = 64, 4, 2
    gpu, (ref,) = make_pair([16, 0], hq, hkv, d, dtype=dtype, max_context=160, chunk_cap=1)
    rng = np.random.default_rng(5)
    pos = PositionCache()
    for step in range(120):
        for layer in range(2):
            q = rng.standard_normal(hq * d).astype(np.float32)
            k = rng.standard_normal(hkv * d).astype(np.float32)
            v = rng.standard_normal(hkv * d).astype(np.float32)
            got = gpu.attention(layer, q, k, v, pos)
            ref.append(layer, stored(k, dtype), stored(v, dtype), step)
            want = orc.gqa_attention(q, 1, hq, [step], ref.view(layer))
            assert_attention_close(got, want, hq, d, dtype, f"step {step} layer {layer}")
        pos.advance(1)
        if step % 40 == 39:
            for layer in range(2):
                assert_view_equal(gpu, ref, layer, dtype)


# crates/wgpu-compute/tests/fused_kernels.rs:506-624: the seven geometries of the flash-vs-two-pass test,
# (rows, stored, first_pos, start_pos, window, ring, seed); q/k/v = lcg(seed), lcg(seed+1), lcg(seed+2).
FLASH_GEOMS = [
    (1, 300, 0, 299, None, None, 31),
    (1, 64, 40, 103, 16, 64, 33),
    (3, 37, 5, 5, None, None, 35),
    (64, 1024, 0, 960, None, None, 37),
    (64, 575, 1425, 1936, 512, 575, 39),
    (64, 2111, 128_961, 131_008, 2048, 2111, 41),
    (16, 300, 0, 284, None, None, 43),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("geom", FLASH_GEOMS, ids=[f"seed{g[-1]}" for g in FLASH_GEOMS])
def test_reference_flash_geometries(dtype, geom):
    """The reference's seeded attention geometries (4 query heads, 2 KV heads, head dim 64): a resident
    store of `stored` rows starting at first_pos, `rows` queries at start_pos.., causal and window masks.
    The row of absolute position p sits at storage row p % capacity of the seeded buffers, as in the
    reference's device buffers.

    When the queries are the newest stored rows the case runs through the backend's attention call (with a
    chunk cap that gives the device ring at least the reference's ring); the one geometry whose
    store extends past its queries runs through the view-level call with positions shifted to start at 0
    (no rotation happens inside attention, so only position differences matter)."""
    rows, stored_n, first_pos, start_pos, window, ring, seed = geom
    hq, hkv, d = 4, 2, 64
    kv_width = hkv * d
    capacity = ring if ring else first_pos + stored_n
    q = orc.lcg(seed, rows * hq * d)
    k_all = orc.lcg(seed + 1, capacity * kv_width).reshape(capacity, kv_width)
    v_all = orc.lcg(seed + 2, capacity * kv_width).reshape(capacity, kv_width)
    end = first_pos + stored_n
    positions = np.arange(first_pos, end)
    k_rows = k_all[positions % capacity]
    v_rows = v_all[positions % capacity]

    # expected, in float64: row r at p = start_pos + r sees stored positions kp <= p with kp > p - window
    want = np.empty_like(q)
    for r in range(rows):
        p = start_pos + r
        vis = [i for i, kp in enumerate(positions) if kp <= p and (window is None or kp > p - window)]
        kk = stored(k_rows[vis], dtype).reshape(len(vis), hkv, d).astype(np.float64)
        vv = stored(v_rows[vis], dtype).reshape(len(vis), hkv, d).astype(np.float64)
        for h in range(hq):
            s = kk[:, h // 2, :] @ q.reshape(rows, hq, d)[r, h].astype(np.float64) / np.sqrt(d)
            w = np.exp(s - s.max())
            w /= w.sum()
            want.reshape(rows, hq, d)[r, h] = w @ vv[:, h // 2, :]

    if end == start_pos + rows:
        chunk_cap = (ring - window + 1) if window else rows
        assert rows <= chunk_cap
        gpu = CudaCompute(1, hq, hkv, d, n_slots=1, max_context=max(end, 8), chunk_cap=chunk_cap, kv_dtype=dtype,
                          layer_window=[window or 0])
        pre = start_pos - first_pos
        if window:
            keep = min(pre, window)
            gpu.restore_bulk(0, start_pos - keep, k_rows[pre - keep:pre], v_rows[pre - keep:pre])
        else:
            assert first_pos == 0
            gpu.restore_bulk(0, 0, k_rows[:pre], v_rows[:pre])
        pos = PositionCache()
        pos.advance(start_pos)
        got = gpu.attention(0, q, k_rows[pre:], v_rows[pre:], pos)
        assert gpu.next_position(0) == end
    else:
        assert window is None
        gpu = CudaCompute(1, hq, hkv, d, n_slots=1, max_context=stored_n, chunk_cap=1, kv_dtype=dtype)
        gpu.restore_bulk(0, 0, k_rows, v_rows)
        got = gpu.gqa_attention(0, q, [start_pos - first_pos + r for r in range(rows)])
    assert_attention_close(got, want, hq, d, dtype, f"geometry seed {seed}")
    if window is None:
        ref = orc.KvCache([orc.GLOBAL], hkv, d)
        ref.restore_bulk(0, 0, stored(k_rows, dtype), stored(v_rows, dtype))
        o = orc.gqa_attention(q, rows, hq, [start_pos - first_pos + r for r in range(rows)], ref.view(0))
        assert_attention_close(got, o, hq, d, dtype, f"geometry seed {seed} vs the oracle routine")


@pytest.mark.parametrize("dtype", DTYPES)
def test_chunked_rows_equal_row_by_row(dtype):
    """A multi-row call (append all rows, then attend causally) equals the reference's row-by-row order
    (crates/cpu-compute/src/cpu.rs:592-646) on global and sliding layers."""
    hq, hkv, d = 8, 2, 64
    gpu, (ref,) = make_pair([0, 6], hq, hkv, d, dtype=dtype, max_context=64, chunk_cap=7)
    rng = np.random.default_rng(21)
    pos = PositionCache()
    for rows in (5, 7, 1, 3, 7):
        for layer in range(2):
            q = rng.standard_normal((rows, hq * d)).astype(np.float32)
            k = rng.standard_normal((rows, hkv * d)).astype(np.float32)
            v = rng.standard_normal((rows, hkv * d)).astype(np.float32)
            got = gpu.attention(layer, q, k, v, pos).reshape(rows, -1)
            for r in range(rows):
                p = pos.position() + r
                ref.append(layer, stored(k[r], dtype), stored(v[r], dtype), p)
                want = orc.gqa_attention(q[r], 1, hq, [p], ref.view(layer))
                assert_attention_close(got[r], want, hq, d, dtype, f"rows={rows} r={r} layer={layer}")
        pos.advance(rows)


def test_batched_slots_with_ragged_lengths():
    """Continuous batching: 5 slots with different context lengths advance together, one token each."""
    hq, hkv, d = 32, 8, 128
    lens = [256, 1, 777, 64, 1500]
    gpu, refs = make_pair([0], hq, hkv, d, dtype=KvDtype.F16, n_slots=5, max_context=1600, chunk_cap=1)
    rng = np.random.default_rng(8)
    for slot, n in enumerate(lens):
        k = rng.standard_normal((n, hkv * d)).astype(np.float32)
        v = rng.standard_normal((n, hkv * d)).astype(np.float32)
        gpu.append_rows(0, k, v, 0, slot=slot)
        refs[slot].append_rows(0, stored(k, KvDtype.F16), stored(v, KvDtype.F16), 0)
    for step in range(3):
        q = rng.standard_normal((5, hq * d)).astype(np.float32)
        k = rng.standard_normal((5, hkv * d)).astype(np.float32)
        v = rng.standard_normal((5, hkv * d)).astype(np.float32)
        order = [3, 0, 4, 1, 2]
        positions = [lens[s] + step for s in order]
        got = gpu.attention_batch(0, order, positions, 1, q, k, v).reshape(5, -1)
        for i, slot in enumerate(order):
            refs[slot].append(0, stored(k[i], KvDtype.F16), stored(v[i], KvDtype.F16), positions[i])
            want = orc.gqa_attention(q[i], 1, hq, [positions[i]], refs[slot].view(0))
            assert_attention_close(got[i], want, hq, d, KvDtype.F16, f"step {step} slot {slot}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows", [1, 5])
def test_pinned_host_buffers_give_the_staged_result(dtype, rows):
    """The host-buffer call takes pageable and pinned host buffers alike (the bench's end-to-end leg passes pinned
    ones by raw pointer): same kernels, same inputs, so the outputs are equal, and so are the rows the calls stored."""
    import torch

    hq, hkv, d, n = 32, 8, 128, 700
    rng = np.random.default_rng(rows + 17)
    k0 = rng.standard_normal((n, hkv * d)).astype(np.float32)
    v0 = rng.standard_normal((n, hkv * d)).astype(np.float32)
    outs, views = [], []
    for pinned in (False, True):
        gpu, _ = make_pair([0], hq, hkv, d, dtype=dtype, max_context=n + 32, chunk_cap=8)
        gpu.append_rows(0, k0, v0, 0)
        r2 = np.random.default_rng(99)
        pos = n
        got = []
        for step in range(3):
            q = r2.standard_normal((rows, hq * d)).astype(np.float32)
            k = r2.standard_normal((rows, hkv * d)).astype(np.float32)
            v = r2.standard_normal((rows, hkv * d)).astype(np.float32)
            if pinned:
                tq, tk, tv = (torch.from_numpy(a).pin_memory() for a in (q, k, v))
                to = torch.empty(rows * hq * d, dtype=torch.float32).pin_memory()
                sl, ps = (C.c_uint32 * 1)(0), (C.c_uint64 * 1)(pos)
                gpu.attention_batch_ptrs(0, sl, ps, 1, rows, tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), to.data_ptr(),
                                         device=False)
                got.append(to.numpy().copy())
            else:
                got.append(gpu.attention_batch(0, [0], [pos], rows, q, k, v).copy())
            pos += rows
        outs.append(np.concatenate(got))
        views.append(gpu.view(0))
    assert np.all(np.isfinite(outs[1]))
    assert attention_error_max(outs[0], outs[1], hq, d) <= 1e-6
    assert views[0][1].tobytes() == views[1][1].tobytes() and views[0][2].tobytes() == views[1][2].tobytes()


def attention_error_max(a, b, hq, d):
    a, b = a.reshape(-1, hq, d), b.reshape(-1, hq, d)
    return float(np.max(np.abs(a - b).max(axis=2) / np.maximum(np.linalg.norm(b, axis=2), 1e-30)))
