"""The whole-forward host call (itk_attention_layers_host): every layer's attention step of one forward from host
buffers in one call, uploads / kernels / downloads of consecutive layers overlapped on three streams.  Its results
must equal the per-layer host call's bit for bit (same kernels, same launches), match the oracle, leave the cache
bit-equal to the oracle's, and a refusal on any layer must leave every layer where it was."""
import numpy as np
import pytest

from itak_torch_rebuild_b200 import CudaCompute, CudaComputeError, KvDtype, _lib

from kvparity import assert_attention_close, assert_view_equal, make_pair, stored
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


MODES = {
    "default": None,  # a small decode step on an f16 cache runs as one step of the replayable loop; other small forwards in bulk
    "bulk-copies": {"layers_host_decode_loop": 0},
    "pipelined-copies": {"layers_host_decode_loop": 0, "layers_host_bulk_bytes": 0},
}


@pytest.mark.parametrize("mode", list(MODES))
@pytest.mark.parametrize("dtype,d,rows", [(KvDtype.F16, 128, 1), (KvDtype.F16, 128, 7), (KvDtype.F32, 64, 1), (KvDtype.F32, 64, 5)])
def test_one_call_per_forward_equals_one_call_per_layer(dtype, d, rows, mode):
    """Every form of the call: the decode step as a step of the replayable loop (its launches cut the work differently,
    so it agrees with the per-layer call to rounding), a small forward's bulk copies, and the per-layer copies
    pipelined against the kernels (both the same launches as the per-layer call: equal bit for bit)."""
    layer_window, hq, hkv = [0, 0, 24, 0], 8, 2
    lens = [130, 33, 77]
    layers, n = len(layer_window), len(lens)
    loop_step = mode == "default" and dtype == KvDtype.F16 and rows == 1
    a, refs = make_pair(layer_window, hq, hkv, d, dtype=dtype, n_slots=n, max_context=256, chunk_cap=8, options=MODES[mode])
    b, _ = make_pair(layer_window, hq, hkv, d, dtype=dtype, n_slots=n, max_context=256, chunk_cap=8)
    rng = np.random.default_rng(d + rows)
    for slot, ln in enumerate(lens):
        for layer in range(layers):
            k = rng.standard_normal((ln, hkv * d)).astype(np.float32)
            v = rng.standard_normal((ln, hkv * d)).astype(np.float32)
            at = 0
            while at < ln:  # ring layers take at most chunk_cap rows per call
                m = min(8, ln - at)
                a.append_rows(layer, k[at:at + m], v[at:at + m], at, slot=slot)
                b.append_rows(layer, k[at:at + m], v[at:at + m], at, slot=slot)
                at += m
            refs[slot].append_rows(layer, stored(k, dtype), stored(v, dtype), 0)
    slots = list(range(n))
    pos = list(lens)
    for _ in range(3):  # three forwards: the staging is reused, positions move
        q = rng.standard_normal((layers, n, rows, hq * d)).astype(np.float32)
        k = rng.standard_normal((layers, n, rows, hkv * d)).astype(np.float32)
        v = rng.standard_normal((layers, n, rows, hkv * d)).astype(np.float32)
        got = a.attention_layers_host(slots, pos, rows, q, k, v).reshape(layers, n, rows, hq * d)
        for layer in range(layers):
            per_layer = b.attention_batch(layer, slots, pos, rows, q[layer], k[layer], v[layer]).reshape(n, rows, hq * d)
            if loop_step:
                assert np.abs(got[layer] - per_layer).max() <= 1e-5 * np.abs(per_layer).max(), f"layer {layer}"
            else:
                assert got[layer].tobytes() == per_layer.tobytes(), f"layer {layer}: differs from the per-layer call"
            for slot in range(n):
                for r in range(rows):  # the reference's order: append a row, attend it (a ring layer evicts as it goes)
                    refs[slot].append(layer, stored(k[layer, slot, r], dtype), stored(v[layer, slot, r], dtype), pos[slot] + r)
                    want = orc.gqa_attention(q[layer, slot, r], 1, hq, [pos[slot] + r], refs[slot].view(layer))
                    assert_attention_close(got[layer, slot, r], want, hq, d, dtype, f"layer {layer} slot {slot} row {r}")
        pos = [p + rows for p in pos]
    for slot in range(n):
        for layer in range(layers):
            assert a.next_position(layer, slot=slot) == pos[slot]
            assert_view_equal(a, refs[slot], layer, dtype, slot=slot)


def test_a_refusal_on_any_layer_leaves_every_layer_untouched():
    hq, hkv, d = 8, 2, 64
    gpu = CudaCompute(3, hq, hkv, d, n_slots=1, max_context=64, chunk_cap=4, kv_dtype=KvDtype.F16)
    rng = np.random.default_rng(0)
    for layer in range(3):
        gpu.append_rows(layer, rng.standard_normal((10, hkv * d)), rng.standard_normal((10, hkv * d)), 0)
    gpu.append(2, rng.standard_normal(hkv * d), rng.standard_normal(hkv * d), 10)  # layer 2 is one position ahead
    q = rng.standard_normal((3, 1, 1, hq * d)).astype(np.float32)
    kv = rng.standard_normal((3, 1, 1, hkv * d)).astype(np.float32)
    with pytest.raises(CudaComputeError) as e:
        gpu.attention_layers_host([0], [10], 1, q, kv, kv)
    assert e.value.code == _lib.ERR_STEP_FAILED and "layer 2" in e.value.msg
    assert [gpu.next_position(layer) for layer in range(3)] == [10, 10, 11]
    with pytest.raises(CudaComputeError) as e:  # more rows than the chunk cap
        gpu.attention_layers_host([0], [10], 5, np.zeros((3, 1, 5, hq * d), np.float32), np.zeros((3, 1, 5, hkv * d), np.float32),
                                  np.zeros((3, 1, 5, hkv * d), np.float32))
    assert e.value.code == _lib.ERR_CAPACITY


def test_options_are_set_by_name_and_refused_by_name():
    gpu = CudaCompute(1, 8, 2, 64, n_slots=1, max_context=16, chunk_cap=1, kv_dtype=KvDtype.F16)
    for name, value in (("decode_ctas", 120), ("decode_splits", 3), ("pdl", 0), ("decode_fused_sum", 0), ("separate_append", 1),
                        ("force_general", 1), ("verify_tc", 0), ("gather_poll_limit", 1000), ("decode_lanes", 2),
                        ("decode_lane_stagger", 50)):
        gpu.set_option(name, value)
    for name, value in (("no_such_option", 1), ("decode_ctas", -1), ("gather_poll_limit", 0), ("decode_lanes", 3),
                        ("decode_lane_stagger", 1000)):
        with pytest.raises(CudaComputeError) as e:
            gpu.set_option(name, value)
        assert e.value.code == _lib.ERR_INVALID_ARGUMENT and "set_option" in e.value.msg
    gpu.append(0, np.zeros(128), np.zeros(128), 0)
    gpu.resident_begin([0], 2)
    with pytest.raises(CudaComputeError) as e:
        gpu.set_option("pdl", 1)
    assert "resident loop" in e.value.msg
    gpu.resident_end(0)
