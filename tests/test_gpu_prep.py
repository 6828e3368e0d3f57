"""GPU parity of the on-device attention preparation (per-head RMSNorm + rotary rotation ahead of the append)
against the oracle's composition of the reference's CPU functions (crates/torch-math/src/norm.rs:21-53,
rope_interleaved.rs:65-117, rope.rs:63-117; the fused order is crates/wgpu-compute/src/kernels/k9_attn_prep.rs:1-40).

The prepared rows are f64 arithmetic rounded once to f32 on both sides; they may differ in the last f32 bit (the
order of the f64 sum of squares, the last bit of sin / cos), so stored K rows are compared at 4 f32 ulps (f32 cache)
or one half ulp-step (f16 cache, on at most 0.1 % of the elements), and attention at the task's tolerance."""
import numpy as np
import pytest

from itak_torch_rebuild_b200 import CudaComputeError, KvDtype, PositionCache, _lib
from oracle import oracle as orc

from kvparity import as_f32, assert_attention_close, make_pair, stored

pytestmark = pytest.mark.gpu


def assert_prepared_rows_close(gpu, ref, layer, dtype):
    first, k, v = gpu.view(layer)
    pos, wk, wv = ref.view(layer).dump()
    assert k.shape[0] == len(pos) and (not pos or first == pos[0])
    got_k, want_k = as_f32(k, dtype).reshape(-1), np.asarray(wk, dtype=np.float32).reshape(-1)
    if dtype == KvDtype.F32:
        ulp = np.spacing(np.maximum(np.abs(want_k), np.float32(1e-30)))
        assert np.all(np.abs(got_k - want_k) <= 4 * ulp), "prepared K rows differ by more than 4 ulps"
    else:
        diff = got_k != want_k
        assert diff.mean() <= 1e-3, f"{diff.mean():.2%} of the f16 K elements differ"
        assert np.all(np.abs(got_k - want_k)[diff] <= np.abs(want_k[diff]) * 2.0 ** -9)
    # V rows are not prepared: bit for bit
    got_v = as_f32(v, dtype).reshape(-1)
    assert got_v.tobytes() == np.asarray(wv, dtype=np.float32).reshape(-1).tobytes()


CASES = [
    # hq, hkv, d, norm, base, rotary_dim, pairing
    (8, 2, 128, True, 500000.0, None, 0),   # Glimmer-style: Q/K norm then adjacent-pair rotation
    (32, 8, 128, False, 500000.0, None, 0),  # Llama-3 shape, rotation only
    (32, 4, 64, False, 10000.0, None, 0),   # TinyLlama shape
    (8, 2, 128, True, 10000.0, None, 1),    # half-split (NeoX) pairing
    (4, 2, 64, True, 10000.0, 32, 0),       # partial rotation: channels past rotary_dim pass through
    (4, 4, 96, True, None, None, 0),        # norm only (NoPE layer)
]


@pytest.mark.parametrize("dtype", [KvDtype.F32, KvDtype.F16])
@pytest.mark.parametrize("hq,hkv,d,norm,base,rot,pairing", CASES)
def test_prepared_attention_matches_the_cpu_composition(dtype, hq, hkv, d, norm, base, rot, pairing):
    gpu, (ref,) = make_pair([0], hq, hkv, d, dtype=dtype, max_context=600, chunk_cap=8)
    rng = np.random.default_rng(hq * 131 + d + pairing)
    qw = (1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32) if norm else None
    kw = (1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32) if norm else None
    gpu.set_layer_prep(0, q_norm_weight=qw, k_norm_weight=kw, norm_eps=1e-6, rope_base=base, rotary_dim=rot,
                       pairing=pairing)
    pos = PositionCache()
    # a prefill chunk of 5 rows, a chunk of 8, then single-row decode steps, all with raw rows
    for rows in (5, 8, 1, 1, 1):
        q = rng.standard_normal((rows, hq * d)).astype(np.float32)
        k = rng.standard_normal((rows, hkv * d)).astype(np.float32)
        v = rng.standard_normal((rows, hkv * d)).astype(np.float32)
        got = gpu.attention_prep(0, q, k, v, pos)
        start = pos.position()
        qp = orc.prepare_rows(q, hq, d, start, weight=qw, eps=1e-6, rope_base=base, rotary_dim=rot, pairing=pairing)
        kp = orc.prepare_rows(k, hkv, d, start, weight=kw, eps=1e-6, rope_base=base, rotary_dim=rot, pairing=pairing)
        ref.append_rows(0, stored(kp.reshape(rows, -1), dtype), stored(v, dtype), start)
        want = orc.gqa_attention(qp.reshape(-1), rows, hq, list(range(start, start + rows)), ref.view(0))
        assert_attention_close(got, want, hq, d, dtype, f"rows={rows} at {start}")
        pos.advance(rows)
    assert_prepared_rows_close(gpu, ref, 0, dtype)


def test_prepared_batch_at_large_positions_and_ragged_slots():
    """Continuous-batching shape: ragged positions up to 32K (angles of ~3e4 rad need the f64 range reduction)."""
    hq, hkv, d = 16, 4, 128
    gpu, refs = make_pair([0], hq, hkv, d, dtype=KvDtype.F16, n_slots=3, max_context=33000, chunk_cap=1)
    rng = np.random.default_rng(77)
    gpu.set_layer_prep(0, rope_base=500000.0)
    starts = [32700, 257, 9000]
    # prefill each slot with seeded rows (already "prepared": restore_bulk takes rows as they are)
    for s, n in enumerate(starts):
        k = rng.standard_normal((n, hkv * d)).astype(np.float32)
        v = rng.standard_normal((n, hkv * d)).astype(np.float32)
        gpu.restore_bulk(0, 0, k, v, slot=s)
        refs[s].restore_bulk(0, 0, stored(k, KvDtype.F16), stored(v, KvDtype.F16))
    for step in range(2):
        q = rng.standard_normal((3, hq * d)).astype(np.float32)
        k = rng.standard_normal((3, hkv * d)).astype(np.float32)
        v = rng.standard_normal((3, hkv * d)).astype(np.float32)
        positions = [n + step for n in starts]
        got = gpu.attention_batch_prep(0, [0, 1, 2], positions, 1, q, k, v).reshape(3, hq * d)
        for s in range(3):
            qp = orc.prepare_rows(q[s], hq, d, positions[s], rope_base=500000.0)
            kp = orc.prepare_rows(k[s], hkv, d, positions[s], rope_base=500000.0)
            refs[s].append(0, stored(kp.reshape(-1), KvDtype.F16), stored(v[s], KvDtype.F16), positions[s])
            want = orc.gqa_attention(qp.reshape(-1), 1, hq, [positions[s]], refs[s].view(0))
            assert_attention_close(got[s], want, hq, d, KvDtype.F16, f"slot {s} step {step}")


def test_prep_refusals_leave_state_untouched():
    gpu, (ref,) = make_pair([0, 0], 4, 2, 64, dtype=KvDtype.F32, max_context=64, chunk_cap=4)
    q, k, v = np.zeros(4 * 64, np.float32), np.ones(2 * 64, np.float32), np.ones(2 * 64, np.float32)
    pos = PositionCache()
    with pytest.raises(CudaComputeError) as e:  # no configuration for the layer
        gpu.attention_prep(1, q, k, v, pos)
    assert e.value.code == _lib.ERR_INVALID_ARGUMENT and "itk_layer_prep_set" in e.value.msg
    # the reference's own refusals, by name (rope_interleaved.rs:72-95, norm.rs:34-40)
    with pytest.raises(CudaComputeError) as e:
        gpu.set_layer_prep(0, rope_base=1.0)
    assert e.value.code == _lib.ERR_STEP_FAILED and "base must be finite and > 1" in e.value.msg
    with pytest.raises(CudaComputeError) as e:
        gpu.set_layer_prep(0, rope_base=10000.0, rotary_dim=3)
    assert "rotary_dim must be even" in e.value.msg
    with pytest.raises(CudaComputeError) as e:
        gpu.set_layer_prep(0, q_norm_weight=np.ones(64, np.float32), norm_eps=0.0)
    assert "eps must be finite and > 0" in e.value.msg
    with pytest.raises(CudaComputeError) as e:
        gpu.set_layer_prep(0, q_norm_weight=np.ones(3, np.float32))
    assert e.value.code == _lib.ERR_SHAPE_MISMATCH
    gpu.set_layer_prep(0, rope_base=10000.0)
    with pytest.raises(CudaComputeError) as e:  # position desync is still refused before anything is stored
        desync = PositionCache()
        desync.advance(5)
        gpu.attention_prep(0, q, k, v, desync)
    assert gpu.next_position(0) == 0 and gpu.stored_len(0) == 0
    gpu.attention_prep(0, q, k, v, pos)
    assert gpu.next_position(0) == 1


@pytest.mark.parametrize("dtype", [KvDtype.F32, KvDtype.F16])
@pytest.mark.parametrize("sliding,seed", [(True, 91), (False, 97)])
def test_reference_fused_preparation_cases(dtype, sliding, seed):
    """The two cases the reference checks its fused preparation with
    (crates/wgpu-compute/tests/fused_kernels.rs:68-108, 433-441): 3 rows, 4 query / 2 KV heads, head dim 64, rows
    starting at position 7, base 500000, eps 1e-5, weights lcg + 1, inputs from the test's generator; the sliding case
    has a ring of 8 slots, so the rows land in slots 7, 0, 1.  There the fused kernel is compared with the unfused
    chain; here the device path is compared with the CPU functions that chain stands for."""
    rows, hq, hkv, d, start, base, eps = 3, 4, 2, 64, 7, 500000.0, 1e-5
    window = [5] if sliding else [0]  # ring = window + chunk_cap = 8
    gpu, (ref,) = make_pair(window, hq, hkv, d, dtype=dtype, max_context=16, chunk_cap=3)
    q = orc.lcg(seed, rows * hq * d).reshape(rows, -1)
    k = orc.lcg(seed + 1, rows * hkv * d).reshape(rows, -1)
    v = orc.lcg(seed + 2, rows * hkv * d).reshape(rows, -1)
    q_w = orc.lcg(seed + 3, d) + np.float32(1.0)
    k_w = orc.lcg(seed + 4, d) + np.float32(1.0)
    # positions 0..6 first (prepared rows of any content), so that the case's rows start at 7
    fill_k, fill_v = orc.lcg(seed + 5, start * hkv * d).reshape(start, -1), orc.lcg(seed + 6, start * hkv * d).reshape(start, -1)
    for p in range(start):
        gpu.append(0, fill_k[p], fill_v[p], p)
        ref.append(0, stored(fill_k[p], dtype), stored(fill_v[p], dtype), p)
    gpu.set_layer_prep(0, q_norm_weight=q_w, k_norm_weight=k_w, norm_eps=eps, rope_base=base)
    pos = PositionCache()
    pos.advance(start)
    got = gpu.attention_prep(0, q, k, v, pos)
    qp = orc.prepare_rows(q, hq, d, start, weight=q_w, eps=eps, rope_base=base)
    kp = orc.prepare_rows(k, hkv, d, start, weight=k_w, eps=eps, rope_base=base)
    # the CPU cache's ring is the window itself, so the oracle goes row by row as the CPU backend does
    # (crates/cpu-compute/src/cpu.rs:592-646); the device ring has the chunk's headroom and takes the rows at once
    kp, qp = kp.reshape(rows, -1), qp.reshape(rows, -1)
    want = []
    for r in range(rows):
        ref.append(0, stored(kp[r], dtype), stored(v[r], dtype), start + r)
        want.append(orc.gqa_attention(qp[r], 1, hq, [start + r], ref.view(0)))
    assert_attention_close(got, np.concatenate(want), hq, d, dtype, "fused preparation case")
    assert_prepared_rows_close(gpu, ref, 0, dtype)
