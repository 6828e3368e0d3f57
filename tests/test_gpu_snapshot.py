"""GPU parity of the prefix-KV seam: snapshot capture, restore (install) and import from host rows, against
the oracle's KvSnapshot (crates/itak-kv/src/snapshot.rs) - bit-exact by contract."""
import numpy as np
import pytest

from itak_torch_rebuild_b200 import CudaCompute, CudaComputeError, KvDtype, PositionCache, _lib
from oracle import oracle as orc

from kvparity import (as_f32, assert_attention_close, assert_rows_bit_equal, assert_view_equal, make_pair, stored,
                      typed_itkv_bytes)

pytestmark = pytest.mark.gpu

DTYPES = [KvDtype.F32, KvDtype.F16]


def fill(gpu, ref, window, hkv, d, tokens, dtype, seed=0, slot=0):
    rng = np.random.default_rng(seed)
    for layer in range(len(window)):
        k = rng.standard_normal((tokens, hkv * d)).astype(np.float32)
        v = rng.standard_normal((tokens, hkv * d)).astype(np.float32)
        at = 0
        while at < tokens:  # chunks no larger than the backend's chunk cap on ring layers
            n = min(gpu.chunk_cap, tokens - at)
            gpu.append_rows(layer, k[at:at + n], v[at:at + n], at, slot=slot)
            at += n
        if ref is not None:
            ref.append_rows(layer, stored(k, dtype), stored(v, dtype), 0)


def assert_snapshot_equals_oracle(snap, osnap, dtype, layers):
    assert snap.token_count == osnap.token_count
    for layer in range(layers):
        first, k, v = snap.layer(layer)
        ofirst, ok, ov = osnap.layer(layer)
        assert first == ofirst
        assert_rows_bit_equal(k, ok, dtype, f"snapshot layer {layer} keys")
        assert_rows_bit_equal(v, ov, dtype, f"snapshot layer {layer} values")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens", [1, 3, 4, 10, 70])
def test_capture_equals_the_oracle_snapshot(dtype, tokens):
    """crates/itak-kv/src/snapshot.rs:247-302: per layer the visible rows in position order; the
    70-token / window 4 / chunk 64 case wraps the ring, the corruption case of
    crates/wgpu-compute/tests/prefix_kv_session.rs:5-13."""
    window, hkv, d = [4, 0, 4], 2, 3
    gpu, (ref,) = make_pair(window, 2, hkv, d, dtype=dtype, max_context=128, chunk_cap=64)
    fill(gpu, ref, window, hkv, d, tokens, dtype, seed=tokens)
    snap = gpu.capture_prefix_snapshot()
    osnap = orc.KvSnapshot.capture(ref, "model-a")
    assert_snapshot_equals_oracle(snap, osnap, dtype, 3)
    assert snap.payload_bytes == sum(min(tokens, w) if w else tokens for w in window) * hkv * d * 2 * (
        2 if dtype == KvDtype.F16 else 4)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens", [3, 9, 70])
def test_restore_rebuilds_the_same_views_and_continues(dtype, tokens):
    """crates/itak-kv/src/snapshot.rs:656-690 and crates/itak-kv/tests/restore_fixture.rs:116-189: a restored
    slot has the captured slot's views and positions, and continues bit-identically with it."""
    window, hq, hkv, d = [4, 0, 0, 4], 4, 2, 8
    gpu, refs = make_pair(window, hq, hkv, d, dtype=dtype, n_slots=2, max_context=128, chunk_cap=64)
    ref = refs[0]
    fill(gpu, ref, window, hkv, d, tokens, dtype, seed=tokens + 1)
    snap = gpu.capture_prefix_snapshot(slot=0)
    fill(gpu, None, window, hkv, d, 5, dtype, seed=99, slot=1)  # slot 1 holds another sequence first
    assert gpu.install_prefix_snapshot(snap, slot=1) == tokens
    restored = orc.KvSnapshot.capture(ref, "m").restore()
    for layer in range(4):
        assert gpu.next_position(layer, slot=1) == tokens
        assert_view_equal(gpu, ref, layer, dtype, slot=1)
        assert_view_equal(gpu, restored, layer, dtype, slot=1)
    rng = np.random.default_rng(4)
    p0, p1 = PositionCache(), PositionCache()
    p0.advance(tokens)
    p1.advance(tokens)
    for step in range(5):
        for layer in range(4):
            q = rng.standard_normal(hq * d).astype(np.float32)
            k = rng.standard_normal(hkv * d).astype(np.float32)
            v = rng.standard_normal(hkv * d).astype(np.float32)
            cold = gpu.attention(layer, q, k, v, p0, slot=0)
            warm = gpu.attention(layer, q, k, v, p1, slot=1)
            assert cold.tobytes() == warm.tobytes()
            ref.append(layer, stored(k, dtype), stored(v, dtype), tokens + step)
            want = orc.gqa_attention(q, 1, hq, [tokens + step], ref.view(layer))
            assert_attention_close(warm, want, hq, d, dtype, f"step {step} layer {layer}")
        p0.advance(1)
        p1.advance(1)


@pytest.mark.parametrize("dtype", DTYPES)
def test_import_from_host_rows_matches_the_oracle_restore(dtype):
    """A snapshot built from the ITKV layer blocks of the oracle (f32 rows, crates/itak-kv/src/snapshot.rs:13-29)
    installs the state the oracle's restore builds."""
    window, hkv, d, tokens = [4, 0, 4], 2, 8, 11
    ref = orc.KvCache([orc.LayerKind.Windowed(w) if w else orc.GLOBAL for w in window], hkv, d)
    rng = np.random.default_rng(6)
    for layer in range(3):
        ref.append_rows(layer, rng.standard_normal((tokens, hkv * d)), rng.standard_normal((tokens, hkv * d)), 0)
    osnap = orc.KvSnapshot.from_bytes(orc.KvSnapshot.capture(ref, "m").to_bytes(),
                                      orc.KvGeometry(ref.pattern, hkv, d))
    gpu = CudaCompute(3, 2, hkv, d, n_slots=1, max_context=64, chunk_cap=8, kv_dtype=dtype, layer_window=window)
    snap = gpu.snapshot_from_host(osnap.token_count, [osnap.layer(i) for i in range(3)])
    gpu.install_prefix_snapshot(snap)
    want = osnap.restore()
    if dtype == KvDtype.F16:
        rounded = orc.KvCache(ref.pattern, hkv, d)
        for i in range(3):
            first, k, v = osnap.layer(i)
            rounded.restore_bulk(i, first, stored(k, dtype), stored(v, dtype))
        want = rounded
    for layer in range(3):
        assert gpu.next_position(layer) == tokens
        assert_view_equal(gpu, want, layer, dtype)


def test_snapshot_refusals_are_named_and_leave_the_slot_untouched():
    """crates/itak-kv/src/snapshot.rs:693-706 (divergent cache) and crates/wgpu-compute/src/session.rs:410-467
    (geometry, empty, oversized) - each before any state moves."""
    window, hkv, d = [4, 0], 2, 8
    gpu, _ = make_pair(window, 2, hkv, d, dtype=KvDtype.F16, n_slots=2, max_context=16, chunk_cap=8)
    gpu.append(0, np.zeros(16), np.zeros(16), 0)
    with pytest.raises(CudaComputeError) as e:
        gpu.capture_prefix_snapshot()
    assert e.value.code == _lib.ERR_INCOHERENT_CACHE
    gpu.append(1, np.zeros(16), np.zeros(16), 0)
    snap = gpu.capture_prefix_snapshot()
    other = CudaCompute(2, 2, hkv, 16, n_slots=1, max_context=16, chunk_cap=8, kv_dtype=KvDtype.F16,
                        layer_window=window)
    other.append(0, np.ones(32), np.ones(32), 0)
    other.append(1, np.ones(32), np.ones(32), 0)
    with pytest.raises(CudaComputeError) as e:
        other.install_prefix_snapshot(snap)
    assert e.value.code == _lib.ERR_GEOMETRY_MISMATCH and "geometry" in e.value.msg
    assert other.next_position(0) == 1
    empty = gpu.capture_prefix_snapshot(slot=1)
    assert empty.token_count == 0
    with pytest.raises(CudaComputeError) as e:
        gpu.install_prefix_snapshot(empty, slot=0)
    assert e.value.code == _lib.ERR_STEP_FAILED and "zero tokens" in e.value.msg
    assert gpu.next_position(0) == 1
    big = CudaCompute(2, 2, hkv, d, n_slots=1, max_context=64, chunk_cap=8, kv_dtype=KvDtype.F16, layer_window=window)
    fill(big, None, window, hkv, d, 20, KvDtype.F16)
    with pytest.raises(CudaComputeError) as e:
        gpu.install_prefix_snapshot(big.capture_prefix_snapshot())
    assert e.value.code == _lib.ERR_STEP_FAILED and "context capacity" in e.value.msg
    with pytest.raises(CudaComputeError) as e:
        gpu.snapshot_from_host(5, [(0, np.zeros(5 * 16), np.zeros(5 * 16)), (0, np.zeros(5 * 16), np.zeros(5 * 16))])
    assert e.value.code == _lib.ERR_INCONSISTENT_SNAPSHOT and "first stored position" in e.value.msg


def test_shared_prefix_snapshot_at_full_size_round_trips():
    """The prefix-KV configuration at full size: 2048-token prefix, 32 layers, 8 KV heads, head dim 128, f16
    (256 MiB), captured once and restored into other sessions.  Size-independent properties: a restore
    followed by a capture reproduces the snapshot byte for byte (sampled layers compared on the host), every
    session reports position 2048, and decode attention over a restored session equals decode attention
    over the original, bit for bit (launched alone) and to rounding (launched as one batch)."""
    layers, hq, hkv, d, tokens, sessions = 32, 32, 8, 128, 2048, 4
    gpu = CudaCompute(layers, hq, hkv, d, n_slots=sessions + 1, max_context=tokens + 64, chunk_cap=512,
                      kv_dtype=KvDtype.F16)
    rng = np.random.default_rng(12)
    for layer in range(layers):
        k = rng.standard_normal((tokens, hkv * d)).astype(np.float32)
        v = rng.standard_normal((tokens, hkv * d)).astype(np.float32)
        gpu.append_rows(layer, k, v, 0, slot=0)
        if layer == 5:
            keep_k, keep_v = k, v
    snap = gpu.capture_prefix_snapshot(slot=0)
    assert snap.payload_bytes == 268_435_456
    first, k5, v5 = snap.layer(5)
    assert first == 0
    assert_rows_bit_equal(k5, keep_k, KvDtype.F16, "layer 5 keys")
    assert_rows_bit_equal(v5, keep_v, KvDtype.F16, "layer 5 values")
    for s in range(1, sessions + 1):
        assert gpu.install_prefix_snapshot(snap, slot=s) == tokens
    again = gpu.capture_prefix_snapshot(slot=sessions)
    for layer in (0, 5, 17, 31):
        a, b = snap.layer(layer), again.layer(layer)
        assert a[0] == b[0] and a[1].tobytes() == b[1].tobytes() and a[2].tobytes() == b[2].tobytes()
    # One launch per session: the kernel's work partition (and with it the order of the f32 sums) depends on
    # the batch a sequence is launched with, so bit-equality is a property of equal launches.
    q = rng.standard_normal((1, hq * d)).astype(np.float32)
    kn = rng.standard_normal((1, hkv * d)).astype(np.float32)
    vn = rng.standard_normal((1, hkv * d)).astype(np.float32)
    outs = [gpu.attention_batch(7, [s], [tokens], 1, q, kn, vn).copy() for s in range(sessions + 1)]
    for s in range(1, sessions + 1):
        assert outs[s].tobytes() == outs[0].tobytes()
    # and as one batch the sessions agree to rounding
    qb, kb, vb = (np.repeat(x, sessions + 1, axis=0) for x in (q, kn, vn))
    out = gpu.attention_batch(9, list(range(sessions + 1)), [tokens] * (sessions + 1), 1, qb, kb, vb)
    out = out.reshape(sessions + 1, -1)
    assert np.abs(out - out[0]).max() <= 1e-5 * np.abs(out[0]).max()


@pytest.mark.parametrize("dtype", DTYPES)
def test_itkv_bytes_equal_the_oracle_encoding_and_round_trip(dtype):
    """crates/itak-kv/src/snapshot.rs:13-29, 381-540: the device snapshot's ITKV bytes equal, byte for byte, the
    oracle's encoding of the same cache (wrapped ring layers included), and bytes produced by the oracle install the
    oracle's state on the device."""
    import struct

    window, hkv, d, tokens = [4, 0, 4], 2, 8, 70
    gpu, (ref,) = make_pair(window, 2, hkv, d, dtype=dtype, max_context=128, chunk_cap=64)
    fill(gpu, ref, window, hkv, d, tokens, dtype, seed=21)
    want = orc.KvSnapshot.capture(ref, "model-a").to_bytes()
    got = gpu.capture_prefix_snapshot().to_itkv("model-a")
    assert got == want
    assert struct.unpack_from("<Q", got, len(got) - 8)[0] == orc.checksum(got[:-8])

    other = CudaCompute(3, 2, hkv, d, n_slots=1, max_context=128, chunk_cap=64, kv_dtype=dtype, layer_window=window)
    snap = other.snapshot_from_itkv(want, expected_fingerprint="model-a")
    assert snap.token_count == tokens
    other.install_prefix_snapshot(snap)
    for layer in range(3):
        assert_view_equal(other, ref, layer, dtype)
    assert other.capture_prefix_snapshot().to_itkv("model-a") == want


def test_itkv_decode_refusals_are_named():
    """crates/itak-kv/src/snapshot.rs:709-813 and 345-371 on the device side's decoder."""
    import struct

    window, hkv, d = [4, 0], 2, 4
    gpu, (ref,) = make_pair(window, 2, hkv, d, dtype=KvDtype.F32, max_context=32, chunk_cap=8)
    fill(gpu, ref, window, hkv, d, 5, KvDtype.F32, seed=2)
    good = gpu.capture_prefix_snapshot().to_itkv("model-a")

    def refusal(data, fingerprint=None):
        with pytest.raises(CudaComputeError) as e:
            gpu.snapshot_from_itkv(data, fingerprint)
        return e.value

    flipped = bytearray(good)
    flipped[len(good) - 12] ^= 0xFF
    assert refusal(bytes(flipped)).code == _lib.ERR_CHECKSUM_MISMATCH
    assert refusal(good[:8]).code == _lib.ERR_TRUNCATED
    bad = bytearray(good)
    bad[0] = ord("X")
    assert refusal(bytes(bad)).code == _lib.ERR_BAD_MAGIC
    v3 = bytearray(good)
    v3[4] = 3
    assert refusal(bytes(v3)).code == _lib.ERR_UNSUPPORTED_VERSION
    e = refusal(good + b"\0")
    assert e.code == _lib.ERR_INCONSISTENT_SNAPSHOT and "trailing" in e.msg
    forged = b"ITKV" + struct.pack("<IIQIII", 1, 0, 0, 1, 1, 0xFFFFFFFF)
    assert refusal(forged).code == _lib.ERR_INCONSISTENT_SNAPSHOT
    overflow = b"ITKV" + struct.pack("<II", 1, 1) + b"x" + struct.pack("<QIII", 1 << 32, 65536, 65536, 1)
    overflow += bytes(4) + struct.pack("<QQQ", 0, 0, 0)
    overflow += struct.pack("<Q", orc.checksum(overflow))
    assert refusal(overflow).code == _lib.ERR_INCONSISTENT_SNAPSHOT
    assert refusal(good, "model-b").code == _lib.ERR_FINGERPRINT_MISMATCH
    foreign = CudaCompute(2, 2, hkv, 8, n_slots=1, max_context=32, chunk_cap=8, kv_dtype=KvDtype.F32, layer_window=window)
    with pytest.raises(CudaComputeError) as e:
        foreign.snapshot_from_itkv(good, "model-a")
    assert e.value.code == _lib.ERR_GEOMETRY_MISMATCH
    gpu.snapshot_from_itkv(good, "model-a")


def test_itkv_version_2_keeps_half_rows_as_they_are():
    """The typed format version (no counterpart in the reference, which refuses to snapshot an f16 cache,
    crates/wgpu-compute/src/session.rs:383-398): the bytes equal the hand-written encoding of the oracle's captured
    rows as half bit patterns, take half the payload of version 1, install bit for bit into another f16 backend, and
    widen exactly into an f32 one; version 1 of the same snapshot still equals the oracle's f32 encoding."""
    window, hkv, d, tokens = [4, 0, 4], 2, 8, 70
    gpu, (ref,) = make_pair(window, 2, hkv, d, dtype=KvDtype.F16, max_context=128, chunk_cap=64)
    fill(gpu, ref, window, hkv, d, tokens, KvDtype.F16, seed=33)
    oracle_snap = orc.KvSnapshot.capture(ref, "model-a")
    snap = gpu.capture_prefix_snapshot()
    got = snap.to_itkv("model-a", version=2)
    assert got == typed_itkv_bytes(oracle_snap, "model-a", hkv, d, window, half=True)
    v1 = snap.to_itkv("model-a", version=1)
    assert v1 == oracle_snap.to_bytes()
    payload = sum(oracle_snap.layer(i)[1].size for i in range(3)) * 2
    assert len(v1) - len(got) == payload * 2 - 4  # half the row bytes, one more header word

    other = CudaCompute(3, 2, hkv, d, n_slots=1, max_context=128, chunk_cap=64, kv_dtype=KvDtype.F16, layer_window=window)
    up = other.snapshot_from_itkv(got, expected_fingerprint="model-a")
    assert up.token_count == tokens
    other.install_prefix_snapshot(up)
    for layer in range(3):
        assert_view_equal(other, ref, layer, KvDtype.F16)
    assert other.capture_prefix_snapshot().to_itkv("model-a", version=2) == got

    wide = CudaCompute(3, 2, hkv, d, n_slots=1, max_context=128, chunk_cap=64, kv_dtype=KvDtype.F32, layer_window=window)
    wide.install_prefix_snapshot(wide.snapshot_from_itkv(got, expected_fingerprint="model-a"))
    for layer in range(3):
        assert_view_equal(wide, ref, layer, KvDtype.F32)  # the oracle holds the f16-rounded values as f32
    # an f32 cache written as version 2 declares f32 rows
    assert wide.capture_prefix_snapshot().to_itkv("model-a", version=2) == typed_itkv_bytes(
        oracle_snap, "model-a", hkv, d, window, half=False)
    with pytest.raises(CudaComputeError) as e:
        snap.to_itkv("model-a", version=3)
    assert e.value.code == _lib.ERR_UNSUPPORTED_VERSION


def test_itkv_version_2_decode_refusals_are_named():
    """The strict decoder's refusals hold for the typed version too: unknown element type, truncation inside the
    rows, trailing bytes, a flipped payload bit, and a row count whose byte size overflows."""
    import struct

    window, hkv, d = [4, 0], 2, 4
    gpu, (ref,) = make_pair(window, 2, hkv, d, dtype=KvDtype.F16, max_context=32, chunk_cap=8)
    fill(gpu, ref, window, hkv, d, 5, KvDtype.F16, seed=2)
    good = gpu.capture_prefix_snapshot().to_itkv("model-a", version=2)

    def refusal(data, fingerprint=None):
        with pytest.raises(CudaComputeError) as e:
            gpu.snapshot_from_itkv(data, fingerprint)
        return e.value

    def resum(data):
        return bytes(data[:-8]) + struct.pack("<Q", orc.checksum(bytes(data[:-8])))

    tag = bytearray(good)
    tag[8] = 7
    e = refusal(resum(tag))
    assert e.code == _lib.ERR_INCONSISTENT_SNAPSHOT and "element type" in e.msg
    assert refusal(good[:10]).code == _lib.ERR_TRUNCATED
    assert refusal(good[: len(good) - 20]).code == _lib.ERR_TRUNCATED
    e = refusal(good + b"\0")
    assert e.code == _lib.ERR_INCONSISTENT_SNAPSHOT and "trailing" in e.msg
    flipped = bytearray(good)
    flipped[len(good) - 12] ^= 0x01
    assert refusal(bytes(flipped)).code == _lib.ERR_CHECKSUM_MISMATCH
    overflow = b"ITKV" + struct.pack("<III", 2, 1, 1) + b"x" + struct.pack("<QIII", 1 << 33, 65536, 65536, 1)
    overflow += bytes(4) + struct.pack("<QQQ", 0, 0, 1 << 33)
    overflow += struct.pack("<Q", orc.checksum(overflow))
    assert refusal(overflow).code == _lib.ERR_INCONSISTENT_SNAPSHOT
    assert refusal(good, "model-b").code == _lib.ERR_FINGERPRINT_MISMATCH
    gpu.snapshot_from_itkv(good, "model-a")
