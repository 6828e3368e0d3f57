"""Shared helpers of the GPU parity tests: build the CUDA backend and the oracle side by side and
compare them on the same seeded inputs."""
from __future__ import annotations

import struct

import numpy as np

from itak_torch_rebuild_b200 import CudaCompute, KvDtype
from oracle import oracle as orc

# Attention tolerance: max-abs error relative to the output vector's norm, per (row, head).
TOL_F32_KV = 1e-4
TOL_F16_KV = 2e-3


def pattern_of(layer_window):
    return [orc.LayerKind.Windowed(w) if w else orc.GLOBAL for w in layer_window]


def make_pair(layer_window, hq, hkv, d, *, dtype=KvDtype.F16, n_slots=1, max_context=1024, chunk_cap=8, options=None):
    """(CudaCompute, [oracle KvCache per slot]) over the same geometry."""
    gpu = CudaCompute(len(layer_window), hq, hkv, d, n_slots=n_slots, max_context=max_context, chunk_cap=chunk_cap,
                      kv_dtype=dtype, layer_window=list(layer_window), options=options)
    refs = [orc.KvCache(pattern_of(layer_window), hkv, d) for _ in range(n_slots)]
    return gpu, refs


def stored(x, dtype):
    """What a cache of `dtype` holds for f32 input x, as f32 (the oracle's input)."""
    x = np.asarray(x, dtype=np.float32)
    return orc.round_through_f16(x) if dtype == KvDtype.F16 else x


def as_f32(rows, dtype):
    """Rows read back from the device (raw half bits or f32) as f32 values."""
    return orc.f16_bits_to_f32(rows) if dtype == KvDtype.F16 else np.asarray(rows, dtype=np.float32)


def assert_rows_bit_equal(got, want_f32, dtype, what=""):
    """Device rows equal the oracle's rows bit for bit (half bit patterns for an f16 cache)."""
    want_f32 = np.asarray(want_f32, dtype=np.float32)
    if dtype == KvDtype.F16:
        want_bits = orc.f32_to_f16_bits(want_f32).reshape(got.shape)
        assert got.dtype == np.uint16
        assert np.array_equal(got, want_bits), f"{what}: f16 bit patterns differ"
    else:
        assert got.dtype == np.float32
        assert got.tobytes() == want_f32.reshape(got.shape).tobytes(), f"{what}: f32 bytes differ"


def assert_view_equal(gpu, ref, layer, dtype, slot=0):
    """The device gather equals the oracle view: same first position, same rows, same bits."""
    first, k, v = gpu.view(layer, slot=slot)
    pos, wk, wv = ref.view(layer).dump()
    assert k.shape[0] == len(pos), f"layer {layer}: {k.shape[0]} rows vs {len(pos)}"
    if pos:
        assert first == pos[0]
    assert_rows_bit_equal(k, wk, dtype, f"layer {layer} keys")
    assert_rows_bit_equal(v, wv, dtype, f"layer {layer} values")


def attention_error(got, want, hq, d):
    """max over (row, head) of max-abs error divided by that output vector's L2 norm."""
    got = np.asarray(got, dtype=np.float64).reshape(-1, d)
    want = np.asarray(want, dtype=np.float64).reshape(-1, d)
    norm = np.linalg.norm(want, axis=1)
    norm = np.where(norm > 0, norm, 1.0)
    return float((np.abs(got - want).max(axis=1) / norm).max())


def assert_attention_close(got, want, hq, d, dtype, what=""):
    tol = TOL_F16_KV if dtype == KvDtype.F16 else TOL_F32_KV
    assert np.all(np.isfinite(got)), f"{what}: non-finite output"
    err = attention_error(got, want, hq, d)
    assert err <= tol, f"{what}: error {err:.3e} of the output norm exceeds {tol:.0e}"
    return err


def typed_itkv_bytes(snapshot, fingerprint, hkv, d, window, half):
    """Version 2 of the wire format written out by hand from its documented layout: magic, u32 version 2, u32 element
    type (0 = f32, 1 = half), then the version-1 fields, rows in the element type, FNV-1a-64 over all of it."""
    fp = fingerprint.encode()
    out = bytearray(b"ITKV" + struct.pack("<III", 2, 1 if half else 0, len(fp)) + fp)
    out += struct.pack("<QIII", snapshot.token_count, hkv, d, len(window))
    blocks = [snapshot.layer(i) for i in range(len(window))]
    for w, (first, k, _) in zip(window, blocks):
        out += struct.pack("<B3xQQQ", 1 if w else 0, w, first, k.size // (hkv * d))
    for _, k, v in blocks:
        for rows in (k, v):
            out += (orc.f32_to_f16_bits(rows).astype("<u2") if half else rows.astype("<f4")).tobytes()
    return bytes(out + struct.pack("<Q", orc.checksum(bytes(out))))
