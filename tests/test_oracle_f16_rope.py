"""The oracle's f32<->f16 conversions and RoPE against the reference's tests:
crates/wgpu-compute/tests/kv_f16.rs:81-173, crates/torch-math/src/rope.rs:133-201,
crates/torch-math/src/rope_interleaved.rs:125-201."""
import numpy as np
import pytest

from oracle import oracle as orc
from oracle.oracle import OracleError


def test_every_finite_f16_round_trips_exactly():
    """kv_f16.rs:81-98: all 63,488 finite f16 patterns decode and re-encode to themselves."""
    bits = np.concatenate([np.arange(0x0000, 0x7C00), np.arange(0x8000, 0xFC00)]).astype(np.uint16)
    assert bits.size == 63_488
    values = orc.f16_bits_to_f32(bits)
    assert np.all(np.isfinite(values))
    assert np.array_equal(orc.f32_to_f16_bits(values), bits)
    # and the decode agrees with IEEE half
    assert np.array_equal(values, bits.view(np.float16).astype(np.float32))


class Rng:
    """kv_f16.rs:249-264"""

    def __init__(self, seed):
        self.s = seed

    def next_u8(self):
        self.s = (self.s * 6364136223846793005 + 1442695040888963407) & ((1 << 64) - 1)
        return self.s >> 56


def test_f16_round_trip_stays_inside_the_half_ulp_bound():
    """kv_f16.rs:100-162: relative error <= 2^-11 for normal results, absolute <= 2^-25 below 2^-14."""
    xs = []
    for e in range(-20, 16):
        for m in (1.0, 1.0009766, 1.5, 1.9990234, 0.5, 0.75):
            x = np.float32(m) * np.float32(2.0) ** e
            xs += [x, -x]
    rng = Rng(0x0F160BAD)
    for _ in range(200_000):
        sign = 1.0 if rng.next_u8() & 1 == 0 else -1.0
        e = (rng.next_u8() % 36) - 20
        mant = np.float32(1.0) + (np.float32(rng.next_u8()) / np.float32(256.0) + np.float32(rng.next_u8()) / np.float32(65536.0))
        xs.append(np.float32(sign) * mant * np.float32(2.0) ** e)
    x = np.array(xs, dtype=np.float32)
    x = x[np.isfinite(x) & (np.abs(x) < 65504.0)]
    rt = orc.round_through_f16(x)
    err = np.abs(rt - x)
    normal = np.abs(x) >= np.float32(2.0) ** -14
    rel = err[normal] / np.abs(x[normal])
    assert rel.max() <= 0.00048828125
    assert rel.max() > 0.0
    assert err[~normal].max() <= 0.000000029802322
    assert x.size > 200_000
    # and the rounding itself is IEEE round-to-nearest-even
    assert np.array_equal(orc.f32_to_f16_bits(x), x.astype(np.float16).view(np.uint16))


def test_special_values():
    """k1_q4k_gemv.rs:285-329: inf keeps class, NaN -> sign|0x7e00, overflow -> inf, tiny -> signed zero."""
    nan_neg = np.array([0xFFC12345], dtype=np.uint32).view(np.float32)[0]
    x = np.array([np.inf, -np.inf, np.nan, nan_neg, 65520.0, -1e9, 1e-10, -1e-10, 65504.0, 2.0 ** -24, 2.0 ** -25,
                  np.float32(2.0 ** -25) * np.float32(1.0000001), 0.0, -0.0], dtype=np.float32)
    got = orc.f32_to_f16_bits(x).tolist()
    assert got == [0x7C00, 0xFC00, 0x7E00, 0xFE00, 0x7C00, 0xFC00, 0x0000, 0x8000, 0x7BFF, 0x0001, 0x0000, 0x0001,
                   0x0000, 0x8000]


def test_packed_word_layout_is_even_low_odd_high():
    """kv_f16.rs:164-173: element 2i in the low half of word i, 2i+1 in the high half."""
    def pack(lo, hi):
        b = orc.f32_to_f16_bits([lo, hi])
        return int(b[0]) | (int(b[1]) << 16)

    for lo, hi in [(1.5, -0.25), (0.0, 65504.0)]:
        w = pack(lo, hi)
        back = orc.f16_bits_to_f32(np.array([w & 0xFFFF, w >> 16], dtype=np.uint16))
        assert back.tolist() == [lo, hi]
    # the little-endian u16 pair in memory IS that word
    b = orc.f32_to_f16_bits([1.5, -0.25])
    assert int(b.view(np.uint32)[0]) == pack(1.5, -0.25)


def close(a, b, tol):
    return np.all(np.abs(np.asarray(a, dtype=np.float64) - np.asarray(b, dtype=np.float64)) <= tol)


def test_rope_interleaved_known_rotations():
    """rope_interleaved.rs:125-145: (cos 1, sin 1, cos 0.01, sin 0.01)."""
    out = orc.rope_interleaved([1.0, 0.0, 1.0, 0.0], 1, 10_000.0, 4)
    assert close(out, [0.5403023058681398, 0.8414709848078965, 0.9999500004166653, 0.009999833334166664], 1e-5)


def test_rope_interleaved_zero_position_and_norm():
    """rope_interleaved.rs:147-158"""
    x = [1.0, 2.0, 3.0, 4.0]
    assert orc.rope_interleaved(x, 0, 500_000.0, 4).tolist() == x
    out = orc.rope_interleaved(x, 7, 500_000.0, 4).astype(np.float64)
    assert abs((out ** 2).sum() - 30.0) <= 0.01


def test_rope_interleaved_partial():
    """rope_interleaved.rs:160-190: rotary_dim 4 of 8 rotates two adjacent pairs, passes the tail."""
    x = [1.0, 0.0, 1.0, 0.0, 9.0, -4.0, 7.0, 3.0]
    out = orc.rope_interleaved(x, 1, 10_000.0, 8, 4)
    assert close(out, [0.5403023058681398, 0.8414709848078965, 0.9999500004166653, 0.009999833334166664,
                       9.0, -4.0, 7.0, 3.0], 1e-5)
    neox = orc.rope(x, 1, 10_000.0, 8, 4)
    assert np.any(np.abs(out - neox) > 0.1)
    y = [0.3, -1.2, 2.5, 0.7, 1.1, -0.4, 0.9, 2.2]
    assert orc.rope_interleaved(y, 5, 500_000.0, 8, 8).tobytes() == orc.rope_interleaved(y, 5, 500_000.0, 8).tobytes()


def test_rope_half_split_known_rotations():
    """rope.rs:133-168: (cos1 - sin1, 0, sin1 + cos1, 0) and pair 1 at rate 0.01."""
    assert orc.rope([0.3, -1.2, 2.5, 0.7], 0, 500_000.0, 4).tolist() == [np.float32(v) for v in [0.3, -1.2, 2.5, 0.7]]
    assert close(orc.rope([1.0, 0.0, 1.0, 0.0], 1, 10_000.0, 4), [-0.30116868, 0.0, 1.3817733, 0.0], 1e-5)
    assert close(orc.rope([0.0, 1.0, 0.0, 0.0], 1, 10_000.0, 4), [0.0, 0.9999500004166653, 0.0, 0.009999833334166664], 1e-5)


def test_rope_half_split_partial_norm_and_base():
    """rope.rs:170-201"""
    out = orc.rope([1.0, 2.0, 3.0, 4.0], 7, 500_000.0, 4).astype(np.float64)
    assert abs((out ** 2).sum() - 30.0) <= 0.01
    out = orc.rope([1.0, 0.0, 9.0, -4.0], 3, 10_000.0, 4, 2)
    assert out[2] == 9.0 and out[3] == -4.0
    assert abs(out[0] - (-0.9899924966004454)) <= 1e-5 and abs(out[1] - 0.1411200080598672) <= 1e-5
    out = orc.rope([0.0, 1.0, 0.0, 0.0], 1, 500_000.0, 4)
    assert abs(out[3] - 0.0014142135) <= 1e-6 and abs(out[1] - 0.999999) <= 1e-6


def test_rope_bad_config_is_an_error():
    """rope.rs:203-, rope_interleaved.rs:192-: length mismatch, odd dims, base <= 1."""
    for fn in (orc.rope, orc.rope_interleaved):
        with pytest.raises(OracleError) as e:
            fn([1.0, 0.0], 0, 10_000.0, 4)
        assert e.value.code == orc.SHAPE_MISMATCH
        with pytest.raises(OracleError):
            fn([1.0, 0.0, 0.0], 0, 10_000.0, 3)
        with pytest.raises(OracleError):
            fn([1.0, 0.0], 0, 1.0, 2)
        with pytest.raises(OracleError):
            fn([1.0, 0.0, 1.0, 0.0], 0, 10_000.0, 4, 6)


def test_rope_rows_matches_per_head_calls():
    x = orc.lcg(5, 3 * 2 * 8).reshape(3, 2, 8)
    got = orc.rope_rows(x, 2, 8, 40, 500_000.0)
    for r in range(3):
        for h in range(2):
            assert got[r, h].tobytes() == orc.rope_interleaved(x[r, h], 40 + r, 500_000.0, 8).tobytes()
