"""The oracle's RMSNorm against the reference's own tests (crates/torch-math/src/norm.rs:56-121), and the
preparation the reference composes from it (crates/wgpu-compute/src/kernels/k9_attn_prep.rs:1-40)."""
import math

import numpy as np
import pytest

from oracle import oracle as orc
from oracle.oracle import OracleError


def test_constant_vector_normalizes_to_weight():
    """norm.rs:60-65: mean(x^2) = 4, so each element maps to 2 / sqrt(4 + eps), 1 up to the eps correction."""
    out = orc.rms_norm([2.0, 2.0, 2.0, 2.0], [1.0, 1.0, 1.0, 1.0], 1e-6)
    assert np.allclose(out, 1.0, atol=1e-5)


def test_known_vector():
    """norm.rs:67-73: mean of squares of [1,2,3,4] is 7.5."""
    out = orc.rms_norm([1.0, 2.0, 3.0, 4.0], [1.0, 1.0, 1.0, 1.0], 1e-5)
    assert np.allclose(out, [0.36515, 0.73030, 1.09545, 1.46061], atol=1e-4)


def test_weight_scales_output():
    """norm.rs:75-79"""
    out = orc.rms_norm([2.0, 2.0, 2.0, 2.0], [2.0, 2.0, 2.0, 2.0], 1e-6)
    assert np.allclose(out, 2.0, atol=1e-5)


def test_eps_is_a_parameter_not_a_constant():
    """norm.rs:81-88: with eps = 4 the divisor is sqrt(8)."""
    out = orc.rms_norm([2.0, 2.0, 2.0, 2.0], [1.0, 1.0, 1.0, 1.0], 4.0)
    assert abs(float(out[0]) - 1.0 / math.sqrt(2.0)) < 1e-6


def test_refusals():
    """norm.rs:90-120: empty input, weight length, eps not finite and > 0."""
    with pytest.raises(OracleError) as e:
        orc.rms_norm([], [], 1e-6)
    assert "empty" in str(e.value)
    with pytest.raises(OracleError) as e:
        orc.rms_norm([1.0, 2.0], [1.0], 1e-6)
    assert e.value.code == orc.SHAPE_MISMATCH and "got 1, expected 2" in str(e.value)
    for eps in (0.0, -1e-6, float("nan"), float("inf")):
        with pytest.raises(OracleError) as e:
            orc.rms_norm([1.0], [1.0], eps)
        assert "eps must be finite and > 0" in str(e.value)


def test_f64_accumulation_matches_numpy_float64():
    """The restatement is the f64 expression of norm.rs:43-52, rounded once."""
    rng = np.random.default_rng(3)
    x = rng.standard_normal(6656).astype(np.float32)  # Glimmer's hidden width, the case the f64 sum is there for
    w = rng.standard_normal(6656).astype(np.float32)
    inv = 1.0 / np.sqrt(np.sum(x.astype(np.float64) ** 2) / x.size + np.float64(np.float32(1e-6)))
    want = (x.astype(np.float64) * inv * w.astype(np.float64)).astype(np.float32)
    got = orc.rms_norm(x, w, 1e-6)
    # numpy's pairwise f64 sum and the sequential one differ by ~1e-16 relative: at most the last f32 bit
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-30)) < 2e-7


def test_prepare_rows_is_norm_then_rotation_per_head():
    rng = np.random.default_rng(5)
    heads, d = 3, 8
    x = rng.standard_normal((2, heads, d)).astype(np.float32)
    w = rng.standard_normal(d).astype(np.float32)
    got = orc.prepare_rows(x, heads, d, 7, weight=w, eps=1e-5, rope_base=10000.0)
    for r in range(2):
        for h in range(heads):
            want = orc.rope_interleaved(orc.rms_norm(x[r, h], w, 1e-5), 7 + r, 10000.0, d)
            assert np.array_equal(got[r, h], want)
    # no weight, no base: untouched
    assert np.array_equal(orc.prepare_rows(x, heads, d, 0), x)
