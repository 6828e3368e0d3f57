"""The oracle's draft-model (DFlash) attention against the two checks the reference itself applies to that step
(crates/dflash/src/model.rs): the closed form of its analytic model (:727-822: Q = K = 0, so every query is the
uniform mean of the visible value rows) and the naive f64 formula of :1065-1110, causal and non-causal, global and
sliding."""
import numpy as np
import pytest

from oracle import oracle as orc


def naive_f64(q, positions, cpos, ck, cv, bk, bv, hq, hkv, kl, vl, causal, sliding, window):
    """model.rs:1065-1110, written from the formula."""
    rows = len(positions)
    out = np.zeros((rows, hq * vl))
    group = hq // hkv
    keys = [(int(p), ck[i], cv[i]) for i, p in enumerate(cpos)] + [(int(positions[m]), bk[m], bv[m]) for m in range(rows)]
    for r in range(rows):
        p = int(positions[r])
        vis = [(kp, k, v) for kp, k, v in keys if not (causal and kp > p) and not (sliding and kp <= p - window)]
        for h in range(hq):
            kvh = h // group
            qh = q[r, h * kl:(h + 1) * kl].astype(np.float64)
            s = np.array([qh @ k[kvh * kl:(kvh + 1) * kl].astype(np.float64) for _, k, _ in vis]) / np.sqrt(kl)
            e = np.exp(s - s.max())
            w = e / e.sum()
            for i, (_, _, v) in enumerate(vis):
                out[r, h * vl:(h + 1) * vl] += w[i] * v[kvh * vl:(kvh + 1) * vl].astype(np.float64)
    return out


def test_zero_queries_give_the_uniform_mean_of_the_visible_rows():
    """model.rs:755-760: two cached rows at positions 0 and 1, a block of three rows at 2..5, non-causal: every
    query sees all five value rows with equal weight."""
    hq, hkv, kl, vl = 2, 1, 4, 4
    rng = np.random.default_rng(1)
    cv = rng.standard_normal((2, hkv * vl)).astype(np.float32)
    bv = rng.standard_normal((3, hkv * vl)).astype(np.float32)
    ck, bk = np.zeros((2, hkv * kl), np.float32), np.zeros((3, hkv * kl), np.float32)
    q = np.zeros((3, hq * kl), np.float32)
    out = orc.draft_attention(q, [2, 3, 4], [0, 1], ck, cv, bk, bv, hq, hkv, kl, vl)
    mean = np.concatenate([cv, bv]).astype(np.float64).mean(axis=0)
    for r in range(3):
        for h in range(hq):
            assert np.allclose(out[r, h * vl:(h + 1) * vl], mean, atol=1e-6)
    # causal: row r sees the cached rows and block rows 0..r only
    out = orc.draft_attention(q, [2, 3, 4], [0, 1], ck, cv, bk, bv, hq, hkv, kl, vl, causal=True)
    for r in range(3):
        mean = np.concatenate([cv, bv[: r + 1]]).astype(np.float64).mean(axis=0)
        assert np.allclose(out[r, :vl], mean, atol=1e-6)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("sliding,window", [(False, 0), (True, 4), (True, 1)])
def test_matches_the_naive_f64_formula(causal, sliding, window):
    """model.rs:1147-1180 (block_forward_matches_naive_reference_noncausal_and_causal), for the attention step alone;
    a sparse committed set (the cache is a position map) and the signed window comparison kp <= p - window."""
    hq, hkv, kl, vl, rows = 4, 2, 16, 8, 4
    rng = np.random.default_rng(17 + int(causal) + window)
    cpos = [0, 1, 2, 5, 6, 9]  # sparse: positions 3, 4, 7, 8 were never injected
    positions = list(range(10, 10 + rows))
    q = rng.standard_normal((rows, hq * kl)).astype(np.float32)
    ck = rng.standard_normal((len(cpos), hkv * kl)).astype(np.float32)
    cv = rng.standard_normal((len(cpos), hkv * vl)).astype(np.float32)
    bk = rng.standard_normal((rows, hkv * kl)).astype(np.float32)
    bv = rng.standard_normal((rows, hkv * vl)).astype(np.float32)
    got = orc.draft_attention(q, positions, cpos, ck, cv, bk, bv, hq, hkv, kl, vl, causal, sliding, window)
    want = naive_f64(q, positions, cpos, ck, cv, bk, bv, hq, hkv, kl, vl, causal, sliding, window)
    assert np.max(np.abs(got - want)) < 1e-5


def test_window_one_sees_only_the_query_itself_when_causal():
    """kp > p - 1 and kp <= p leaves kp == p: the block's own row, which both masks always admit
    (model.rs:428-431)."""
    hq, hkv, kl, vl = 1, 1, 2, 3
    bv = np.arange(9, dtype=np.float32).reshape(3, 3)
    out = orc.draft_attention(np.ones((3, 2), np.float32), [5, 6, 7], [0, 4], np.ones((2, 2), np.float32),
                              np.full((2, 3), 100.0, np.float32), np.ones((3, 2), np.float32), bv, hq, hkv, kl, vl,
                              causal=True, sliding=True, window=1)
    assert np.allclose(out, bv)


def test_refusals():
    with pytest.raises(orc.OracleError) as e:
        orc.draft_attention(np.zeros((1, 3)), [0], [], [], [], np.zeros((1, 2)), np.zeros((1, 2)), 3, 2, 1, 1)
    assert e.value.code == orc.NON_DIVISIBLE_HEADS
