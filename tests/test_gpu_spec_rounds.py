"""The speculative (DFlash-style) path end to end on the device: shared prefix restored into sessions, rounds
of append 7 rows + tensor-core causal verify attention + truncate to the accepted length
(crates/itak-spec/src/session.rs:663-747: checkpoint -> block forward -> rewind(base + 1 + accepted) -> release)."""

import numpy as np
import pytest

from itak_torch_rebuild_b200 import CudaCompute, KvDtype
from oracle import oracle as orc

from kvparity import assert_attention_close, assert_view_equal, stored

pytestmark = pytest.mark.gpu

DEPTH = 6  # draft depth; a round appends DEPTH + 1 rows


def accepted_lengths(rng, n):
    """Accepted draft tokens per round: geometric with acceptance probability 0.7 per token, capped at DEPTH."""
    a = rng.geometric(0.3, size=n) - 1  # failures before the first rejection
    return np.minimum(a, DEPTH)


@pytest.mark.parametrize("hq,hkv,d", [(32, 8, 128), (8, 2, 64), (16, 1, 128)])
def test_verify_rounds_match_the_oracle(hq, hkv, d):
    """Reduced size (2 layers, 3 sessions, prefix 300, 6 rounds): every verify output equals the oracle's
    multi-query gqa_attention, and after every truncation the device views equal the oracle's rewound cache."""
    layers, sessions, prefix, rounds, dtype = 2, 3, 300, 6, KvDtype.F16
    rows = DEPTH + 1
    gpu = CudaCompute(layers, hq, hkv, d, n_slots=sessions + 1, max_context=prefix + rounds * rows + 8,
                      chunk_cap=rows, kv_dtype=dtype)
    rng = np.random.default_rng(hq + d)
    refs = [orc.KvCache([orc.GLOBAL] * layers, hkv, d) for _ in range(sessions)]
    for layer in range(layers):
        k = rng.standard_normal((prefix, hkv * d)).astype(np.float32)
        v = rng.standard_normal((prefix, hkv * d)).astype(np.float32)
        gpu.append_rows(layer, k, v, 0, slot=sessions)
        for ref in refs:
            ref.append_rows(layer, stored(k, dtype), stored(v, dtype), 0)
    snap = gpu.capture_prefix_snapshot(slot=sessions)
    for s in range(sessions):
        assert gpu.install_prefix_snapshot(snap, slot=s) == prefix
    pos = [prefix] * sessions
    worst = 0.0
    for rnd in range(rounds):
        acc = accepted_lengths(rng, sessions)
        cps = [gpu.cache_checkpoint(rows, slot=s) for s in range(sessions)]
        rcps = [ref.checkpoint(rows) for ref in refs]
        for layer in range(layers):
            q = rng.standard_normal((sessions, rows, hq * d)).astype(np.float32)
            k = rng.standard_normal((sessions, rows, hkv * d)).astype(np.float32)
            v = rng.standard_normal((sessions, rows, hkv * d)).astype(np.float32)
            got = gpu.attention_batch(layer, list(range(sessions)), pos, rows, q, k, v).reshape(sessions, rows, -1)
            for s, ref in enumerate(refs):
                ref.append_rows(layer, stored(k[s], dtype), stored(v[s], dtype), pos[s])
                want = orc.gqa_attention(q[s], rows, hq, list(range(pos[s], pos[s] + rows)), ref.view(layer))
                worst = max(worst, assert_attention_close(got[s], want, hq, d, dtype, f"round {rnd} layer {layer} session {s}"))
        for s in range(sessions):
            keep = pos[s] + 1 + int(acc[s])
            gpu.cache_rewind(cps[s], keep, slot=s)
            gpu.cache_release(cps[s], slot=s)
            refs[s].rewind_to(rcps[s], keep)
            refs[s].release(rcps[s])
            pos[s] = keep
            for layer in range(layers):
                assert gpu.next_position(layer, slot=s) == keep
        s = rnd % sessions
        assert_view_equal(gpu, refs[s], rnd % layers, dtype, slot=s)
    assert worst < 2e-3


def test_verify_kernel_agrees_with_the_cuda_core_kernel():
    """A/B: the tensor-core verify kernel against the general kernel on the same rows (windowed and global)."""
    hq, hkv, d, rows = 32, 8, 128, 7
    rng = np.random.default_rng(77)
    k0 = rng.standard_normal((500, hkv * d)).astype(np.float32)
    v0 = rng.standard_normal((500, hkv * d)).astype(np.float32)
    q = rng.standard_normal((rows, hq * d)).astype(np.float32)
    k = rng.standard_normal((rows, hkv * d)).astype(np.float32)
    v = rng.standard_normal((rows, hkv * d)).astype(np.float32)
    outs = []
    for force in (0, 1):
        gpu = CudaCompute(2, hq, hkv, d, n_slots=1, max_context=600, chunk_cap=rows, kv_dtype=KvDtype.F16,
                          layer_window=[0, 128], options={"force_general": force})
        from itak_torch_rebuild_b200 import PositionCache

        pos = PositionCache()
        res = []
        for layer in range(2):
            at = 0
            while at < 500:
                gpu.append_rows(layer, k0[at:at + rows], v0[at:at + rows], at)
                at += rows
            pos._p = gpu.next_position(layer)
            res.append(gpu.attention(layer, q, k, v, pos))
        outs.append(np.concatenate(res))
    err = np.abs(outs[0] - outs[1]).max()
    assert err < 1e-5, err


def test_speculative_sessions_at_full_size_equal_never_speculated_sessions():
    """The prefix-KV + speculative configuration at full size: 32 layers, 32 query / 8 KV heads, head dim 128,
    f16, a 2048-token shared prefix restored into 16 sessions, 64 rounds of 7 appended rows, verify, truncate.
    Size-independent property: a session that speculated and truncated holds, bit for bit, the rows of a
    session that only ever appended the kept tokens, and a decode step over both gives identical bits."""
    layers, hq, hkv, d, prefix, sessions, rounds = 32, 32, 8, 128, 2048, 16, 64
    rows = DEPTH + 1
    cap = prefix + rounds * rows + 8
    spec = CudaCompute(layers, hq, hkv, d, n_slots=sessions + 1, max_context=cap, chunk_cap=rows, kv_dtype=KvDtype.F16)
    plain = CudaCompute(layers, hq, hkv, d, n_slots=sessions + 1, max_context=cap, chunk_cap=rows, kv_dtype=KvDtype.F16)
    rng = np.random.default_rng(2024)
    for layer in range(layers):
        k = rng.standard_normal((prefix, hkv * d)).astype(np.float32)
        v = rng.standard_normal((prefix, hkv * d)).astype(np.float32)
        at = 0
        while at < prefix:  # the staging buffer holds (sessions + 1) * rows rows
            n = min(112, prefix - at)
            spec.append_rows(layer, k[at:at + n], v[at:at + n], at, slot=sessions)
            plain.append_rows(layer, k[at:at + n], v[at:at + n], at, slot=sessions)
            at += n
    snap_s, snap_p = spec.capture_prefix_snapshot(slot=sessions), plain.capture_prefix_snapshot(slot=sessions)
    for s in range(sessions):
        spec.install_prefix_snapshot(snap_s, slot=s)
        plain.install_prefix_snapshot(snap_p, slot=s)
    pos = [prefix] * sessions
    slots = list(range(sessions))
    for rnd in range(rounds):
        acc = accepted_lengths(rng, sessions)
        cps = [spec.cache_checkpoint(rows, slot=s) for s in slots]
        # one seeded block per round, shared by the layers (only the copy/truncate law is under test here)
        q = rng.standard_normal((sessions, rows, hq * d)).astype(np.float32)
        k = rng.standard_normal((sessions, rows, hkv * d)).astype(np.float32)
        v = rng.standard_normal((sessions, rows, hkv * d)).astype(np.float32)
        for layer in range(layers):
            out = spec.attention_batch(layer, slots, pos, rows, q, k, v)
            if layer == 0 and rnd % 16 == 0:
                assert np.all(np.isfinite(out))
        for s in slots:
            kept = 1 + int(acc[s])
            spec.cache_rewind(cps[s], pos[s] + kept, slot=s)
            spec.cache_release(cps[s], slot=s)
            for layer in range(layers):
                plain.append_rows(layer, k[s, :kept], v[s, :kept], pos[s], slot=s)
            pos[s] += kept
    assert len(set(pos)) > 1, "sessions should have diverged in length"
    for s in (0, 7, 15):
        for layer in (0, 13, 31):
            a, b = spec.view(layer, slot=s), plain.view(layer, slot=s)
            assert a[0] == b[0] == 0 and a[1].shape[0] == pos[s]
            assert a[1].tobytes() == b[1].tobytes() and a[2].tobytes() == b[2].tobytes()
    q = rng.standard_normal((sessions, hq * d)).astype(np.float32)
    k = rng.standard_normal((sessions, hkv * d)).astype(np.float32)
    v = rng.standard_normal((sessions, hkv * d)).astype(np.float32)
    a = spec.attention_batch(5, slots, pos, 1, q, k, v)
    b = plain.attention_batch(5, slots, pos, 1, q, k, v)
    assert a.tobytes() == b.tobytes()
