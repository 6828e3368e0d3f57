"""The tcgen05 (tensor-memory) multi-row attention kernel against the oracle's multi-query gqa_attention
(crates/attention/src/attention.rs:160-213) and against the mma.sync kernel it replaces: every pair-block
width (replicated 4x, 2x, not at all, several blocks), key splits, partial tiles, ring wrap and windows."""

import numpy as np
import pytest

from itak_torch_rebuild_b200 import CudaCompute, KvDtype, PositionCache
from oracle import oracle as orc

from kvparity import assert_view_equal, attention_error, make_pair, stored

pytestmark = pytest.mark.gpu

D = 128
DTYPE = KvDtype.F16
# The hi/lo f16 operand split carries ~22 bits of the f32 queries and weights: f32-grade results.
TIGHT = 2e-5


def build(layer_window, hq, hkv, n0, rows, *, env=None, n_slots=1, seed=0):
    """Backend + oracle caches holding n0 seeded rows per layer; windowed layers are fed chunk by chunk."""
    gpu, refs = make_pair(list(layer_window), hq, hkv, D, dtype=DTYPE, n_slots=n_slots, max_context=n0 + 4 * rows + 8,
                          chunk_cap=rows, options=env)
    rng = np.random.default_rng(seed)
    for slot in range(n_slots):
        for layer, w in enumerate(layer_window):
            k = rng.standard_normal((n0, hkv * D)).astype(np.float32)
            v = rng.standard_normal((n0, hkv * D)).astype(np.float32)
            step = n0 if w == 0 else rows
            at = 0
            while at < n0:
                m = min(step, n0 - at)
                gpu.append_rows(layer, k[at:at + m], v[at:at + m], at, slot=slot)
                at += m
            refs[slot].append_rows(layer, stored(k, DTYPE), stored(v, DTYPE), 0)
    return gpu, refs


def run_blocks(gpu, refs, layer_window, hq, hkv, n0, rows, blocks, seed):
    """`blocks` multi-row calls per layer on slot 0; returns the worst error against the oracle."""
    rng = np.random.default_rng(seed)
    pos = PositionCache()
    pos.advance(n0)
    worst = 0.0
    outs = []
    for _ in range(blocks):
        start = pos.position()
        for layer in range(len(layer_window)):
            q = rng.standard_normal((rows, hq * D)).astype(np.float32)
            k = rng.standard_normal((rows, hkv * D)).astype(np.float32)
            v = rng.standard_normal((rows, hkv * D)).astype(np.float32)
            got = gpu.attention(layer, q, k, v, pos).reshape(rows, -1)
            assert np.all(np.isfinite(got))
            outs.append(got)
            for r in range(rows):  # the reference's order: append a row, attend it
                refs[0].append(layer, stored(k[r], DTYPE), stored(v[r], DTYPE), start + r)
                want = orc.gqa_attention(q[r], 1, hq, [start + r], refs[0].view(layer))
                worst = max(worst, attention_error(got[r], want, hq, D))
        pos.advance(rows)
    gpu.synchronize()  # raises if a bounded wait in the kernel ran out
    return worst, outs


@pytest.mark.parametrize("rows,hq,hkv", [
    (7, 32, 8),    # 28 pairs: four replicas of a 32-pair block (the speculative configuration)
    (2, 8, 8),     # group 1: 2 pairs
    (8, 32, 8),    # exactly 32 pairs
    (12, 32, 8),   # 48 pairs: two replicas of a 64-pair block
    (7, 64, 8),    # group 8: 56 pairs
    (31, 32, 8),   # 124 pairs: one block, no replication
    (33, 32, 8),   # 132 pairs: two blocks
    (64, 64, 8),   # 512 pairs: eight blocks
    (65, 32, 8),   # past the old 64-row limit: five blocks, the last one nearly empty
    (200, 32, 8),  # a prefill chunk: thirteen blocks, each streaming the keys up to its own last row
    (5, 24, 2),    # group 12: two head chunks (8 + 4 heads)
])
@pytest.mark.parametrize("n0", [0, 57, 500])
def test_every_block_width_matches_the_oracle(rows, hq, hkv, n0):
    gpu, refs = build([0], hq, hkv, n0, rows, seed=rows + n0)
    worst, _ = run_blocks(gpu, refs, [0], hq, hkv, n0, rows, blocks=2, seed=3)
    assert worst < TIGHT, worst
    assert_view_equal(gpu, refs[0], 0, DTYPE)


def test_a_whole_prefill_chunk_runs_on_the_tensor_memory_kernel():
    """512 rows in one call (4096 row-head pairs, sixty-four blocks per KV head) behind a short prefix: every block
    streams the keys up to its own last row only, the last block's CTAs store the chunk's rows."""
    rows, hq, hkv, n0 = 512, 64, 8, 100
    gpu, refs = build([0], hq, hkv, n0, rows, seed=77)
    worst, _ = run_blocks(gpu, refs, [0], hq, hkv, n0, rows, blocks=1, seed=78)
    assert worst < TIGHT, worst
    assert_view_equal(gpu, refs[0], 0, DTYPE)


@pytest.mark.parametrize("n0", [1, 63, 64, 65, 127, 128, 192, 1000, 2048, 4500])
def test_every_tail_length(n0):
    gpu, refs = build([0], 32, 8, n0, 7, seed=n0)
    worst, _ = run_blocks(gpu, refs, [0], 32, 8, n0, 7, blocks=1, seed=5)
    assert worst < TIGHT, worst


@pytest.mark.parametrize("splits", [1, 2, 3, 7, 40])
def test_every_key_split(splits):
    """Forced split counts, including more splits than tiles (empty CTAs take part in the merge)."""
    n0 = 1500
    gpu, refs = build([0], 32, 8, n0, 7, env={"decode_splits": splits}, seed=1)
    worst, _ = run_blocks(gpu, refs, [0], 32, 8, n0, 7, blocks=2, seed=6)
    assert worst < TIGHT, worst
    assert gpu.stats()["last_splits"] == min(splits, (n0 + 14 + 63) // 64)


def test_windows_and_ring_wrap():
    """Sliding layers: per-row window masks, a ring that has wrapped many times, windows shorter and longer
    than a tile."""
    layer_window = [0, 40, 128, 300]
    n0, rows = 1000, 7
    gpu, refs = build(layer_window, 32, 8, n0, rows, seed=11)
    worst, _ = run_blocks(gpu, refs, layer_window, 32, 8, n0, rows, blocks=3, seed=12)
    assert worst < TIGHT, worst
    for layer in range(len(layer_window)):
        assert_view_equal(gpu, refs[0], layer, DTYPE)


def test_large_scores_keep_the_stale_maximum_exact():
    """Scores spread over hundreds of log2 units and rising along the keys, so that maxima grow both by less
    and by more than the rescale step: the lazily rescaled accumulator must still match."""
    hq, hkv, rows, n0 = 32, 8, 7, 700
    gpu, refs = make_pair([0], hq, hkv, D, dtype=DTYPE, max_context=n0 + 32, chunk_cap=rows)
    rng = np.random.default_rng(31)
    ramp = np.linspace(0.05, 3.0, n0, dtype=np.float32)[:, None]
    k = rng.standard_normal((n0, hkv * D)).astype(np.float32) * ramp
    v = rng.standard_normal((n0, hkv * D)).astype(np.float32)
    gpu.append_rows(0, k, v, 0)
    refs[0].append_rows(0, stored(k, DTYPE), stored(v, DTYPE), 0)
    pos = PositionCache()
    pos.advance(n0)
    q = 4.0 * rng.standard_normal((rows, hq * D)).astype(np.float32)
    kn = 3.0 * rng.standard_normal((rows, hkv * D)).astype(np.float32)
    vn = rng.standard_normal((rows, hkv * D)).astype(np.float32)
    got = gpu.attention(0, q, kn, vn, pos).reshape(rows, -1)
    refs[0].append_rows(0, stored(kn, DTYPE), stored(vn, DTYPE), n0)
    want = orc.gqa_attention(q, rows, hq, list(range(n0, n0 + rows)), refs[0].view(0))
    assert attention_error(got, want, hq, D) < TIGHT


def test_agrees_with_the_mma_sync_kernel_on_batched_sessions():
    """A/B on 5 sessions of different lengths in one launch: tcgen05 kernel vs the mma.sync kernel."""
    hq, hkv, rows = 32, 8, 7
    lens = [300, 64, 2047, 5, 1111]
    rng = np.random.default_rng(17)
    data = [(rng.standard_normal((n, hkv * D)).astype(np.float32), rng.standard_normal((n, hkv * D)).astype(np.float32))
            for n in lens]
    q = rng.standard_normal((len(lens), rows, hq * D)).astype(np.float32)
    k = rng.standard_normal((len(lens), rows, hkv * D)).astype(np.float32)
    v = rng.standard_normal((len(lens), rows, hkv * D)).astype(np.float32)
    outs = []
    for flag in (1, 0):
        gpu = CudaCompute(1, hq, hkv, D, n_slots=len(lens), max_context=2100, chunk_cap=rows, kv_dtype=DTYPE,
                          options={"verify_tc": flag})
        for slot, (k0, v0) in enumerate(data):
            gpu.append_rows(0, k0, v0, 0, slot=slot)
        outs.append(gpu.attention_batch(0, list(range(len(lens))), lens, rows, q, k, v))
        gpu.synchronize()
    assert attention_error(outs[0], outs[1], hq, D) < 1e-5


def test_a_wait_that_runs_out_is_reported_and_the_next_call_succeeds():
    """Every wait inside the kernel is bounded.  With the first key tile of every CTA loaded but never reported (a test
    switch) and the bound set to about a millisecond, the wait for that tile runs out: every role leaves its loop, the
    kernel returns, the call that synchronises is refused by name - and the backend goes on working: the same slot,
    reset and refilled, matches the oracle again.  Nothing faults and nothing hangs."""
    from itak_torch_rebuild_b200 import CudaComputeError, _lib

    hq, hkv, n0, rows = 32, 8, 300, 7
    gpu, refs = build([0], hq, hkv, n0, rows, env={"tc_wait_kclocks": 2000, "tc_withhold_first_tile": 1}, seed=41)
    rng = np.random.default_rng(42)
    pos = PositionCache()
    pos.advance(n0)
    q = rng.standard_normal((rows, hq * D)).astype(np.float32)
    k = rng.standard_normal((rows, hkv * D)).astype(np.float32)
    v = rng.standard_normal((rows, hkv * D)).astype(np.float32)
    with pytest.raises(CudaComputeError) as e:
        gpu.attention(0, q, k, v, pos)
    assert e.value.code == _lib.ERR_CUDA and "bounded wait" in e.value.msg
    gpu.set_option("tc_withhold_first_tile", 0)
    gpu.set_option("tc_wait_kclocks", 0)
    # what the refused launch left in the slot is not defined: the sequence starts again
    gpu.reset(0)
    rng = np.random.default_rng(43)
    k0 = rng.standard_normal((n0, hkv * D)).astype(np.float32)
    v0 = rng.standard_normal((n0, hkv * D)).astype(np.float32)
    gpu.append_rows(0, k0, v0, 0)
    ref = orc.KvCache([orc.GLOBAL], hkv, D)
    ref.append_rows(0, stored(k0, DTYPE), stored(v0, DTYPE), 0)
    worst, _ = run_blocks(gpu, [ref], [0], hq, hkv, n0, rows, blocks=2, seed=44)
    assert worst <= TIGHT
    assert_view_equal(gpu, ref, 0, DTYPE)
    gpu.close()
