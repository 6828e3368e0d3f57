"""The tensor-core attention kernel of an f32 cache (three-term tf32 products) against the oracle's gqa_attention
(crates/attention/src/attention.rs:104-215) and against the CUDA-core kernel it stands in front of: decode rows
and multi-row blocks at both head dims, every pair-block width, forced key splits, partial tiles, ring wrap,
windows and ragged batches."""

import numpy as np
import pytest

from itak_torch_rebuild_b200 import KvDtype, PositionCache
from oracle import oracle as orc

from kvparity import TOL_F32_KV, assert_view_equal, attention_error, make_pair

pytestmark = pytest.mark.gpu

DTYPE = KvDtype.F32
# Three tf32 terms carry ~21 bits of every product: far inside the f32-cache tolerance.
TIGHT = 1e-5


def build(layer_window, hq, hkv, d, n0, rows, *, options=None, n_slots=1, seed=0, blocks=4):
    """Backend + oracle caches holding n0 seeded rows per layer; windowed layers are fed chunk by chunk."""
    gpu, refs = make_pair(list(layer_window), hq, hkv, d, dtype=DTYPE, n_slots=n_slots,
                          max_context=n0 + blocks * rows + 8, chunk_cap=rows, options=options)
    rng = np.random.default_rng(seed)
    for slot in range(n_slots):
        for layer, w in enumerate(layer_window):
            k = rng.standard_normal((n0, hkv * d)).astype(np.float32)
            v = rng.standard_normal((n0, hkv * d)).astype(np.float32)
            step = n0 if w == 0 else rows
            at = 0
            while at < n0:
                m = min(step, n0 - at)
                gpu.append_rows(layer, k[at:at + m], v[at:at + m], at, slot=slot)
                at += m
            refs[slot].append_rows(layer, k, v, 0)
    return gpu, refs


def run_blocks(gpu, refs, layer_window, hq, hkv, d, n0, rows, blocks, seed):
    """`blocks` calls of `rows` rows per layer on slot 0; returns the worst error against the oracle and the outputs."""
    rng = np.random.default_rng(seed)
    pos = PositionCache()
    pos.advance(n0)
    worst = 0.0
    outs = []
    for _ in range(blocks):
        start = pos.position()
        for layer in range(len(layer_window)):
            q = rng.standard_normal((rows, hq * d)).astype(np.float32)
            k = rng.standard_normal((rows, hkv * d)).astype(np.float32)
            v = rng.standard_normal((rows, hkv * d)).astype(np.float32)
            got = gpu.attention(layer, q, k, v, pos).reshape(rows, -1)
            assert np.all(np.isfinite(got))
            outs.append(got)
            for r in range(rows):  # the reference's order: append a row, attend it
                refs[0].append(layer, k[r], v[r], start + r)
                want = orc.gqa_attention(q[r], 1, hq, [start + r], refs[0].view(layer))
                worst = max(worst, attention_error(got[r], want, hq, d))
        pos.advance(rows)
    gpu.synchronize()
    return worst, outs


@pytest.mark.parametrize("rows,hq,hkv", [
    (1, 32, 4),    # decode, group 8: 8 pairs, the four warps share the keys (the TinyLlama shape)
    (1, 4, 4),     # decode, group 1: one pair
    (2, 32, 4),    # 16 pairs: still the shared-key shape
    (3, 32, 4),    # 24 pairs: one 64-pair block
    (7, 16, 4),    # 28 pairs
    (8, 32, 4),    # exactly 64 pairs
    (9, 32, 4),    # 72 pairs: two blocks, the second nearly empty
    (65, 8, 8),    # group 1, 65 pairs
    (40, 24, 2),   # group 12: two head chunks (8 + 4 heads) with different block counts
])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("n0", [0, 57, 500])
def test_every_block_width_matches_the_oracle(rows, hq, hkv, d, n0):
    gpu, refs = build([0], hq, hkv, d, n0, rows, seed=rows + n0 + d)
    worst, _ = run_blocks(gpu, refs, [0], hq, hkv, d, n0, rows, blocks=3, seed=3)
    assert worst <= TIGHT, f"error {worst:.3e} of the output norm"
    assert_view_equal(gpu, refs[0], 0, DTYPE)
    gpu.close()


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("n", [1, 2, 15, 16, 17, 63, 64, 65, 127, 128, 129, 300, 1000, 4097])
def test_decode_at_every_tail_length(n, d):
    """One decode row at every tile-boundary case of the context length."""
    gpu, refs = build([0], 8, 2, d, n, 1, seed=n * 7 + d)
    worst, _ = run_blocks(gpu, refs, [0], 8, 2, d, n, 1, blocks=2, seed=n)
    assert worst <= TIGHT
    gpu.close()


@pytest.mark.parametrize("rows", [1, 7, 100])
@pytest.mark.parametrize("splits", [1, 2, 3, 5, 16])
def test_forced_key_splits_merge_to_the_same_answer(rows, splits):
    """Any number of CTAs per cell gives the same answer to rounding: the last arrival's log-sum-exp merge, parts
    left empty by the causal bound included."""
    outs = []
    for s in (1, splits):
        gpu, refs = build([0], 32, 4, 64, 700, rows, options={"decode_splits": s}, seed=9)
        worst, got = run_blocks(gpu, refs, [0], 32, 4, 64, 700, rows, blocks=2, seed=4)
        assert worst <= TIGHT
        assert gpu.stats()["last_splits"] == min(s, -(-(700 + 2 * rows) // 32))  # never more parts than 32-key tiles
        outs.append(np.concatenate(got))
        gpu.close()
    assert np.abs(outs[0] - outs[1]).max() <= 1e-5 * np.abs(outs[0]).max()


def test_tensor_kernel_agrees_with_the_cuda_core_kernel():
    """The same calls through the tensor-core kernel and, with force_general = 1, through the CUDA-core kernel that
    follows the reference's summation order."""
    res = []
    for opts in (None, {"force_general": 1}):
        gpu, refs = build([0, 24], 32, 4, 64, 300, 5, options=opts, seed=2)
        _, got = run_blocks(gpu, refs, [0, 24], 32, 4, 64, 300, 5, blocks=3, seed=6)
        res.append(np.concatenate(got))
        gpu.close()
    assert np.abs(res[0] - res[1]).max() <= 2e-5 * np.abs(res[1]).max()


@pytest.mark.parametrize("rows", [1, 7, 100])
def test_the_launch_that_stores_the_rows_equals_the_separate_append(rows):
    """By default the attention launch copies the call's new rows into the cache itself; with separate_append = 1
    the append kernel does, in a launch of its own.  Same cache bytes (checked against the oracle in both), same
    outputs to the last bit (the kernel reads the same values either way), one launch fewer per call."""
    res = []
    for opts in (None, {"separate_append": 1}):
        gpu, refs = build([0, 40], 32, 4, 64, 150, rows, options=opts, seed=3)
        before = gpu.stats()["kernel_launches"]
        worst, got = run_blocks(gpu, refs, [0, 40], 32, 4, 64, 150, rows, blocks=3, seed=5)
        assert worst <= TIGHT
        for layer in range(2):
            assert_view_equal(gpu, refs[0], layer, DTYPE)
        res.append((np.concatenate(got), gpu.stats()["kernel_launches"] - before))
        gpu.close()
    assert np.array_equal(res[0][0], res[1][0])
    assert res[1][1] == res[0][1] + 6


@pytest.mark.parametrize("rows", [1, 6, 40])
def test_sliding_layers_mask_and_wrap(rows):
    """Window 48 on a ring that wraps several times next to a global layer: every row of a block has its own
    window (crates/attention/src/attention.rs:77-85), and a block's key range starts at its first row's."""
    lw = [48, 0, 100]
    gpu, refs = build(lw, 16, 4, 64, 130, rows, seed=rows, blocks=6)
    worst, _ = run_blocks(gpu, refs, lw, 16, 4, 64, 130, rows, blocks=6, seed=8)
    assert worst <= TIGHT
    for layer in range(3):
        assert_view_equal(gpu, refs[0], layer, DTYPE)
    gpu.close()


def test_tinyllama_prefill_then_decode():
    """The reference's own configuration at shape: 32 q / 4 KV heads, head dim 64, a 512-row prefill in one call,
    then decode steps (rows checked on a sample: the oracle's prefill takes seconds)."""
    hq, hkv, d, prefill = 32, 4, 64, 512
    gpu, (ref,) = make_pair([0], hq, hkv, d, dtype=DTYPE, max_context=prefill + 16, chunk_cap=prefill)
    rng = np.random.default_rng(1)
    q = rng.standard_normal((prefill, hq * d)).astype(np.float32)
    k = rng.standard_normal((prefill, hkv * d)).astype(np.float32)
    v = rng.standard_normal((prefill, hkv * d)).astype(np.float32)
    pos = PositionCache()
    got = gpu.attention(0, q, k, v, pos).reshape(prefill, -1)
    pos.advance(prefill)
    ref.append_rows(0, k, v, 0)
    for r in (0, 1, 7, 8, 63, 64, 65, 255, 256, 500, 511):
        want = orc.gqa_attention(q[r], 1, hq, [r], _prefix(hkv, d, k, v, r))
        assert attention_error(got[r], want, hq, d) <= TIGHT, f"row {r}"
    for step in range(4):
        qs = rng.standard_normal(hq * d).astype(np.float32)
        ks = rng.standard_normal(hkv * d).astype(np.float32)
        vs = rng.standard_normal(hkv * d).astype(np.float32)
        out = gpu.attention(0, qs, ks, vs, pos)
        ref.append(0, ks, vs, pos.position())
        want = orc.gqa_attention(qs, 1, hq, [pos.position()], ref.view(0))
        assert attention_error(out, want, hq, d) <= TIGHT
        pos.advance(1)
    assert_view_equal(gpu, ref, 0, DTYPE)
    gpu.close()


def _prefix(hkv, d, k, v, r):
    """The view a cache holding rows 0..r gives (row r's causal view inside a block)."""
    c = orc.KvCache([orc.GLOBAL], hkv, d)
    c.append_rows(0, k[:r + 1], v[:r + 1], 0)
    return c.view(0)


def test_ragged_batch_of_slots():
    """Sequences of different lengths in one launch, one decode row each, then a 5-row block each."""
    hq, hkv, d = 32, 4, 64
    lens = [3, 700, 64, 129, 1]
    n = len(lens)
    gpu, refs = make_pair([0], hq, hkv, d, dtype=DTYPE, n_slots=n, max_context=800, chunk_cap=5)
    rng = np.random.default_rng(12)
    for slot, ln in enumerate(lens):
        k = rng.standard_normal((ln, hkv * d)).astype(np.float32)
        v = rng.standard_normal((ln, hkv * d)).astype(np.float32)
        gpu.append_rows(0, k, v, 0, slot=slot)
        refs[slot].append_rows(0, k, v, 0)
    at = list(lens)
    for rows in (1, 5, 1):
        q = rng.standard_normal((n, rows, hq * d)).astype(np.float32)
        k = rng.standard_normal((n, rows, hkv * d)).astype(np.float32)
        v = rng.standard_normal((n, rows, hkv * d)).astype(np.float32)
        got = gpu.attention_batch(0, list(range(n)), at, rows, q, k, v).reshape(n, rows, -1)
        for i in range(n):
            for r in range(rows):
                refs[i].append(0, k[i, r], v[i, r], at[i] + r)
                want = orc.gqa_attention(q[i, r], 1, hq, [at[i] + r], refs[i].view(0))
                assert attention_error(got[i, r], want, hq, d) <= TIGHT, f"slot {i} row {r}"
            at[i] += rows
    assert TIGHT < TOL_F32_KV
    gpu.close()


def test_unaligned_device_buffers_are_refused_by_name():
    """Device buffers must start on 16-byte boundaries (the kernels move them as 16-byte vectors): a buffer that does
    not is a named refusal that launches nothing and leaves the slot where it was."""
    import ctypes as C

    import torch

    from itak_torch_rebuild_b200.backend import CudaComputeError

    hq, hkv, d, n0 = 8, 2, 64, 100
    gpu, refs = build([0], hq, hkv, d, n0, 1, seed=21)
    dev = torch.device("cuda", 0)
    tq = torch.zeros(hq * d + 4, device=dev)
    tk = torch.zeros(hkv * d + 4, device=dev)
    tv = torch.zeros(hkv * d + 4, device=dev)
    out = torch.empty(hq * d, device=dev)
    before = gpu.stats()["kernel_launches"]
    one, at = (C.c_uint32 * 1)(0), (C.c_uint64 * 1)(n0)
    for off_q, off_k in ((4, 0), (0, 4), (8, 8)):
        with pytest.raises(CudaComputeError, match="16-byte aligned"):
            gpu.attention_batch_ptrs(0, one, at, 1, 1, tq.data_ptr() + off_q, tk.data_ptr() + off_k, tv.data_ptr(),
                                     out.data_ptr(), device=True)
    assert gpu.stats()["kernel_launches"] == before
    gpu.attention_batch_ptrs(0, one, at, 1, 1, tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out.data_ptr(), device=True)
    gpu.synchronize()
    refs[0].append(0, np.zeros(hkv * d, np.float32), np.zeros(hkv * d, np.float32), n0)
    assert_view_equal(gpu, refs[0], 0, DTYPE)
    gpu.close()
