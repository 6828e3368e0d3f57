"""The decode kernel's work partition, checked on the CPU through itk_decode_plan (host arithmetic only, the same
functions the kernel evaluates): whatever the batch, every 64-key tile of every (sequence, cell) is walked by exactly
one CTA, the CTAs that share a cell are numbered 0..parts-1 without gaps, no cell needs more parts than the scratch has
slots, and the cell-aligned plan is taken exactly when it costs at most a sixteenth more tiles per CTA."""
import ctypes as C

import numpy as np
import pytest

from itak_torch_rebuild_b200 import _lib


def plan(keys, cells_per_seq, ctas, splits=64):
    lib = _lib.load()
    n = len(keys)
    k = (C.c_uint32 * n)(*keys)
    aligned = C.c_uint32()
    runs = (C.c_uint32 * (6 * ctas))()
    rc = lib.itk_decode_plan(k, n, cells_per_seq, ctas, splits, C.byref(aligned), runs)
    assert rc == 0
    return bool(aligned.value), np.frombuffer(runs, dtype=np.uint32).reshape(ctas, 6).copy()


def check_partition(keys, cells_per_seq, ctas, splits=64):
    aligned, runs = plan(keys, cells_per_seq, ctas, splits)
    tiles = [(k + 63) // 64 for k in keys]
    seen = {}    # (seq, hy, tile) -> cta
    sharers = {}  # (seq, hy) -> {part: cta}
    declared = {}
    for cta, (seq, hy, tile, ntiles, parts, part) in enumerate(runs):
        first = True
        for _ in range(ntiles):
            assert seq < len(keys) and hy < cells_per_seq and tile < tiles[seq], (cta, seq, hy, tile)
            assert (seq, hy, tile) not in seen, f"tile {(seq, hy, tile)} walked twice"
            seen[(seq, hy, tile)] = cta
            if first:
                sharers.setdefault((seq, hy), {})[int(part)] = cta
                declared[(seq, hy)] = int(parts)
                first = False
            tile += 1  # the kernel's cursor: next tile, next cell, next sequence
            if tile == tiles[seq]:
                tile, hy = 0, hy + 1
                if hy == cells_per_seq:
                    hy, seq = 0, seq + 1
                assert not aligned or _ == ntiles - 1, "an aligned run crosses a cell boundary"
    total = sum(t * cells_per_seq for t in tiles)
    assert len(seen) == total, f"{total - len(seen)} tiles are walked by nobody"
    for cell, parts in declared.items():
        assert parts <= splits or not aligned
        got = sharers[cell]
        # numbering of the CTAs that START in this cell is consistent with the declared count
        assert all(0 <= p < parts for p in got), (cell, parts, sorted(got))
    return aligned, runs


def test_shard_shapes_of_the_long_context_configuration_are_cell_aligned():
    """8 sequences at context 32768+: one KV head per GPU (8 cells) gives every cell 36 of 288 CTAs, two heads 17 of
    280; the whole layer on one GPU (64 cells over 296 CTAs) keeps equal runs."""
    aligned, runs = check_partition([32772] * 8, 1, 288)
    assert aligned and (runs[:, 3] > 0).sum() == 8 * 35 and runs[:, 3].max() == 15  # 513 tiles = 34 x 15 + 3
    aligned, runs = check_partition([32772] * 8, 2, 280)
    assert aligned and runs[:, 3].max() == 31
    aligned, runs = check_partition([32772] * 8, 8, 296)
    assert not aligned and runs[:, 3].max() == 111
    # equal runs: no CTA idles, and the runs differ by at most the last one's remainder
    busy = runs[runs[:, 3] > 0, 3]
    assert (busy[:-1] == 111).all()


def test_ragged_batches_keep_equal_runs():
    rng = np.random.default_rng(3)
    keys = rng.integers(256, 8193, size=16).tolist()  # the continuous-batching configuration's lengths
    aligned, runs = check_partition(keys, 8, 296)
    assert not aligned
    busy = runs[runs[:, 3] > 0, 3]
    assert (busy[:-1] == busy[0]).all() and busy[-1] <= busy[0]  # equal runs, the last one takes the remainder
    assert len(busy) >= 290  # rounding the run length up idles a few CTAs at most


@pytest.mark.parametrize("seed", range(40))
def test_every_tile_is_walked_exactly_once(seed):
    rng = np.random.default_rng(seed)
    n = int(rng.integers(1, 17))
    if seed % 3 == 0:  # uniform batches reach the aligned plan
        keys = [int(rng.integers(1, 40000))] * n
    else:
        keys = rng.integers(1, 20000, size=n).tolist()
    cells = int(rng.choice([1, 2, 4, 8, 16]))
    ctas = int(rng.choice([1, 2, 3, 7, 37, 148, 288, 296]))
    splits = int(rng.choice([2, 8, 64]))
    check_partition(keys, cells, ctas, splits)


def test_refusals():
    lib = _lib.load()
    aligned = C.c_uint32()
    runs = (C.c_uint32 * 6)()
    assert lib.itk_decode_plan((C.c_uint32 * 1)(0), 1, 1, 1, 2, C.byref(aligned), runs) == _lib.ERR_INVALID_ARGUMENT
    assert lib.itk_decode_plan((C.c_uint32 * 1)(5), 0, 1, 1, 2, C.byref(aligned), runs) == _lib.ERR_INVALID_ARGUMENT
    assert lib.itk_decode_plan((C.c_uint32 * 1)(5), 1, 1, 0, 2, C.byref(aligned), runs) == _lib.ERR_INVALID_ARGUMENT


def batch_limits(n_seqs, cells_per_seq):
    lib = _lib.load()
    per, parts, slots = C.c_uint32(), C.c_uint32(), C.c_uint64()
    rc = lib.itk_decode_batch_limits(n_seqs, cells_per_seq, C.byref(per), C.byref(parts), C.byref(slots))
    return rc, per.value, parts.value, slots.value


@pytest.mark.parametrize("n_seqs,cells_per_seq", [(8, 8), (64, 8), (50, 96), (64, 128), (64, 2 * 37), (1, 4736), (3, 4000)])
def test_large_decode_batches_never_overrun_the_split_scratch(n_seqs, cells_per_seq):
    """A batch whose (sequence, head) cells exceed half the scratch goes out as several launches: every launch keeps
    cells x parts within the scratch and every cell keeps the two slots a stream-K cut can need (50 sequences of 96
    MHA heads, or 64 of 128 head cells, used to leave one slot per cell and write past the end)."""
    rc, per, parts, slots = batch_limits(n_seqs, cells_per_seq)
    assert rc == _lib.OK
    assert 1 <= per <= min(n_seqs, 64)
    assert 2 <= parts <= 64
    assert per * cells_per_seq * parts <= slots
    # and the plan the launcher derives for such a launch never numbers a part beyond that bound
    keys = [777] * per
    if per * cells_per_seq <= 4096:
        _, runs = plan(keys, cells_per_seq, 296, parts)
        assert runs[:, 4].max() <= max(parts, 2)


def test_a_sequence_whose_cells_do_not_fit_twice_is_refused():
    rc, _, _, slots = batch_limits(1, 4737)
    assert rc == _lib.ERR_CAPACITY and slots == 9472
