"""GPU parity of the draft-model (DFlash) attention entry point against the oracle
(crates/dflash/src/model.rs:388-466 restated; device form crates/wgpu-compute/src/kernels/k17_dflash.rs:109-251).

f32 math on both sides; the dot products and the softmax sums run in a different order on the device, so the
tolerance is the f32-cache attention tolerance: max-abs error <= 1e-4 of the output norm per (row, head)."""
import ctypes as C

import numpy as np
import pytest

from itak_torch_rebuild_b200 import _lib
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def run_device(q, positions_start, cpos, ck_compact, cv_compact, bk, bv, hq, hkv, kl, vl, causal, sliding, window,
               rows=None, block_rows=None):
    import torch

    lib = _lib.load()
    dev = torch.device("cuda", 0)
    rows = q.shape[0] if rows is None else rows
    block_rows = bk.shape[0] if block_rows is None else block_rows
    # position-addressed committed arrays, as the device form binds them; untouched rows hold NaN so that a read of
    # a position that is not in the list would show
    span = (max(cpos) + 1) if len(cpos) else 1
    ck = np.full((span, hkv * kl), np.nan, np.float32)
    cv = np.full((span, hkv * vl), np.nan, np.float32)
    for i, p in enumerate(cpos):
        ck[p], cv[p] = ck_compact[i], cv_compact[i]
    t = lambda a, dt=torch.float32: torch.as_tensor(np.ascontiguousarray(a), dtype=dt).to(dev)
    dq, dck, dcv, dbk, dbv = t(q), t(ck), t(cv), t(bk), t(bv)
    dpos = torch.as_tensor(np.asarray(cpos, dtype=np.int32), dtype=torch.int32).to(dev) if len(cpos) else None
    out = torch.full((rows, hq * vl), float("nan"), device=dev)
    err = C.create_string_buffer(256)
    rc = lib.itk_draft_attention(dq.data_ptr(), dck.data_ptr(), dcv.data_ptr(), dpos.data_ptr() if dpos is not None else None,
                                 len(cpos), dbk.data_ptr(), dbv.data_ptr(), positions_start, rows, block_rows, hq, hkv, kl,
                                 vl, int(causal), int(sliding), window, float(1.0 / np.sqrt(np.float32(kl))),
                                 out.data_ptr(), None, err, 256)
    torch.cuda.synchronize()
    return rc, err.value.decode(), out.cpu().numpy()


def rel_err(got, want, hq, vl):
    g, w = got.reshape(-1, hq, vl), want.reshape(-1, hq, vl)
    return float(np.max(np.abs(g - w).max(axis=2) / np.maximum(np.linalg.norm(w, axis=2), 1e-30)))


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("sliding,window", [(False, 0), (True, 64), (True, 1)])
@pytest.mark.parametrize("hq,hkv,kl,vl,rows,committed", [(8, 2, 128, 128, 16, 700), (4, 4, 256, 256, 7, 33),
                                                          (6, 3, 40, 24, 3, 0), (32, 8, 128, 128, 16, 2048)])
def test_draft_attention_matches_the_oracle(causal, sliding, window, hq, hkv, kl, vl, rows, committed):
    rng = np.random.default_rng(hq * 7 + kl + committed + int(causal))
    # a sparse committed set: about one position in eight was never injected
    universe = np.arange(committed + committed // 8 + 1)
    cpos = sorted(rng.choice(universe, size=committed, replace=False).tolist()) if committed else []
    start = (max(cpos) + 1) if cpos else 5
    q = rng.standard_normal((rows, hq * kl)).astype(np.float32)
    ck = rng.standard_normal((committed, hkv * kl)).astype(np.float32)
    cv = rng.standard_normal((committed, hkv * vl)).astype(np.float32)
    bk = rng.standard_normal((rows, hkv * kl)).astype(np.float32)
    bv = rng.standard_normal((rows, hkv * vl)).astype(np.float32)
    rc, msg, got = run_device(q, start, cpos, ck, cv, bk, bv, hq, hkv, kl, vl, causal, sliding, window)
    assert rc == 0, msg
    want = orc.draft_attention(q, list(range(start, start + rows)), cpos, ck, cv, bk, bv, hq, hkv, kl, vl, causal,
                               sliding, window)
    assert np.all(np.isfinite(got))
    assert rel_err(got, want, hq, vl) <= 1e-4


def test_zero_queries_give_the_uniform_mean():
    """The reference's analytic case (crates/dflash/src/model.rs:755-760) through the device path."""
    hq, hkv, kl, vl = 2, 1, 4, 4
    rng = np.random.default_rng(1)
    cv = rng.standard_normal((2, vl)).astype(np.float32)
    bv = rng.standard_normal((3, vl)).astype(np.float32)
    z = lambda n: np.zeros((n, kl), np.float32)
    rc, msg, got = run_device(np.zeros((3, hq * kl), np.float32), 2, [0, 1], z(2), cv, z(3), bv, hq, hkv, kl, vl, False,
                              False, 0)
    assert rc == 0, msg
    mean = np.concatenate([cv, bv]).astype(np.float64).mean(axis=0)
    assert np.allclose(got.reshape(3, hq, vl), mean, atol=1e-6)


def test_refusals_are_named():
    """crates/wgpu-compute/src/kernels/k17_dflash.rs:276-316"""
    z = np.zeros((1, 4), np.float32)
    rc, msg, _ = run_device(z, 0, [], z[:0], z[:0], z, z, 3, 2, 2, 2, False, False, 0)
    assert rc == _lib.ERR_INVALID_ARGUMENT and "whole multiple of kv_heads" in msg
    rc, msg, _ = run_device(z, 0, [], z[:0], z[:0], z, z, 2, 2, 2, 2, False, False, 0, rows=0)
    assert rc == _lib.ERR_INVALID_ARGUMENT and "at least one query row" in msg
    big = np.zeros((1, 300), np.float32)
    rc, msg, _ = run_device(big, 0, [], big[:0], big[:0], big, big, 1, 1, 300, 300, False, False, 0)
    assert rc == _lib.ERR_INVALID_ARGUMENT and "supported range" in msg


class Rng:
    """crates/wgpu-compute/tests/dflash_session.rs:46-61"""

    def __init__(self, seed):
        self.s = seed

    def next_f32(self):
        self.s = (self.s * 6364136223846793005 + 1442695040888963407) & ((1 << 64) - 1)
        return np.float32(self.s >> 56) / np.float32(256.0) - np.float32(0.5)


def rotate_on_device(x, positions, heads, d, rot, pairing, base):
    import torch

    lib = _lib.load()
    dev = torch.device("cuda", 0)
    dx = torch.as_tensor(np.ascontiguousarray(x, dtype=np.float32)).to(dev)
    dp = torch.as_tensor(np.asarray(positions, dtype=np.int32), dtype=torch.int32).to(dev)
    err = C.create_string_buffer(256)
    rc = lib.itk_rope_rows(dx.data_ptr(), dp.data_ptr(), len(positions), heads, d, rot, pairing, base, None, err, 256)
    torch.cuda.synchronize()
    return rc, err.value.decode(), dx.cpu().numpy()


def test_rotate_matches_torch_math_rope_on_the_reference_case():
    """crates/wgpu-compute/tests/dflash_session.rs:653-700: 3 rows at positions 0, 5, 127, 2 heads, head dim 8, inputs
    from the test's generator seeded 0x207a7e, NeoX pairing, base 10000, in place; the reference allows 1e-4 of
    absolute drift against torch_math::rope for its f32 shader, the f64 device arithmetic gets 2 ulps."""
    rows, heads, d = 3, 2, 8
    positions = [0, 5, 127]
    rng = Rng(0x207A7E)
    x = np.array([rng.next_f32() for _ in range(rows * heads * d)], dtype=np.float32).reshape(rows, heads, d)
    rc, msg, got = rotate_on_device(x, positions, heads, d, d, 1, 10000.0)
    assert rc == 0, msg
    for r, p in enumerate(positions):
        for h in range(heads):
            want = orc.rope(x[r, h], p, 10000.0, d)
            assert np.max(np.abs(got[r, h] - want)) < 1e-4
            assert np.all(np.abs(got[r, h] - want) <= 2 * np.spacing(np.abs(want)) + 1e-7)


@pytest.mark.parametrize("pairing", [0, 1])
@pytest.mark.parametrize("heads,d,rot", [(8, 128, 128), (4, 64, 32), (2, 256, 256)])
def test_rotate_at_scattered_positions(pairing, heads, d, rot):
    rng = np.random.default_rng(d + pairing)
    positions = [0, 3, 4, 1000, 32767, 131071, 7]
    x = rng.standard_normal((len(positions), heads, d)).astype(np.float32)
    rc, msg, got = rotate_on_device(x, positions, heads, d, rot, pairing, 500000.0)
    assert rc == 0, msg
    fn = orc.rope_interleaved if pairing == 0 else orc.rope
    for r, p in enumerate(positions):
        for h in range(heads):
            want = fn(x[r, h], p, 500000.0, d, rot)
            assert np.all(np.abs(got[r, h] - want) <= 4 * np.spacing(np.abs(want)) + 1e-7), (r, h)


def test_rotate_refusals_are_named():
    """crates/wgpu-compute/src/kernels/k17_dflash.rs:255-271"""
    x = np.zeros((1, 1, 8), np.float32)
    rc, msg, _ = rotate_on_device(x, [], 1, 8, 8, 1, 10000.0)
    assert rc == _lib.ERR_INVALID_ARGUMENT and msg == "rotate needs at least one row and head, got rows 0, heads 1"
    rc, msg, _ = rotate_on_device(np.zeros((1, 1, 7), np.float32), [0], 1, 7, 6, 1, 10000.0)
    assert rc == _lib.ERR_INVALID_ARGUMENT and msg == "head_dim 7 must be even and at least 2"
    rc, msg, _ = rotate_on_device(x, [0], 1, 8, 8, 1, 1.0)
    assert rc == _lib.ERR_INVALID_ARGUMENT and "base must be finite and > 1" in msg
