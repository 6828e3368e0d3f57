"""The committed fixtures of tests/golden/ (written by tests/golden/make_golden.py from the oracle, on the inputs of
the reference's own fixtures): the byte formats parsed by hand from their documented layouts
(crates/itak-kv/src/snapshot.rs:13-29, crates/itak-kv/src/store.rs:5-21), reproduced by the oracle and by the
product, and an attention result reproduced by the oracle (bit for bit) and by the CUDA path (to tolerance)."""
import json
import os
import struct

import numpy as np
import pytest

from itak_torch_rebuild_b200.prefix_store import PrefixStore
from oracle import oracle as orc
from oracle import prefix_store as ops

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TOKENS = [10, 20, 30, 40, 50]


def read(name):
    with open(os.path.join(GOLDEN, name), "rb") as f:
        return f.read()


def fnv1a64(data: bytes, basis=0xcbf29ce484222325) -> int:
    h = basis
    for b in data:
        h = ((h ^ b) * 0x00000100000001b3) & 0xFFFFFFFFFFFFFFFF
    return h


def test_snapshot_fixture_follows_the_documented_layout():
    """snapshot.rs:13-29, field by field, with the checksum recomputed here."""
    data = read("snapshot_model_a.itkv")
    assert data[:4] == b"ITKV"
    version, fp_len = struct.unpack_from("<II", data, 4)
    assert version == 1 and data[12:12 + fp_len] == b"model-a"
    at = 12 + fp_len
    token_count, hkv, d, layers = struct.unpack_from("<QIII", data, at)
    assert (token_count, hkv, d, layers) == (5, 2, 3, 2)
    at += 20
    headers = []
    for _ in range(layers):
        kind, r0, r1, r2, window, first, rows = struct.unpack_from("<BBBBQQQ", data, at)
        assert (r0, r1, r2) == (0, 0, 0)
        headers.append((kind, window, first, rows))
        at += 28
    assert headers == [(1, 4, 1, 4), (0, 0, 0, 5)]  # windowed(4): last 4 rows from position 1; global: all 5
    floats = sum(rows * hkv * d * 2 for _, _, _, rows in headers)
    assert len(data) == at + 4 * floats + 8
    (stored,) = struct.unpack_from("<Q", data, len(data) - 8)
    assert stored == fnv1a64(data[:-8])
    # first K row of the global layer: token 10 at position 0, layer 1: 10 + (0*10 + 1 + i) / 11 (store.rs:680-682)
    global_k = at + 4 * headers[0][3] * hkv * d * 2
    row = struct.unpack_from("<6f", data, global_k)
    want = [np.float32(10) + np.float32(1 + i) / np.float32(11.0) for i in range(6)]
    assert list(np.float32(row)) == want


def test_entry_fixture_follows_the_documented_layout():
    """store.rs:5-21"""
    data, payload = read("entry_model_a.kv"), read("snapshot_model_a.itkv")
    assert data[:8] == b"ITKVPENT"
    version, reserved, created, last_used, key, count, tokens_bytes, payload_bytes, reserved2 = struct.unpack_from(
        "<IIQQQQQQQ", data, 8)
    assert (version, reserved, created, last_used, count, tokens_bytes, payload_bytes, reserved2) == (
        1, 0, 100, 100, 5, 20, len(payload), 0)
    token_bytes = b"".join(struct.pack("<I", t) for t in TOKENS)
    assert key == fnv1a64(token_bytes)  # hash.rs:44-47
    assert data[72:92] == token_bytes and data[92:] == payload
    disc = fnv1a64(token_bytes, 0x84222325cbf29ce4)  # hash.rs:21, 51-56
    assert read("entry_model_a.name").decode().strip() == f"{key:016x}-5-{disc:016x}.kv"


def test_oracle_and_product_reproduce_the_fixtures(tmp_path):
    payload, entry = read("snapshot_model_a.itkv"), read("entry_model_a.kv")
    name = read("entry_model_a.name").decode().strip()
    snap = orc.KvSnapshot.from_bytes(payload)
    assert snap.token_count == 5 and snap.to_bytes() == payload
    assert ops.entry_bytes(TOKENS, payload, 100) == entry and ops.file_name_for(TOKENS) == name
    store = PrefixStore(str(tmp_path), 1 << 20)
    store.put(TOKENS, payload, 100)
    assert (tmp_path / name).read_bytes() == entry
    # and an entry file dropped into a directory is served as it is
    other = tmp_path / "other"
    other.mkdir()
    (other / name).write_bytes(entry)
    hit = PrefixStore(str(other), 1 << 20).lookup(TOKENS + [60], now=101)
    assert hit.token_count == 5 and hit.snapshot_bytes == payload


def golden_attention():
    g = json.loads(read("attention_seed35.json"))
    rows, stored_n, first, seed, hq, hkv, d = (g[k] for k in ("rows", "stored", "first_pos", "seed", "q_heads", "kv_heads",
                                                              "head_dim"))
    q = orc.lcg(seed, rows * hq * d)
    k = orc.lcg(seed + 1, (first + stored_n) * hkv * d).reshape(-1, hkv * d)[first:]
    v = orc.lcg(seed + 2, (first + stored_n) * hkv * d).reshape(-1, hkv * d)[first:]
    return g, q, k, v, np.asarray(g["out"], dtype=np.float32)


def test_oracle_reproduces_the_attention_fixture_bit_for_bit():
    g, q, k, v, want = golden_attention()
    cache = orc.KvCache([orc.GLOBAL], g["kv_heads"], g["head_dim"])
    cache.append_rows(0, k, v, 0)
    start = g["stored"] - g["rows"]
    got = orc.gqa_attention(q, g["rows"], g["q_heads"], list(range(start, start + g["rows"])), cache.view(0))
    assert got.tobytes() == want.tobytes()


@pytest.mark.gpu
def test_cuda_path_reproduces_the_attention_fixture():
    from itak_torch_rebuild_b200 import CudaCompute, KvDtype, PositionCache

    g, q, k, v, want = golden_attention()
    rows, hq, hkv, d, n = g["rows"], g["q_heads"], g["kv_heads"], g["head_dim"], g["stored"]
    gpu = CudaCompute(1, hq, hkv, d, n_slots=1, max_context=64, chunk_cap=rows, kv_dtype=KvDtype.F32)
    gpu.append_rows(0, k[: n - rows], v[: n - rows], 0)
    pos = PositionCache()
    pos.advance(n - rows)
    got = gpu.attention(0, q, k[n - rows:], v[n - rows:], pos)
    err = np.abs(got - want).reshape(rows, hq, d).max(axis=2) / np.linalg.norm(want.reshape(rows, hq, d), axis=2)
    assert err.max() <= 1e-4  # the f32-cache tolerance
