"""Writes the fixtures of this directory from the CPU oracle (run from the repository root:
``python tests/golden/make_golden.py``).  The reference is a Rust workspace and cannot be executed here, so these
are not outputs of the reference itself: they are outputs of its restatement, after that restatement passed the
reference's own known-answer tests (tests/test_oracle_*.py), on the inputs of the reference's own fixtures.  They
freeze the byte formats and a few attention results so that a change to the oracle or to the product that moves a
bit shows up against a committed file, not only against the other implementation.

  snapshot_model_a.itkv     the snapshot of crates/itak-kv/src/store.rs:674-691 for tokens [10, 20, 30, 40, 50] and
                            fingerprint "model-a" (layers windowed(4) + global, 2 KV heads, head dim 3), ITKV bytes
  entry_model_a.kv          the prefix-store entry file PrefixStore::put writes for it at now = 100 (store.rs:5-21)
  entry_model_a.name        its file name (store.rs:459-468)
  attention_seed35.json     crates/wgpu-compute/tests/fused_kernels.rs:506-624, geometry 3 (3 rows, 37 stored rows from
                            position 5, 4 query / 2 KV heads, head dim 64, lcg seeds 35..37): f32-cache outputs
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

from oracle import oracle as orc  # noqa: E402
from oracle import prefix_store as ops  # noqa: E402


def store_snapshot(tokens, fingerprint):
    geometry = orc.KvGeometry([orc.LayerKind.Windowed(4), orc.GLOBAL], 2, 3)
    cache = orc.KvCache(geometry.layers, geometry.num_kv_heads, geometry.head_dim)
    row = geometry.row_floats()
    for position, token in enumerate(tokens):
        for layer in range(len(geometry.layers)):
            k = [np.float32(token) + np.float32(position * 10 + layer + i) / np.float32(11.0) for i in range(row)]
            v = [-(np.float32(token) + np.float32(position + layer * 3 + i) / np.float32(5.0)) for i in range(row)]
            cache.append(layer, k, v, position)
    return orc.KvSnapshot.capture(cache, fingerprint)


def attention_seed35():
    rows, stored_n, first_pos, seed, hq, hkv, d = 3, 37, 5, 35, 4, 2, 64
    q = orc.lcg(seed, rows * hq * d)
    k = orc.lcg(seed + 1, (first_pos + stored_n) * hkv * d).reshape(-1, hkv * d)[first_pos:]
    v = orc.lcg(seed + 2, (first_pos + stored_n) * hkv * d).reshape(-1, hkv * d)[first_pos:]
    cache = orc.KvCache([orc.GLOBAL], hkv, d)
    # positions shifted to start at 0: nothing inside attention depends on absolute positions
    cache.append_rows(0, k, v, 0)
    start = stored_n - rows
    out = orc.gqa_attention(q, rows, hq, list(range(start, start + rows)), cache.view(0))
    return {"rows": rows, "stored": stored_n, "first_pos": first_pos, "seed": seed, "q_heads": hq, "kv_heads": hkv,
            "head_dim": d, "out": [float(x) for x in out]}


def main():
    tokens = [10, 20, 30, 40, 50]
    snap = store_snapshot(tokens, "model-a")
    payload = snap.to_bytes()
    with open(os.path.join(HERE, "snapshot_model_a.itkv"), "wb") as f:
        f.write(payload)
    with open(os.path.join(HERE, "entry_model_a.kv"), "wb") as f:
        f.write(ops.entry_bytes(tokens, payload, 100))
    with open(os.path.join(HERE, "entry_model_a.name"), "w") as f:
        f.write(ops.file_name_for(tokens) + "\n")
    with open(os.path.join(HERE, "attention_seed35.json"), "w") as f:
        json.dump(attention_seed35(), f)
    print("wrote", sorted(os.listdir(HERE)))


if __name__ == "__main__":
    main()
