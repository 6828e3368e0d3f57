"""The N > 1 path on CPU: two gloo ranks shard the KV heads of one layer, each computes its heads' attention
with the CPU oracle standing in for the device, the per-head outputs are all-gathered as ``bench.py`` does, and
the gathered tensor equals the unsharded result bit for bit."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from itak_torch_rebuild_b200 import sharding  # noqa: E402


def test_plan_covers_every_head_and_sequence_once():
    for hq, hkv, seqs in [(64, 8, 8), (32, 8, 16), (32, 2, 3)]:
        for world in (1, 2, 4, 8):
            if world <= hkv and hkv % world:
                continue
            seen = set()
            for r in range(world):
                s = sharding.plan(hq, hkv, seqs, r, world)
                for h in range(s.kv_head_begin, s.kv_head_begin + s.kv_heads):
                    for q in range(s.seq_begin, s.seq_begin + s.seqs):
                        assert (h, q) not in seen
                        seen.add((h, q))
                assert s.q_heads == s.kv_heads * (hq // hkv)
            assert len(seen) == hkv * seqs
    assert sharding.gathered_head_order(64, 8, 8) == list(range(64))
    with pytest.raises(ValueError):
        sharding.plan(64, 8, 8, 0, 3)


def _worker(rank, world, port, hq, hkv, d, n, out_queue):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as orc

    rng = np.random.default_rng(5)  # every rank draws the same global tensors
    k = rng.standard_normal((n, hkv, d)).astype(np.float32)
    v = rng.standard_normal((n, hkv, d)).astype(np.float32)
    q = rng.standard_normal((hq, d)).astype(np.float32)
    s = sharding.plan(hq, hkv, 1, rank, world)
    cache = orc.KvCache([orc.GLOBAL], s.kv_heads, d)
    hs = slice(s.kv_head_begin, s.kv_head_begin + s.kv_heads)
    cache.append_rows(0, k[:, hs].reshape(n, -1), v[:, hs].reshape(n, -1), 0)
    local = orc.gqa_attention(q[s.q_head_begin:s.q_head_begin + s.q_heads], 1, s.q_heads, [n - 1], cache.view(0))
    local_t = torch.from_numpy(local.reshape(s.q_heads * d).copy())
    gathered = torch.empty(world * s.q_heads * d)
    dist.all_gather_into_tensor(gathered, local_t)
    if rank == 0:
        full = orc.KvCache([orc.GLOBAL], hkv, d)
        full.append_rows(0, k.reshape(n, -1), v.reshape(n, -1), 0)
        want = orc.gqa_attention(q, 1, hq, [n - 1], full.view(0))
        order = sharding.gathered_head_order(hq, hkv, world)
        got = gathered.numpy().reshape(hq, d)[np.argsort(order)].reshape(-1)
        out_queue.put(bool(got.tobytes() == want.tobytes()))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_shard_heads_and_gather_the_unsharded_answer():
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, 16, 4, 8, 37, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert q.get() is True
