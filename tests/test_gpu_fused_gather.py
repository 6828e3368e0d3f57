"""The all-gather fused into the decode kernel, on 2 GPUs: each rank holds half of the KV heads, runs the replayable
loop with itk_resident_layer_gather - with and without the two-lane schedule - and every rank's gather buffer must
end up holding every rank's head outputs: the same values an NCCL all-gather of the ordinary per-rank outputs
delivers.  Needs two GPUs; skipped otherwise."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

pytestmark = pytest.mark.gpu


class _DevArray:
    """A device pointer dressed as a CUDA array so torch can view it."""

    def __init__(self, ptr, n):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (ptr, False), "version": 2}


def _worker(rank, world, port, use_graph, lanes, result):
    import torch
    import torch.distributed as dist

    from itak_torch_rebuild_b200 import CudaCompute, KvDtype, sharding

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    layers, hq, hkv, d, steps = 3, 16, 4, 128, 4
    lens = [200, 77]
    n = len(lens)
    sh = sharding.plan(hq, hkv, n, rank, world)
    a = CudaCompute(layers, sh.q_heads, sh.kv_heads, d, n_slots=n, max_context=400, chunk_cap=1, kv_dtype=KvDtype.F16,
                    device=rank, options={"decode_lanes": lanes})  # fused loop
    b = CudaCompute(layers, sh.q_heads, sh.kv_heads, d, n_slots=n, max_context=400, chunk_cap=1, kv_dtype=KvDtype.F16,
                    device=rank)  # ordinary calls
    rng = np.random.default_rng(4)  # every rank draws the same global tensors and keeps its heads
    ks = slice(sh.kv_head_begin * d, (sh.kv_head_begin + sh.kv_heads) * d)
    qs = slice(sh.q_head_begin * d, (sh.q_head_begin + sh.q_heads) * d)
    for slot, ln in enumerate(lens):
        for layer in range(layers):
            k = rng.standard_normal((ln, hkv * d)).astype(np.float32)[:, ks]
            v = rng.standard_normal((ln, hkv * d)).astype(np.float32)[:, ks]
            a.append_rows(layer, k, v, 0, slot=slot)
            b.append_rows(layer, k, v, 0, slot=slot)
    stream = torch.cuda.Stream(device=dev)
    a.set_stream(stream.cuda_stream)
    slot_floats = n * sh.q_heads * d
    data_bytes = layers * world * slot_floats * 4
    ptr, handle = a.gather_create(world, rank, data_bytes)
    handles = [None] * world
    dist.all_gather_object(handles, handle)
    for r in range(world):
        a.gather_open(r, handles[r])
    gathered = torch.as_tensor(_DevArray(ptr, layers * world * slot_floats), device=dev).view(layers, world, n, -1)
    a.gather_reset()
    dist.barrier()
    torch.cuda.synchronize()

    q = rng.standard_normal((steps, layers, n, hq * d)).astype(np.float32)[..., qs]
    k = rng.standard_normal((steps, layers, n, hkv * d)).astype(np.float32)[..., ks]
    v = rng.standard_normal((steps, layers, n, hkv * d)).astype(np.float32)[..., ks]
    q_d = torch.empty((layers, n, sh.q_heads * d), device=dev)
    k_d = torch.empty((layers, n, sh.kv_heads * d), device=dev)
    v_d = torch.empty((layers, n, sh.kv_heads * d), device=dev)

    def step_launches():
        for layer in range(layers):
            off = (layer * world + rank) * slot_floats * 4
            a.resident_layer_gather(layer, q_d[layer].data_ptr(), k_d[layer].data_ptr(), v_d[layer].data_ptr(), off)
        a.resident_advance()

    a.resident_begin(list(range(n)), steps)
    ok = True
    graph = None
    with torch.cuda.stream(stream):
        if use_graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                step_launches()
        for s in range(steps):
            q_d.copy_(torch.from_numpy(np.ascontiguousarray(q[s])))
            k_d.copy_(torch.from_numpy(np.ascontiguousarray(k[s])))
            v_d.copy_(torch.from_numpy(np.ascontiguousarray(v[s])))
            if graph is not None:
                graph.replay()
            else:
                step_launches()
            stream.synchronize()
            dist.barrier()  # every rank's kernels are done, so all peer stores have landed
            torch.cuda.synchronize()
            got = gathered.cpu().numpy()
            for layer in range(layers):
                mine = b.attention_batch(layer, list(range(n)), [lens[i] + s for i in range(n)], 1,
                                         np.ascontiguousarray(q[s, layer]), np.ascontiguousarray(k[s, layer]),
                                         np.ascontiguousarray(v[s, layer])).reshape(n, -1)
                want = torch.empty((world, n, sh.q_heads * d), device=dev)
                dist.all_gather_into_tensor(want, torch.from_numpy(mine).to(dev))
                want = want.cpu().numpy()
                err = np.abs(got[layer] - want).max() / np.abs(want).max()
                ok = ok and bool(err <= 1e-5)
            dist.barrier()
    a.resident_end(steps)
    ok = ok and a.gather_status() == 0
    if rank == 0:
        result.put(ok)
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0)


@pytest.mark.parametrize("lanes", [0, 2])
@pytest.mark.parametrize("use_graph", [False, True])
def test_fused_gather_matches_nccl_all_gather(use_graph, lanes):
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    ctx = mp.get_context("spawn")
    result = ctx.SimpleQueue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, use_graph, lanes, result)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
        if p.is_alive():
            p.kill()
            pytest.fail("a rank did not finish")
        assert p.exitcode == 0
    assert result.get() is True
