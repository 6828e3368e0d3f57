"""The replayable decode loop (device-side positions): its steps equal the ordinary per-layer step calls, both
when launched directly and when one step is captured in a CUDA graph and replayed."""
import numpy as np
import pytest

from itak_torch_rebuild_b200 import CudaCompute, CudaComputeError, KvDtype, _lib

from kvparity import assert_view_equal, attention_error, make_pair, stored
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def build(layer_window, hq, hkv, d, lens, cap, seed):
    gpu, refs = make_pair(layer_window, hq, hkv, d, dtype=KvDtype.F16, n_slots=len(lens), max_context=cap, chunk_cap=1)
    rng = np.random.default_rng(seed)
    for slot, n in enumerate(lens):
        for layer in range(len(layer_window)):
            k = rng.standard_normal((n, hkv * d)).astype(np.float32)
            v = rng.standard_normal((n, hkv * d)).astype(np.float32)
            at = 0
            while at < n:  # one row at a time on ring layers (chunk cap 1), bulk on global ones
                m = n - at if layer_window[layer] == 0 else 1
                gpu.append_rows(layer, k[at:at + m], v[at:at + m], at, slot=slot)
                at += m
            refs[slot].append_rows(layer, stored(k, KvDtype.F16), stored(v, KvDtype.F16), 0)
    return gpu, refs


@pytest.mark.parametrize("use_graph", [False, True])
def test_resident_steps_equal_ordinary_steps(use_graph):
    import torch

    layer_window, hq, hkv, d = [0, 48], 32, 8, 128
    lens, steps = [300, 70, 515], 5
    layers, n = len(layer_window), len(lens)
    a, refs = build(layer_window, hq, hkv, d, lens, 600, seed=3)   # resident loop
    b, _ = build(layer_window, hq, hkv, d, lens, 600, seed=3)      # ordinary calls
    dev = torch.device("cuda", 0)
    stream = torch.cuda.Stream(device=dev)
    a.set_stream(stream.cuda_stream)
    rng = np.random.default_rng(9)
    q = rng.standard_normal((steps, layers, n, hq * d)).astype(np.float32)
    k = rng.standard_normal((steps, layers, n, hkv * d)).astype(np.float32)
    v = rng.standard_normal((steps, layers, n, hkv * d)).astype(np.float32)
    # the step's inputs live in fixed device buffers (a captured step reads the same addresses every replay)
    q_d = torch.empty((layers, n, hq * d), device=dev)
    k_d = torch.empty((layers, n, hkv * d), device=dev)
    v_d = torch.empty((layers, n, hkv * d), device=dev)
    out_d = torch.empty((layers, n, hq * d), device=dev)

    def step_launches():
        for layer in range(layers):
            a.resident_layer(layer, q_d[layer].data_ptr(), k_d[layer].data_ptr(), v_d[layer].data_ptr(),
                             out_d[layer].data_ptr())
        a.resident_advance()

    slots = list(range(n))
    a.resident_begin(slots, steps)
    with pytest.raises(CudaComputeError) as e:
        a.resident_begin(slots, steps)
    assert e.value.code == _lib.ERR_INVALID_ARGUMENT
    graph = None
    with torch.cuda.stream(stream):
        if use_graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                step_launches()
        for s in range(steps):
            q_d.copy_(torch.from_numpy(q[s]))
            k_d.copy_(torch.from_numpy(k[s]))
            v_d.copy_(torch.from_numpy(v[s]))
            if graph is not None:
                graph.replay()
            else:
                step_launches()
            stream.synchronize()
            got = out_d.cpu().numpy()
            for layer in range(layers):
                want = b.attention_batch(layer, slots, [lens[i] + s for i in range(n)], 1, q[s, layer], k[s, layer],
                                         v[s, layer]).reshape(n, -1)
                # the two routes may cut the key ranges differently (different f32 summation order)
                assert attention_error(got[layer], want, hq, d) <= 1e-5, f"step {s} layer {layer}"
    a.resident_end(steps)
    for slot in range(n):
        for layer in range(layers):
            assert a.next_position(layer, slot=slot) == lens[slot] + steps
            fa, ka, va = a.view(layer, slot=slot)
            fb, kb, vb = b.view(layer, slot=slot)
            assert fa == fb and ka.tobytes() == kb.tobytes() and va.tobytes() == vb.tobytes()
    # and the loop's cache equals the oracle fed the same rows
    for slot in range(n):
        for s in range(steps):
            for layer in range(layers):
                refs[slot].append(layer, stored(k[s, layer, slot], KvDtype.F16), stored(v[s, layer, slot], KvDtype.F16),
                                  lens[slot] + s)
        for layer in range(layers):
            assert_view_equal(a, refs[slot], layer, KvDtype.F16, slot=slot)


def test_resident_loop_refusals():
    gpu = CudaCompute(2, 8, 2, 64, n_slots=2, max_context=16, chunk_cap=1, kv_dtype=KvDtype.F16)
    gpu.append(0, np.zeros(128), np.zeros(128), 0)
    with pytest.raises(CudaComputeError) as e:  # layers at different positions
        gpu.resident_begin([0], 2)
    assert e.value.code == _lib.ERR_INCOHERENT_CACHE
    gpu.append(1, np.zeros(128), np.zeros(128), 0)
    with pytest.raises(CudaComputeError) as e:  # past the context capacity
        gpu.resident_begin([0], 16)
    assert e.value.code == _lib.ERR_CAPACITY
    with pytest.raises(CudaComputeError) as e:
        gpu.resident_layer(0, 1, 1, 1, 1)
    assert e.value.code == _lib.ERR_INVALID_ARGUMENT and "not active" in e.value.msg
    gpu.resident_begin([0], 4)
    with pytest.raises(CudaComputeError) as e:
        gpu.resident_end(5)
    assert e.value.code == _lib.ERR_INVALID_ARGUMENT
    gpu.resident_end(0)
    assert gpu.next_position(0) == 1
    f32 = CudaCompute(1, 8, 2, 64, n_slots=1, max_context=16, chunk_cap=1, kv_dtype=KvDtype.F32)
    with pytest.raises(CudaComputeError) as e:
        f32.resident_begin([0], 1)
    assert e.value.code == _lib.ERR_INVALID_ARGUMENT


@pytest.mark.parametrize("q_scale", [1.0, 40.0])
def test_resident_loop_cells_shared_by_many_ctas(q_scale):
    """A KV-head shard's shape - few (sequence, head) cells, each shared by dozens of CTAs - takes the cell-aligned plan
    and sums the parts with reductions in L2 instead of merging them one by one; scores beyond the range that keeps
    such sums safe (q_scale 40: maxima of several hundred in the log2 domain) send the cell down the exact merge.
    Both must match the oracle on every step and layer (the accumulators are cleared between launches)."""
    import torch

    layer_window, hq, hkv, d = [0, 0], 8, 1, 128
    lens, steps = [2500, 2449], 3
    layers, n = len(layer_window), len(lens)
    a, refs = build(layer_window, hq, hkv, d, lens, 2600, seed=21)
    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(4)
    q = (q_scale * rng.standard_normal((steps, layers, n, hq * d))).astype(np.float32)
    k = rng.standard_normal((steps, layers, n, hkv * d)).astype(np.float32)
    v = rng.standard_normal((steps, layers, n, hkv * d)).astype(np.float32)
    q_d = torch.empty((layers, n, hq * d), device=dev)
    k_d = torch.empty((layers, n, hkv * d), device=dev)
    v_d = torch.empty((layers, n, hkv * d), device=dev)
    out_d = torch.empty((layers, n, hq * d), device=dev)
    slots = list(range(n))
    a.resident_begin(slots, steps)
    for s in range(steps):
        q_d.copy_(torch.from_numpy(q[s]))
        k_d.copy_(torch.from_numpy(k[s]))
        v_d.copy_(torch.from_numpy(v[s]))
        torch.cuda.synchronize()
        for layer in range(layers):
            a.resident_layer(layer, q_d[layer].data_ptr(), k_d[layer].data_ptr(), v_d[layer].data_ptr(),
                             out_d[layer].data_ptr())
        a.resident_advance()
        a.synchronize()
        got = out_d.cpu().numpy()
        for slot in range(n):
            for layer in range(layers):
                refs[slot].append(layer, stored(k[s, layer, slot], KvDtype.F16), stored(v[s, layer, slot], KvDtype.F16),
                                  lens[slot] + s)
                want = orc.gqa_attention(q[s, layer, slot], 1, hq, [lens[slot] + s], refs[slot].view(layer))
                assert attention_error(got[layer, slot], want, hq, d) <= 2e-3, f"step {s} layer {layer} slot {slot}"
    a.resident_end(steps)


class _DevArray:
    """A device pointer dressed as a CUDA array so torch can view it."""

    def __init__(self, ptr, n):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (ptr, False), "version": 2}


@pytest.mark.parametrize("use_graph", [False, True])
@pytest.mark.parametrize("lanes,stagger", [(2, 100), (2, 0), (0, 100)])
@pytest.mark.parametrize("lens", [[2500, 2449, 2610, 2388], [700, 64, 1531, 2047, 300]])
def test_gathering_loop_on_one_rank_equals_the_oracle(use_graph, lanes, stagger, lens):
    """The gathering form of the loop with this GPU as its only rank (the gather buffer is local): with the two-lane
    schedule - half of the CTAs per half of the batch, per-lane arrival counters, no wait for the previous launch
    except through those counters - and without it, every step's gathered rows equal the oracle's attention, the
    cache ends bit-equal to the oracle's, and no wait runs out.  Even and ragged batches (the ragged one cuts the
    lanes unevenly and takes the equal-run plan inside them)."""
    import torch

    layer_window, hq, hkv, d = [0, 0, 0], 8, 1, 128
    steps, layers, n = 4, 3, len(lens)
    a, refs = build(layer_window, hq, hkv, d, lens, max(lens) + 16, seed=5)
    a.set_option("decode_lanes", lanes)
    a.set_option("decode_lane_stagger", stagger)
    dev = torch.device("cuda", 0)
    stream = torch.cuda.Stream(device=dev)
    a.set_stream(stream.cuda_stream)
    rng = np.random.default_rng(11)
    q = rng.standard_normal((steps, layers, n, hq * d)).astype(np.float32)
    k = rng.standard_normal((steps, layers, n, hkv * d)).astype(np.float32)
    v = rng.standard_normal((steps, layers, n, hkv * d)).astype(np.float32)
    q_d = torch.empty((layers, n, hq * d), device=dev)
    k_d = torch.empty((layers, n, hkv * d), device=dev)
    v_d = torch.empty((layers, n, hkv * d), device=dev)
    slot_floats = n * hq * d
    ptr, _ = a.gather_create(1, 0, layers * slot_floats * 4)
    gathered = torch.as_tensor(_DevArray(ptr, layers * slot_floats), device=dev).view(layers, n, hq * d)
    a.gather_reset()

    def step_launches():
        for layer in range(layers):
            a.resident_layer_gather(layer, q_d[layer].data_ptr(), k_d[layer].data_ptr(), v_d[layer].data_ptr(),
                                    layer * slot_floats * 4)
        a.resident_advance()

    a.resident_begin(list(range(n)), steps)
    graph = None
    with torch.cuda.stream(stream):
        if use_graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                step_launches()
        for s in range(steps):
            q_d.copy_(torch.from_numpy(q[s]))
            k_d.copy_(torch.from_numpy(k[s]))
            v_d.copy_(torch.from_numpy(v[s]))
            gathered.fill_(float("nan"))
            stream.synchronize()
            if graph is not None:
                graph.replay()
            else:
                step_launches()
            stream.synchronize()
            got = gathered.cpu().numpy()
            assert np.all(np.isfinite(got)), f"step {s}: a cell was never delivered"
            for layer in range(layers):
                for slot in range(n):
                    refs[slot].append(layer, stored(k[s, layer, slot], KvDtype.F16), stored(v[s, layer, slot], KvDtype.F16),
                                      lens[slot] + s)
                    want = orc.gqa_attention(q[s, layer, slot], 1, hq, [lens[slot] + s], refs[slot].view(layer))
                    assert attention_error(got[layer, slot], want, hq, d) <= 2e-3, f"step {s} layer {layer} slot {slot}"
    a.resident_end(steps)
    assert a.gather_status() == 0
    for slot in range(n):
        for layer in range(layers):
            assert_view_equal(a, refs[slot], layer, KvDtype.F16, slot=slot)


@pytest.mark.parametrize("lanes", [0, 2])
def test_a_peer_that_never_delivers_makes_the_wait_run_out_not_hang(lanes):
    """Failure detection of the fused gather, on one GPU: rank 0 of a two-rank gather whose second rank is a buffer
    that nobody ever signals.  With a short poll limit every launch after the first gives up its wait for that rank,
    records bit 0 in the status word and carries on: the kernels return, this rank's own rows - in its own buffer and
    in the silent peer's - still equal the oracle, and after a reset an ordinary call works."""
    import torch

    layer_window, hq, hkv, d = [0, 0], 8, 1, 128
    lens, steps = [300, 257], 2
    layers, n = 2, len(lens)
    a, refs = build(layer_window, hq, hkv, d, lens, 400, seed=8)
    silent = CudaCompute(layers, hq, hkv, d, n_slots=n, max_context=400, chunk_cap=1, kv_dtype=KvDtype.F16)
    a.set_option("gather_poll_limit", 2000)
    a.set_option("decode_lanes", lanes)
    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(2)
    q = rng.standard_normal((steps, layers, n, hq * d)).astype(np.float32)
    k = rng.standard_normal((steps, layers, n, hkv * d)).astype(np.float32)
    v = rng.standard_normal((steps, layers, n, hkv * d)).astype(np.float32)
    slot_floats = n * hq * d
    world = 2
    nbytes = layers * world * slot_floats * 4
    mine, _ = a.gather_create(world, 0, nbytes)
    theirs, _ = silent.gather_create(world, 1, nbytes)
    a.gather_attach(1, theirs)
    views = [torch.as_tensor(_DevArray(p, layers * world * slot_floats), device=dev).view(layers, world, n, hq * d)
             for p in (mine, theirs)]
    a.gather_reset()
    silent.gather_reset()
    a.resident_begin(list(range(n)), steps)
    for s in range(steps):
        q_d, k_d, v_d = (torch.from_numpy(x[s]).to(dev) for x in (q, k, v))
        for layer in range(layers):
            a.resident_layer_gather(layer, q_d[layer].data_ptr(), k_d[layer].data_ptr(), v_d[layer].data_ptr(),
                                    (layer * world + 0) * slot_floats * 4)
        a.resident_advance()
        a.synchronize()  # returns: nothing hangs on the silent rank
        for layer in range(layers):
            for slot in range(n):
                refs[slot].append(layer, stored(k[s, layer, slot], KvDtype.F16), stored(v[s, layer, slot], KvDtype.F16),
                                  lens[slot] + s)
                want = orc.gqa_attention(q[s, layer, slot], 1, hq, [lens[slot] + s], refs[slot].view(layer))
                for view in views:
                    got = view[layer, 0, slot].cpu().numpy()
                    assert attention_error(got, want, hq, d) <= 2e-3, f"step {s} layer {layer} slot {slot}"
    a.resident_end(steps)
    assert a.gather_status() == 1, "the wait for the silent rank should have run out"
    assert silent.gather_status() == 0
    a.gather_reset()
    assert a.gather_status() == 0
    for slot in range(n):
        for layer in range(layers):
            assert_view_equal(a, refs[slot], layer, KvDtype.F16, slot=slot)
    out = a.attention_batch(0, [0], [lens[0] + steps], 1, q[0, 0, 0], k[0, 0, 0], v[0, 0, 0])
    refs[0].append(0, stored(k[0, 0, 0], KvDtype.F16), stored(v[0, 0, 0], KvDtype.F16), lens[0] + steps)
    want = orc.gqa_attention(q[0, 0, 0], 1, hq, [lens[0] + steps], refs[0].view(0))
    assert attention_error(out, want, hq, d) <= 2e-3
