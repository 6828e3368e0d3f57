"""Measurement of the hot path's other configurations on one B200, each in the JSON shape of a bench.py line
(bench.py runs short forms of all of them inside its default line's `paths` record, or one of them at full
length with `--workload NAME`):

  c1_tinyllama_f32        22 layers, 32 q / 4 KV heads, head dim 64, f32 cache, one sequence: a 512-row prefill
                          (one multi-row call per layer), then 64 decode steps.  Metric: decode steps/s.
  c3_continuous_batching  32 layers, 32 q / 8 KV heads, head dim 128, f16 cache, 16 resident slots with ragged
                          contexts uniform in [256, 8192]; every step appends one token per slot and attends; each
                          slot retires on its own 64-step period (slot i at steps = 4 i mod 64) and is refilled by
                          a reset + bulk append of a new prompt of a freshly drawn length.  Metric: steps/s.
  c4_prefix_restore       a 2048-token shared prefix (32 layers, 8 KV heads, head dim 128, f16 = 256 MiB) captured
                          once and restored into 16 sessions; a "step" is one restore.  Roofline: HBM, 2 x payload.
  c4_spec_verify          16 sessions on that prefix; a "step" is one speculative round for all sessions: append
                          7 rows + causal verify attention over them on every layer, then truncate to 1 + accepted
                          rows (accepted ~ geometric(0.7) capped at 6).  Roofline: HBM, the K/V the block sees.

  c4_chunked_prefill      that model's prompt ingestion: 4 sessions x 2048 tokens, every layer fed in chunks of 512 rows
                          (one multi-row call per layer and chunk: the chunk's rows are appended and attended
                          causally).  Metric: prompt tokens/s.  Roofline: the tensor pipe (useful flops = 4 x rows x
                          heads x visible keys x head dim against the measured dense bf16 rate).

Every line carries `roofline` (the dominant kernel's algorithmic bytes over its CUDA-event time against the measured
HBM peak), `e2e` (the same work driven from host buffers through the C ABI) and `cpu_baseline` (the CPU restatement
of the reference on the same shape, a bounded sample).  Inputs are seeded synthetic N(0,1) tensors.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
LAYERS, HQ, HKV, D, PREFIX, SESSIONS, ROWS = 32, 32, 8, 128, 2048, 16, 7


def _peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (earlier measurement on this pool)"


def _tensor_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["bf16_tflops_sustained"]), "measured (MEASURED_PEAKS.json bf16_tflops_sustained)"
    return 1400.0, "fallback (earlier measurement on this pool)"


def _options(args):
    out = {}
    for item in getattr(args, "option", []) or []:
        name, _, value = item.partition("=")
        out[name] = int(value)
    return out


def _device():
    import torch

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    gen = torch.Generator(device=dev)
    return torch, dev, stream, gen


def _threads_run(fn, items, threads):
    """Run fn(item) over `items` on `threads` host threads (the oracle's C calls release the GIL); wall seconds."""
    lock = threading.Lock()
    todo = list(items)

    def work():
        while True:
            with lock:
                if not todo:
                    return
                it = todo.pop()
            fn(it)

    ts = [threading.Thread(target=work) for _ in range(max(threads, 1))]
    t0 = time.perf_counter()
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    return time.perf_counter() - t0


def _oracle_cache(hkv, d, rows, seed=0):
    import numpy as np

    from oracle import oracle as orc

    rng = np.random.default_rng(seed)
    cache = orc.KvCache([orc.GLOBAL], hkv, d)
    for at in range(0, rows, 4096):
        n = min(4096, rows - at)
        cache.append_rows(0, rng.standard_normal((n, hkv * d), dtype=np.float32),
                          rng.standard_normal((n, hkv * d), dtype=np.float32), at)
    return cache


# ---------------------------------------------------------------------------------------------------------
# config 4: prefix snapshot restore
# ---------------------------------------------------------------------------------------------------------
def _setup_prefix(args, rounds):
    from itak_torch_rebuild_b200 import CudaCompute, KvDtype

    torch, dev, stream, gen = _device()
    layers = getattr(args, "layers", None) or LAYERS
    be = CudaCompute(layers, HQ, HKV, D, n_slots=SESSIONS + 1, max_context=PREFIX + rounds * ROWS + 16, chunk_cap=ROWS,
                     kv_dtype=KvDtype.F16, device=0, options=_options(args))
    be.set_stream(stream.cuda_stream)
    gen.manual_seed(99)
    kb = torch.empty((1, PREFIX, HKV * D), device=dev)
    vb = torch.empty_like(kb)
    for layer in range(layers):
        kb.normal_(generator=gen)
        vb.normal_(generator=gen)
        be.append_rows_device(layer, [SESSIONS], [0], PREFIX, kb.data_ptr(), vb.data_ptr())
    torch.cuda.synchronize()
    return torch, dev, be, stream, gen, layers


def run_prefix_restore(args, sampler_cls, short=False):
    import numpy as np

    from oracle import oracle as orc

    steps = 32 if short else max(args.steps, 16)
    warm = max(args.warmup, 3)
    torch, dev, be, stream, gen, layers = _setup_prefix(args, 1)
    snap = be.capture_prefix_snapshot(slot=SESSIONS)
    payload = snap.payload_bytes
    for w in range(warm):
        be.install_prefix_snapshot(snap, slot=w % SESSIONS)
    torch.cuda.synchronize()
    launches0 = be.stats()["kernel_launches"]
    sampler = sampler_cls(0)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for s in range(steps):
        be.install_prefix_snapshot(snap, slot=s % SESSIONS)  # 256 MiB read + 256 MiB written: far larger than L2
    ev1.record(stream)
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = ev0.elapsed_time(ev1) / steps
    launches = be.stats()["kernel_launches"] - launches0
    # the kernel's own duration for the roofline: the same restores once more with an event pair around each launch
    be.profile_enable(steps + 8)
    for s in range(steps):
        be.install_prefix_snapshot(snap, slot=s % SESSIONS)
    prof = be.profile_read()
    be.profile_enable(0)
    # capture (the gather direction), timed the same way
    be.profile_enable(8)
    caps = [be.capture_prefix_snapshot(slot=i) for i in range(4)]
    cprof = be.profile_read()
    be.profile_enable(0)
    del caps
    peak, src = _peak()
    k_ms = prof["copy_ms"] / max(prof["copy_launches"], 1)
    c_ms = cprof["copy_ms"] / max(cprof["copy_launches"], 1)

    # end to end from host memory: the prefix arrives as bytes of the wire format, is decoded (strictly), uploaded
    # and installed into a session
    wire = snap.to_itkv("bench", version=2)
    reps = 2
    t0 = time.perf_counter()
    for r in range(reps):
        up = be.snapshot_from_itkv(wire, "bench")
        be.install_prefix_snapshot(up, slot=r % SESSIONS)
        be.synchronize()
        del up
    e2e_s = (time.perf_counter() - t0) / reps
    e2e = {"value": 1.0 / e2e_s, "unit": "restores/s", "h2d_bytes_per_step": len(wire), "d2h_bytes_per_step": 0,
           "steps": reps, "call": "itk_snapshot_from_itkv (version-2 f16 wire bytes on the host: strict decode, checksum, "
                                  "upload) + itk_snapshot_restore"}
    del wire

    # CPU: the reference's KvSnapshot::restore (f32) of the same prefix geometry
    geo = orc.KvGeometry([orc.GLOBAL] * layers, HKV, D)
    rng = np.random.default_rng(3)
    block = rng.standard_normal(PREFIX * HKV * D, dtype=np.float32)
    cpu_snap = orc.KvSnapshot.build(geo, "bench", PREFIX, [(0, block, block)] * layers)
    t0 = time.perf_counter()
    cpu_reps = 2
    for _ in range(cpu_reps):
        restored = cpu_snap.restore()
        del restored
    cpu_s = (time.perf_counter() - t0) / cpu_reps
    cpu = {"value": 1.0 / cpu_s, "unit": "restores/s", "cores": 1, "kind": "port",
           "sample": f"{cpu_reps} full restores of the same geometry in f32 (the reference's snapshot element type, "
                     f"{2 * payload} bytes), one thread as the reference"}
    del cpu_snap

    line = {
        "metric": "prefix_restores_per_s", "value": 1e3 / ms, "unit": "restores/s", "n_gpus": 1, "steps": steps,
        "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u16 (f16 bit patterns moved as 16-byte vectors)", "data": "synthetic",
        "config": {"workload": "c4_prefix_restore", "layers": layers, "kv_heads": HKV, "head_dim": D,
                   "prefix_tokens": PREFIX, "sessions": SESSIONS, "payload_bytes": payload,
                   "l2": "each restore moves 2 x payload, larger than L2"},
        "roofline": {"bound": "hbm", "achieved": 2 * payload / (k_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": 2 * payload / (k_ms * 1e-3) / 1e9 / peak,
                     # ncu on this launch: 268.6 MB read + 268.5 MB written against 2 x 268.4 MB algorithmic
                     "traffic": 2 * payload * (268.6 + 268.5) / (2 * 268.4), "peak_source": src,
                     "kernel": "snapshot_copy_kernel<16> (restore scatter)", "bytes_per_launch": 2 * payload,
                     "avg_launch_ms": k_ms, "launches_timed": prof["copy_launches"],
                     "capture_gather": {"avg_launch_ms": c_ms, "achieved": 2 * payload / (c_ms * 1e-3) / 1e9,
                                        "frac": 2 * payload / (c_ms * 1e-3) / 1e9 / peak}},
        "e2e": e2e, "cpu_baseline": cpu, "clocks": clocks, "gpu_launches": launches,
    }
    be.close()
    return line


# ---------------------------------------------------------------------------------------------------------
# config 4: speculative verify rounds
# ---------------------------------------------------------------------------------------------------------
def run_spec_verify(args, sampler_cls, short=False):
    import numpy as np

    from oracle import oracle as orc

    steps = 12 if short else args.steps
    warm = max(args.warmup, 3)
    prof_steps = min(steps, 8)
    e2e_steps = 3
    rounds = warm + steps + prof_steps + e2e_steps + 3
    torch, dev, be, stream, gen, layers = _setup_prefix(args, rounds)
    snap = be.capture_prefix_snapshot(slot=SESSIONS)
    slots = list(range(SESSIONS))
    for s in slots:
        be.install_prefix_snapshot(snap, slot=s)
    rng = np.random.default_rng(5)
    pool = 4
    q = torch.randn((pool, layers, SESSIONS, ROWS, HQ * D), device=dev, generator=gen)
    k = torch.randn((pool, layers, SESSIONS, ROWS, HKV * D), device=dev, generator=gen)
    v = torch.randn((pool, layers, SESSIONS, ROWS, HKV * D), device=dev, generator=gen)
    out = torch.empty((layers, SESSIONS, ROWS, HQ * D), device=dev)
    hq_pin = torch.randn((layers, SESSIONS, ROWS, HQ * D)).pin_memory()
    hk_pin = torch.randn((layers, SESSIONS, ROWS, HKV * D)).pin_memory()
    hv_pin = torch.randn((layers, SESSIONS, ROWS, HKV * D)).pin_memory()
    ho_pin = torch.empty((layers, SESSIONS, ROWS, HQ * D)).pin_memory()
    slots_c = (C.c_uint32 * SESSIONS)(*slots)
    pos = [PREFIX] * SESSIONS
    kv_bytes = 0

    def one_round(i, count, host=False):
        nonlocal kv_bytes
        cps = [be.cache_checkpoint(ROWS, slot=s) for s in slots]
        pc = (C.c_uint64 * SESSIONS)(*pos)
        if host:
            be.attention_layers_host_ptrs(slots_c, pc, SESSIONS, ROWS, hq_pin.data_ptr(), hk_pin.data_ptr(),
                                          hv_pin.data_ptr(), ho_pin.data_ptr())
        else:
            for layer in range(layers):
                be.attention_batch_ptrs(layer, slots_c, pc, SESSIONS, ROWS, q[i % pool, layer].data_ptr(),
                                        k[i % pool, layer].data_ptr(), v[i % pool, layer].data_ptr(),
                                        out[layer].data_ptr(), device=True)
        if count:
            kv_bytes += sum((p + ROWS) for p in pos) * HKV * D * 2 * 2 * layers
        acc = np.minimum(rng.geometric(0.3, size=SESSIONS) - 1, ROWS - 1)
        for s in slots:
            pos[s] += 1 + int(acc[s])
            be.cache_rewind(cps[s], pos[s], slot=s)
            be.cache_release(cps[s], slot=s)

    for w in range(warm):
        one_round(w, False)
    torch.cuda.synchronize()
    launches0 = be.stats()["kernel_launches"]
    sampler = sampler_cls(0)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for s in range(steps):
        one_round(warm + s, True)
    ev1.record(stream)
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = ev0.elapsed_time(ev1) / steps
    launches = be.stats()["kernel_launches"] - launches0
    timed_bytes = kv_bytes
    # The kernel's own duration for the roofline: the same rounds once more with a CUDA-event pair around every
    # launch (the pairs sit between consecutive kernels, so they stay out of the timed region above).
    be.profile_enable(prof_steps * layers * 2 + 8)
    for s in range(prof_steps):
        one_round(warm + steps + s, False)
    prof = be.profile_read()
    be.profile_enable(0)
    kv_bytes = timed_bytes
    verify_tc = bool(_options(args).get("verify_tc", 1))

    # end to end from host buffers: one call per round carries every layer's 7 rows per session up and the results down
    one_round(0, False, host=True)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for s in range(e2e_steps):
        one_round(s, False, host=True)
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    e2e = {"value": SESSIONS / e2e_s, "unit": "session-rounds/s",
           "h2d_bytes_per_step": layers * SESSIONS * ROWS * (HQ + 2 * HKV) * D * 4,
           "d2h_bytes_per_step": layers * SESSIONS * ROWS * HQ * D * 4, "steps": e2e_steps,
           "call": "itk_cache_checkpoint, itk_attention_layers_host (pinned host q/k/v/out of all layers), "
                   "itk_cache_rewind, itk_cache_release per round"}

    # CPU: the reference's gqa_attention with 7 query rows over prefix + block, (session, layer) units on all cores
    threads = os.cpu_count() or 1
    n_ctx = int(sum(pos) / SESSIONS)
    cache = _oracle_cache(HKV, D, n_ctx + ROWS)
    qh = np.random.default_rng(9).standard_normal((threads, ROWS * HQ * D), dtype=np.float32)
    view = cache.view(0)
    secs = _threads_run(lambda i: orc.gqa_attention(qh[i], ROWS, HQ, list(range(n_ctx, n_ctx + ROWS)), view),
                        range(threads), threads)
    cpu_round_s = secs / threads * SESSIONS * layers
    cpu = {"value": SESSIONS / cpu_round_s, "unit": "session-rounds/s", "cores": threads, "kind": "port",
           "sample": f"{threads} of {SESSIONS * layers} (session, layer) units of a round at context {n_ctx} + {ROWS} rows "
                     f"(one shared f32 cache), {threads} host threads, extrapolated to a full round"}

    peak, src = _peak()
    a_ms = prof["attention_ms"] / max(prof["attention_launches"], 1)
    bytes_launch = kv_bytes / steps / layers
    flops_launch = 4.0 * ROWS * HQ * D * (kv_bytes / steps / layers) / (HKV * D * 4)
    line = {
        "metric": "speculative_verify_rounds_per_s", "value": SESSIONS * 1e3 / ms, "unit": "session-rounds/s", "n_gpus": 1,
        "steps": steps, "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 math over an f16 KV cache", "data": "synthetic",
        "config": {"workload": "c4_spec_verify", "layers": layers, "q_heads": HQ, "kv_heads": HKV, "head_dim": D,
                   "sessions": SESSIONS, "prefix_tokens": PREFIX, "rows_per_round": ROWS,
                   "mean_context": sum(pos) / SESSIONS, "l2": f"{bytes_launch / 2**20:.0f} MiB of K/V per launch, larger than L2"},
        # the timed region of a round holds nothing but its layers' attention launches, back to back (checkpoint, rewind
        # and release are host metadata): its CUDA-event time over its launches is the launch duration
        "roofline": {"bound": "hbm", "achieved": bytes_launch / (ms / layers * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": bytes_launch / (ms / layers * 1e-3) / 1e9 / peak,
                     # ncu on a 2-layer capture of the same launch shape: 137.8 MB read + 3.3 MB written against
                     # 136.2 MB algorithmic
                     "traffic": bytes_launch * (137.8 + 3.3) / 136.2, "peak_source": src,
                     "kernel": "verify_tc_kernel (tcgen05)" if verify_tc else "verify_f16_kernel<128> (mma.sync)",
                     "bytes_per_launch": bytes_launch, "avg_launch_ms": ms / layers, "launches_timed": steps * layers,
                     "timed_as": "CUDA events around the timed region / attention launches in it (consecutive layers "
                                 "as programmatic dependents)",
                     "event_pair": {"avg_launch_ms": a_ms, "achieved": bytes_launch / (a_ms * 1e-3) / 1e9,
                                    "frac": bytes_launch / (a_ms * 1e-3) / 1e9 / peak,
                                    "launches_timed": prof["attention_launches"],
                                    "note": "the same rounds with a CUDA-event pair around every launch (no dependent-launch "
                                            "overlap between layers, and the pair itself costs a few microseconds)"},
                     "append_avg_launch_ms": prof["append_ms"] / max(prof["append_launches"], 1),
                     "tensor_tflops": flops_launch / (ms / layers * 1e-3) / 1e12, "kv_splits": be.stats()["last_splits"]},
        "e2e": e2e, "cpu_baseline": cpu, "clocks": clocks, "gpu_launches": launches,
    }
    be.close()
    return line


# ---------------------------------------------------------------------------------------------------------
# config 4's model, prompt ingestion: chunked prefill on the multi-row tensor-core kernel
# ---------------------------------------------------------------------------------------------------------
def run_chunked_prefill(args, sampler_cls, short=False):
    import numpy as np

    from itak_torch_rebuild_b200 import CudaCompute, KvDtype
    from oracle import oracle as orc

    layers = getattr(args, "layers", None) or LAYERS
    sessions, prompt, chunk = 4, PREFIX, 512
    chunks = prompt // chunk
    warm = max(args.warmup, 3)
    reps = 3 if short else max(args.steps, 5)
    torch, dev, stream, gen = _device()
    be = CudaCompute(layers, HQ, HKV, D, n_slots=sessions, max_context=prompt + 8, chunk_cap=chunk, kv_dtype=KvDtype.F16,
                     device=0, options=_options(args))
    be.set_stream(stream.cuda_stream)
    gen.manual_seed(17)
    # one chunk's rows per layer, reused for every chunk (the values do not change the work)
    q = torch.randn((layers, sessions, chunk, HQ * D), device=dev, generator=gen)
    k = torch.randn((layers, sessions, chunk, HKV * D), device=dev, generator=gen)
    v = torch.randn((layers, sessions, chunk, HKV * D), device=dev, generator=gen)
    out = torch.empty((layers, sessions, chunk, HQ * D), device=dev)
    slots_c = (C.c_uint32 * sessions)(*range(sessions))

    def ingest(profile=False, n_chunks=chunks):
        """All sessions' prompts, chunk by chunk through every layer; returns (ms, profile)."""
        for s in range(sessions):
            be.reset(s)
        if profile:
            be.profile_enable(chunks * layers * 2 + 8)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for c in range(n_chunks):
            pc = (C.c_uint64 * sessions)(*([c * chunk] * sessions))
            for layer in range(layers):
                be.attention_batch_ptrs(layer, slots_c, pc, sessions, chunk, q[layer].data_ptr(), k[layer].data_ptr(),
                                        v[layer].data_ptr(), out[layer].data_ptr(), device=True)
        e1.record(stream)
        torch.cuda.synchronize()
        prof = None
        if profile:
            prof = be.profile_read()
            be.profile_enable(0)
        return e0.elapsed_time(e1), prof

    for _ in range(warm):
        ingest()
    launches0 = be.stats()["kernel_launches"]
    sampler = sampler_cls(0)
    sampler.start()
    times = sorted(ingest()[0] for _ in range(reps))
    clocks = sampler.stop()
    launches = be.stats()["kernel_launches"] - launches0
    ms = times[len(times) // 2]
    _, prof = ingest(profile=True)
    be.synchronize()  # raises if a bounded wait of the tensor-core kernel ran out

    # end to end from pinned host buffers: the last chunk of every session, all layers in one call
    hq_pin = q.cpu().pin_memory()
    hk_pin, hv_pin = k.cpu().pin_memory(), v.cpu().pin_memory()
    ho_pin = torch.empty_like(hq_pin).pin_memory()

    def host_chunk():
        cps = [be.cache_checkpoint(chunk, slot=s) for s in range(sessions)]
        pc = (C.c_uint64 * sessions)(*([prompt - chunk] * sessions))
        t0 = time.perf_counter()
        be.attention_layers_host_ptrs(slots_c, pc, sessions, chunk, hq_pin.data_ptr(), hk_pin.data_ptr(), hv_pin.data_ptr(),
                                      ho_pin.data_ptr())
        dt = time.perf_counter() - t0
        for s in range(sessions):  # back to the state before the chunk (host metadata only)
            be.cache_rewind(cps[s], prompt - chunk, slot=s)
            be.cache_release(cps[s], slot=s)
        return dt

    ingest(n_chunks=chunks - 1)
    host_chunk()
    e2e_s = sorted(host_chunk() for _ in range(3))[1]
    e2e = {"value": sessions * chunk / e2e_s, "unit": "tokens/s",
           "h2d_bytes_per_step": layers * sessions * chunk * (HQ + 2 * HKV) * D * 4,
           "d2h_bytes_per_step": layers * sessions * chunk * HQ * D * 4, "steps": 3,
           "call": "itk_attention_layers_host on the prompt's last 512-row chunk of every session (pinned host "
                   "q/k/v/out of all layers, uploads / kernels / downloads of consecutive layers overlapped)"}

    # CPU: the reference's gqa_attention on sampled rows of one (session, layer) prefill, all cores
    threads = os.cpu_count() or 1
    rows_sample = [int(x) for x in np.linspace(0, prompt - 1, threads)]
    qh = np.random.default_rng(9).standard_normal((threads, HQ * D), dtype=np.float32)
    views = [_oracle_cache(HKV, D, r + 1, seed=r).view(0) for r in rows_sample]  # row r attends its causal prefix
    secs = _threads_run(lambda i: orc.gqa_attention(qh[i], 1, HQ, [rows_sample[i]], views[i]), range(threads), threads)
    # rows sampled evenly over the causal triangle: their mean cost is the mean row's
    cpu_s = secs / threads * prompt * sessions * layers
    cpu = {"value": sessions * prompt / cpu_s, "unit": "tokens/s", "cores": threads, "kind": "port",
           "sample": f"{threads} rows spread evenly over one (session, layer) prompt of {prompt} tokens (each attends its "
                     f"causal prefix in an f32 cache), {threads} host threads, extrapolated to {sessions} sessions x {layers} layers"}

    tpeak, tsrc = _tensor_peak()
    peak, _ = _peak()
    flops = 4.0 * HQ * D * (prompt * (prompt + 1) / 2) * sessions * layers
    n_launch = chunks * layers
    a_ms = prof["attention_ms"] / max(prof["attention_launches"], 1)
    kv_bytes = sum((c + 1) * chunk for c in range(chunks)) * sessions * HKV * D * 2 * 2 * layers
    verify_tc = bool(_options(args).get("verify_tc", 1))
    line = {
        "metric": "prefill_tokens_per_s", "value": sessions * prompt * 1e3 / ms, "unit": "tokens/s", "n_gpus": 1,
        "steps": reps, "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 math over an f16 KV cache (queries and weights as two f16 terms)", "data": "synthetic",
        "config": {"workload": "c4_chunked_prefill", "layers": layers, "q_heads": HQ, "kv_heads": HKV, "head_dim": D,
                   "sessions": sessions, "prompt_tokens": prompt, "chunk_rows": chunk,
                   "launch": "one multi-row call per layer and chunk: the append kernel stores the chunk's rows, then the "
                             "attention kernel attends them causally (two launches; a block of up to 64 rows is stored by "
                             "the attention kernel itself)",
                   "l2": f"{kv_bytes / n_launch / 2**20:.0f} MiB of K/V per launch on average: L2-resident, the launch is "
                         "bound by the tensor pipe, not by HBM"},
        "roofline": {"bound": "tensor", "achieved": flops / (ms * 1e-3) / 1e12, "peak": tpeak, "unit": "TFLOP/s",
                     "frac": flops / (ms * 1e-3) / 1e12 / tpeak, "traffic": None, "peak_source": tsrc,
                     "kernel": "verify_tc_kernel (tcgen05)" if verify_tc else "verify_f16_kernel<128> (mma.sync)",
                     "flops_per_launch": flops / n_launch, "avg_launch_ms": ms / n_launch, "launches_timed": reps * n_launch,
                     "useful_flops": "4 x rows x heads x visible keys x head dim; the kernel executes twice that on a full "
                                     "block (every query row and weight row as a hi and a lo f16 term)",
                     "event_pair": {"avg_launch_ms": a_ms, "launches_timed": prof["attention_launches"]},
                     "kv_read_gbs": kv_bytes / (ms * 1e-3) / 1e9, "kv_read_frac_of_hbm_peak": kv_bytes / (ms * 1e-3) / 1e9 / peak},
        "e2e": e2e, "cpu_baseline": cpu, "clocks": clocks, "gpu_launches": launches,
    }
    be.close()
    return line


# ---------------------------------------------------------------------------------------------------------
# config 3: continuous batching over ragged slots with retire / refill
# ---------------------------------------------------------------------------------------------------------
def run_continuous_batching(args, sampler_cls, short=False):
    import numpy as np

    from itak_torch_rebuild_b200 import CudaCompute, KvDtype
    from oracle import oracle as orc

    layers, hq, hkv, d, n_slots, lo, hi = getattr(args, "layers", None) or 32, 32, 8, 128, 16, 256, 8192
    steps = 64 if short else max(args.steps, 64)
    warm = max(args.warmup, 3)
    prof_steps, e2e_steps = 4, 4
    total = warm + steps + prof_steps + e2e_steps + 2
    torch, dev, stream, gen = _device()
    be = CudaCompute(layers, hq, hkv, d, n_slots=n_slots, max_context=hi + total + 8, chunk_cap=1, kv_dtype=KvDtype.F16,
                     device=0, options=_options(args))
    be.set_stream(stream.cuda_stream)
    gen.manual_seed(31)
    rng = np.random.default_rng(0)
    # prompts come from one device pool of seeded rows (a refill's K/V is the prefill's output, which lives on the device)
    pool_k = torch.randn((hi, hkv * d), device=dev, generator=gen)
    pool_v = torch.randn((hi, hkv * d), device=dev, generator=gen)
    pos = [int(x) for x in rng.integers(lo, hi + 1, size=n_slots)]
    for s in range(n_slots):
        for layer in range(layers):
            be.append_rows_device(layer, [s], [0], pos[s], pool_k.data_ptr(), pool_v.data_ptr())
    torch.cuda.synchronize()
    npool = 4
    q = torch.randn((npool, layers, n_slots, hq * d), device=dev, generator=gen)
    k = torch.randn((npool, layers, n_slots, hkv * d), device=dev, generator=gen)
    v = torch.randn((npool, layers, n_slots, hkv * d), device=dev, generator=gen)
    out = torch.empty((layers, n_slots, hq * d), device=dev)
    hq_pin = torch.randn((layers, n_slots, hq * d)).pin_memory()
    hk_pin = torch.randn((layers, n_slots, hkv * d)).pin_memory()
    hv_pin = torch.randn((layers, n_slots, hkv * d)).pin_memory()
    ho_pin = torch.empty((layers, n_slots, hq * d)).pin_memory()
    slots_c = (C.c_uint32 * n_slots)(*range(n_slots))
    state = {"step": 0, "kv_bytes": 0, "refills": 0, "refill_rows": 0}

    loop = {"steps": 0, "active": False}

    def leave_loop():
        if loop["active"]:
            be.resident_end(loop["steps"])
            loop["active"], loop["steps"] = False, 0

    def one_step(count, host=False, direct=False):
        s = state["step"]
        for i in range(n_slots):  # slot i retires on its own 64-step period, staggered by 4 steps
            if s % 64 == (4 * i) % 64 and s > 0:
                leave_loop()  # a refill changes a slot's position: the replayable loop is re-begun behind it
                be.reset(i)
                pos[i] = int(rng.integers(lo, hi + 1))
                for layer in range(layers):
                    be.append_rows_device(layer, [i], [0], pos[i], pool_k.data_ptr(), pool_v.data_ptr())
                if count:
                    state["refills"] += 1
                    state["refill_rows"] += pos[i]
        pc = (C.c_uint64 * n_slots)(*pos)
        j = s % npool
        if host:
            leave_loop()
            be.attention_layers_host_ptrs(slots_c, pc, n_slots, 1, hq_pin.data_ptr(), hk_pin.data_ptr(), hv_pin.data_ptr(),
                                          ho_pin.data_ptr())
        elif direct:
            leave_loop()
            for layer in range(layers):
                be.attention_batch_ptrs(layer, slots_c, pc, n_slots, 1, q[j, layer].data_ptr(), k[j, layer].data_ptr(),
                                        v[j, layer].data_ptr(), out[layer].data_ptr(), device=True)
        else:
            # the replayable loop's launches (device-side positions, consecutive layers as programmatic dependents),
            # launched directly; the loop is re-begun whenever a refill has moved a slot
            if not loop["active"] or loop["steps"] == 4:
                leave_loop()
                be.resident_begin(list(range(n_slots)), 4)
                loop["active"] = True
            for layer in range(layers):
                be.resident_layer(layer, q[j, layer].data_ptr(), k[j, layer].data_ptr(), v[j, layer].data_ptr(),
                                  out[layer].data_ptr())
            be.resident_advance()
            loop["steps"] += 1
        if count:
            state["kv_bytes"] += sum(p + 1 for p in pos) * hkv * d * 2 * 2 * layers
        for i in range(n_slots):
            pos[i] += 1
        state["step"] = s + 1

    for _ in range(warm):
        one_step(False)
    torch.cuda.synchronize()
    launches0 = be.stats()["kernel_launches"]
    sampler = sampler_cls(0)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(steps):
        one_step(True)
    leave_loop()
    ev1.record(stream)
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = ev0.elapsed_time(ev1) / steps
    launches = be.stats()["kernel_launches"] - launches0
    timed_bytes, refills, refill_rows = state["kv_bytes"], state["refills"], state["refill_rows"]
    # the decode kernel's own duration: a few more steps with an event pair around every launch
    state["kv_bytes"] = 0
    be.profile_enable(prof_steps * layers * 40 + 8)
    for _ in range(prof_steps):
        one_step(True, direct=True)
    prof = be.profile_read()
    be.profile_enable(0)
    prof_bytes = state["kv_bytes"]

    one_step(False, host=True)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(e2e_steps - 1):
        one_step(False, host=True)
    e2e_s = (time.perf_counter() - t0) / (e2e_steps - 1)
    e2e = {"value": 1.0 / e2e_s, "unit": "steps/s", "h2d_bytes_per_step": layers * n_slots * (hq + 2 * hkv) * d * 4,
           "d2h_bytes_per_step": layers * n_slots * hq * d * 4, "steps": e2e_steps - 1,
           "call": "itk_attention_layers_host per step (pinned host q/k/v/out of all layers); refills stay on the device"}

    # CPU: one shared f32 cache of 8192 rows; a unit is one (slot, layer) attention at that slot's context
    threads = os.cpu_count() or 1
    cache = _oracle_cache(hkv, d, hi)
    ctxs = [int(x) for x in np.random.default_rng(0).integers(lo, hi + 1, size=n_slots)]
    qh = np.random.default_rng(2).standard_normal((n_slots, hq * d), dtype=np.float32)
    _, secs = orc.attention_units([cache] * n_slots, [0] * n_slots, qh, [c - 1 for c in ctxs], hq, threads)
    cpu_step_s = secs * layers
    cpu = {"value": 1.0 / cpu_step_s, "unit": "steps/s", "cores": threads, "kind": "port",
           "sample": f"one layer's {n_slots} (slot, layer) units at the seeded ragged contexts (one shared f32 cache), "
                     f"{threads} host threads, times {layers} layers; refills not included"}

    peak, src = _peak()
    a_ms = prof["attention_ms"] / max(prof["attention_launches"], 1)
    bytes_launch = prof_bytes / max(prof["attention_launches"], 1)
    line = {
        "metric": "continuous_batching_steps_per_s", "value": 1e3 / ms, "unit": "steps/s", "n_gpus": 1, "steps": steps,
        "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 math over an f16 KV cache", "data": "synthetic",
        "config": {"workload": "c3_continuous_batching", "layers": layers, "q_heads": hq, "kv_heads": hkv, "head_dim": d,
                   "slots": n_slots, "context_range": [lo, hi], "mean_context_at_end": sum(pos) / n_slots,
                   "refills_in_timed_region": refills, "refill_rows": refill_rows,
                   "launch": "the replayable loop's launches issued directly (consecutive layers as programmatic dependents), "
                             "re-begun behind every refill (a refill changes a slot's position)",
                   "l2": f"{timed_bytes / steps / layers / 2**20:.0f} MiB of K/V per launch, larger than L2"},
        "kv_read_gbs": timed_bytes / steps / (ms * 1e-3) / 1e9,
        "roofline": {"bound": "hbm", "achieved": bytes_launch / (a_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": bytes_launch / (a_ms * 1e-3) / 1e9 / peak, "traffic": bytes_launch * (269.24 + 4.3) / 268.60,
                     "peak_source": src, "kernel": "decode_f16_kernel<128,3> (equal-run plan over ragged cells; timed as ordinary direct launches)",
                     "bytes_per_launch": bytes_launch, "avg_launch_ms": a_ms, "launches_timed": prof["attention_launches"],
                     "whole_step_frac": timed_bytes / steps / (ms * 1e-3) / 1e9 / peak,
                     "append_avg_launch_ms": prof["append_ms"] / max(prof["append_launches"], 1)},
        "e2e": e2e, "cpu_baseline": cpu, "clocks": clocks, "gpu_launches": launches,
    }
    be.close()
    return line


# ---------------------------------------------------------------------------------------------------------
# config 1: the reference's own CPU-runnable case (f32 cache, head dim 64): prefill 512, then 64 decode steps
# ---------------------------------------------------------------------------------------------------------
def run_tinyllama_f32(args, sampler_cls, short=False):
    import numpy as np

    from itak_torch_rebuild_b200 import CudaCompute, KvDtype
    from oracle import oracle as orc

    layers, hq, hkv, d, prefill, decode = getattr(args, "layers", None) or 22, 32, 4, 64, 512, 64
    warm = max(args.warmup, 3)
    torch, dev, stream, gen = _device()
    be = CudaCompute(layers, hq, hkv, d, n_slots=2, max_context=prefill + decode + 8, chunk_cap=prefill,
                     kv_dtype=KvDtype.F32, device=0, options=_options(args))
    be.set_stream(stream.cuda_stream)
    gen.manual_seed(0)
    pq = torch.randn((layers, 1, prefill, hq * d), device=dev, generator=gen)
    pk = torch.randn((layers, 1, prefill, hkv * d), device=dev, generator=gen)
    pv = torch.randn((layers, 1, prefill, hkv * d), device=dev, generator=gen)
    pout = torch.empty((layers, 1, prefill, hq * d), device=dev)
    dq = torch.randn((decode, layers, 1, hq * d), device=dev, generator=gen)
    dk = torch.randn((decode, layers, 1, hkv * d), device=dev, generator=gen)
    dv = torch.randn((decode, layers, 1, hkv * d), device=dev, generator=gen)
    dout = torch.empty((layers, 1, hq * d), device=dev)
    one = (C.c_uint32 * 1)(0)

    def run(slot_arr, profile=False):
        """Prefill + decode once from a fresh slot; returns (prefill ms, decode ms, profile of the decode steps)."""
        be.reset(slot_arr[0])
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record(stream)
        p0 = (C.c_uint64 * 1)(0)
        for layer in range(layers):
            be.attention_batch_ptrs(layer, slot_arr, p0, 1, prefill, pq[layer].data_ptr(), pk[layer].data_ptr(),
                                    pv[layer].data_ptr(), pout[layer].data_ptr(), device=True)
        e1.record(stream)
        if profile:
            be.profile_enable(decode * layers * 2 + 8)
        for s in range(decode):
            pc = (C.c_uint64 * 1)(prefill + s)
            for layer in range(layers):
                be.attention_batch_ptrs(layer, slot_arr, pc, 1, 1, dq[s, layer].data_ptr(), dk[s, layer].data_ptr(),
                                        dv[s, layer].data_ptr(), dout[layer].data_ptr(), device=True)
        e2.record(stream)
        torch.cuda.synchronize()
        prof = None
        if profile:
            prof = be.profile_read()
            be.profile_enable(0)
        return e0.elapsed_time(e1), e1.elapsed_time(e2), prof

    for _ in range(warm):
        run(one)
    launches0 = be.stats()["kernel_launches"]
    sampler = sampler_cls(0)
    sampler.start()
    reps = 5 if short else max(args.steps, 5)
    runs = [run(one) for _ in range(reps)]
    clocks = sampler.stop()
    launches = be.stats()["kernel_launches"] - launches0
    pre_ms = sorted(r[0] for r in runs)[len(runs) // 2]
    dec_ms = sorted(r[1] for r in runs)[len(runs) // 2]
    _, _, prof = run(one, profile=True)

    # end to end from host buffers: the prefill as one call for all layers, then one call per decode step
    hpq, hpk, hpv = pq.cpu().pin_memory(), pk.cpu().pin_memory(), pv.cpu().pin_memory()
    hpo = torch.empty_like(hpq).pin_memory()
    hdq, hdk, hdv = dq.cpu().pin_memory(), dk.cpu().pin_memory(), dv.cpu().pin_memory()
    hdo = torch.empty((layers, 1, hq * d)).pin_memory()

    def host_run():
        be.reset(0)
        t0 = time.perf_counter()
        be.attention_layers_host_ptrs(one, (C.c_uint64 * 1)(0), 1, prefill, hpq.data_ptr(), hpk.data_ptr(), hpv.data_ptr(),
                                      hpo.data_ptr())
        t1 = time.perf_counter()
        for s in range(decode):
            be.attention_layers_host_ptrs(one, (C.c_uint64 * 1)(prefill + s), 1, 1, hdq[s].data_ptr(), hdk[s].data_ptr(),
                                          hdv[s].data_ptr(), hdo.data_ptr())
        return t1 - t0, time.perf_counter() - t1

    host_run()
    h_pre, h_dec = host_run()
    e2e = {"value": decode / h_dec, "unit": "steps/s", "h2d_bytes_per_step": layers * (hq + 2 * hkv) * d * 4,
           "d2h_bytes_per_step": layers * hq * d * 4, "steps": decode, "prefill_ms": h_pre * 1e3,
           "call": "itk_attention_layers_host: one call for the 512-row prefill, then one per decode step (pinned host buffers)"}

    # CPU: the reference's own configuration, run whole on one thread (its slot model): prefill rows then decode steps
    rng = np.random.default_rng(0)
    cpu_layers = 2 if short else layers
    cache = orc.KvCache([orc.GLOBAL] * cpu_layers, hkv, d)
    t0 = time.perf_counter()
    for layer in range(cpu_layers):
        cache.append_rows(layer, rng.standard_normal((prefill, hkv * d), dtype=np.float32),
                          rng.standard_normal((prefill, hkv * d), dtype=np.float32), 0)
        orc.gqa_attention(rng.standard_normal(prefill * hq * d, dtype=np.float32), prefill, hq, list(range(prefill)),
                          cache.view(layer))
    cpu_pre = (time.perf_counter() - t0) * layers / cpu_layers
    t0 = time.perf_counter()
    for s in range(decode):
        for layer in range(cpu_layers):
            cache.append(layer, rng.standard_normal(hkv * d, dtype=np.float32), rng.standard_normal(hkv * d, dtype=np.float32),
                         prefill + s)
            orc.gqa_attention(rng.standard_normal(hq * d, dtype=np.float32), 1, hq, [prefill + s], cache.view(layer))
    cpu_dec = (time.perf_counter() - t0) * layers / cpu_layers
    cpu = {"value": decode / cpu_dec, "unit": "steps/s", "cores": 1, "kind": "port", "prefill_ms": cpu_pre * 1e3,
           "sample": f"{cpu_layers} of {layers} layers, the whole prefill and all {decode} decode steps, one thread "
                     f"(the reference runs one thread per sequence), scaled to {layers} layers"}

    peak, src = _peak()
    tpeak, tsrc = _tensor_peak()
    a_ms = prof["attention_ms"] / max(prof["attention_launches"], 1)
    mean_ctx = prefill + (decode + 1) / 2
    bytes_launch = mean_ctx * hkv * d * 2 * 4
    pre_flops = 4.0 * hq * d * (prefill * (prefill + 1) / 2) * layers
    line = {
        "metric": "decode_attention_steps_per_s", "value": decode * 1e3 / dec_ms, "unit": "steps/s", "n_gpus": 1,
        "steps": decode, "warmup": warm, "ms_per_step": dec_ms / decode, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "c1_tinyllama_f32", "layers": layers, "q_heads": hq, "kv_heads": hkv, "head_dim": d,
                   "sequences": 1, "prefill_rows": prefill, "decode_steps": decode, "kv_dtype": "f32", "repeats": reps,
                   "launch": "direct launches, one per layer (the attention kernel stores the new rows itself)",
                   "l2": f"{bytes_launch / 2**20:.2f} MiB of K/V per launch: the whole cache ({layers} layers) fits in L2, "
                         "so this case is launch-latency-bound, not HBM-bound"},
        "prefill": {"ms": pre_ms, "rows": prefill, "tflops": pre_flops / (pre_ms * 1e-3) / 1e12,
                    "frac_of_tensor_peak": pre_flops / (pre_ms * 1e-3) / 1e12 / tpeak, "tensor_peak": tpeak,
                    "tensor_peak_source": tsrc,
                    "kernel": "attn_f32_kernel<64, 1, fold> (mma.sync tf32, three terms per product: a third of the "
                              "executed tensor work is useful)"},
        "roofline": {"bound": "hbm", "achieved": bytes_launch / (a_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": bytes_launch / (a_ms * 1e-3) / 1e9 / peak, "traffic": None, "peak_source": src,
                     "kernel": "attn_f32_kernel<64, 4>", "bytes_per_launch": bytes_launch, "avg_launch_ms": a_ms,
                     "launches_timed": prof["attention_launches"],
                     "append_avg_launch_ms": prof["append_ms"] / max(prof["append_launches"], 1)},
        "e2e": e2e, "cpu_baseline": cpu, "clocks": clocks, "gpu_launches": launches,
    }
    be.close()
    return line


RUNNERS = {
    "c1_tinyllama_f32": run_tinyllama_f32,
    "c3_continuous_batching": run_continuous_batching,
    "c4_prefix_restore": run_prefix_restore,
    "c4_spec_verify": run_spec_verify,
    "c4_chunked_prefill": run_chunked_prefill,
}
