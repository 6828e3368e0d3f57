"""Measurement of the hot path's other rows on one B200, in the JSON shape of bench.py (which dispatches here for
`--workload c4_prefix_restore` and `--workload c4_spec_verify`):

  c4_prefix_restore  a 2048-token shared prefix (32 layers, 8 KV heads, head dim 128, f16 = 256 MiB) captured once
                     and restored into 16 sessions; a "step" is one restore.  Roofline: HBM, 2 x payload per restore.
  c4_spec_verify     16 sessions on that prefix; a "step" is one speculative round for all sessions: append 7 rows +
                     causal verify attention over them on every layer, then truncate to 1 + accepted rows
                     (accepted ~ geometric(0.7) capped at 6).  Roofline: HBM, the K/V the block sees.
Inputs are seeded synthetic N(0,1) tensors generated on the device.
"""
from __future__ import annotations

import ctypes as C
import json
import os

ROOT = os.path.dirname(os.path.abspath(__file__))
LAYERS, HQ, HKV, D, PREFIX, SESSIONS, ROWS = 32, 32, 8, 128, 2048, 16, 7


def _peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (earlier measurement on this pool)"


def _setup(args, rounds):
    import torch

    from itak_torch_rebuild_b200 import CudaCompute, KvDtype

    layers = args.layers or LAYERS
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    be = CudaCompute(layers, HQ, HKV, D, n_slots=SESSIONS + 1, max_context=PREFIX + rounds * ROWS + 16, chunk_cap=ROWS,
                     kv_dtype=KvDtype.F16, device=0)
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    be.set_stream(stream.cuda_stream)
    gen = torch.Generator(device=dev)
    gen.manual_seed(99)
    kb = torch.empty((1, PREFIX, HKV * D), device=dev)
    vb = torch.empty_like(kb)
    for layer in range(layers):
        kb.normal_(generator=gen)
        vb.normal_(generator=gen)
        be.append_rows_device(layer, [SESSIONS], [0], PREFIX, kb.data_ptr(), vb.data_ptr())
    torch.cuda.synchronize()
    return torch, dev, be, stream, gen, layers


def run_prefix_restore(args, sampler_cls):
    torch, dev, be, stream, gen, layers = _setup(args, 1)
    snap = be.capture_prefix_snapshot(slot=SESSIONS)
    payload = snap.payload_bytes
    for w in range(max(args.warmup, 3)):
        be.install_prefix_snapshot(snap, slot=w % SESSIONS)
    torch.cuda.synchronize()
    launches0 = be.stats()["kernel_launches"]
    sampler = sampler_cls(0)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for s in range(args.steps):
        be.install_prefix_snapshot(snap, slot=s % SESSIONS)  # 256 MiB read + 256 MiB written: far larger than L2
    ev1.record(stream)
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = ev0.elapsed_time(ev1) / args.steps
    launches = be.stats()["kernel_launches"] - launches0
    # the kernel's own duration for the roofline: the same restores once more with an event pair around each launch
    be.profile_enable(args.steps + 8)
    for s in range(args.steps):
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
    line = {
        "metric": "prefix_restores_per_s", "value": 1e3 / ms, "unit": "restores/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u16 (f16 bit patterns moved as 16-byte vectors)", "data": "synthetic",
        "config": {"workload": "c4_prefix_restore", "layers": layers, "kv_heads": HKV, "head_dim": D,
                   "prefix_tokens": PREFIX, "sessions": SESSIONS, "payload_bytes": payload,
                   "l2": "each restore moves 2 x payload, larger than L2"},
        "roofline": {"bound": "hbm", "achieved": 2 * payload / (k_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": 2 * payload / (k_ms * 1e-3) / 1e9 / peak, "traffic": None, "peak_source": src,
                     "kernel": "snapshot_copy_kernel<16> (restore scatter)", "bytes_per_launch": 2 * payload,
                     "avg_launch_ms": k_ms, "launches_timed": prof["copy_launches"],
                     "capture_gather": {"avg_launch_ms": c_ms, "achieved": 2 * payload / (c_ms * 1e-3) / 1e9,
                                        "frac": 2 * payload / (c_ms * 1e-3) / 1e9 / peak}},
        "e2e": None, "cpu_baseline": None, "clocks": clocks, "gpu_launches": launches,
    }
    print(json.dumps(line), flush=True)
    be.close()


def run_spec_verify(args, sampler_cls):
    import numpy as np

    prof_steps = min(args.steps, 8)
    rounds = max(args.warmup, 3) + args.steps + prof_steps + 2
    torch, dev, be, stream, gen, layers = _setup(args, rounds)
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
    slots_c = (C.c_uint32 * SESSIONS)(*slots)
    pos = [PREFIX] * SESSIONS
    kv_bytes = 0

    def one_round(i, count):
        nonlocal kv_bytes
        cps = [be.cache_checkpoint(ROWS, slot=s) for s in slots]
        pc = (C.c_uint64 * SESSIONS)(*pos)
        for layer in range(layers):
            be.attention_batch_ptrs(layer, slots_c, pc, SESSIONS, ROWS, q[i % pool, layer].data_ptr(),
                                    k[i % pool, layer].data_ptr(), v[i % pool, layer].data_ptr(), out[layer].data_ptr(),
                                    device=True)
        if count:
            kv_bytes += sum((p + ROWS) for p in pos) * HKV * D * 2 * 2 * layers
        acc = np.minimum(rng.geometric(0.3, size=SESSIONS) - 1, ROWS - 1)
        for s in slots:
            pos[s] += 1 + int(acc[s])
            be.cache_rewind(cps[s], pos[s], slot=s)
            be.cache_release(cps[s], slot=s)

    for w in range(max(args.warmup, 3)):
        one_round(w, False)
    torch.cuda.synchronize()
    launches0 = be.stats()["kernel_launches"]
    sampler = sampler_cls(0)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for s in range(args.steps):
        one_round(args.warmup + s, True)
    ev1.record(stream)
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = ev0.elapsed_time(ev1) / args.steps
    launches = be.stats()["kernel_launches"] - launches0
    timed_bytes = kv_bytes
    # The kernel's own duration for the roofline: the same rounds once more with a CUDA-event pair around every
    # launch (the pairs sit between consecutive kernels, so they stay out of the timed region above).
    be.profile_enable(prof_steps * layers * 2 + 8)
    for s in range(prof_steps):
        one_round(args.warmup + args.steps + s, False)
    prof = be.profile_read()
    be.profile_enable(0)
    kv_bytes = timed_bytes
    peak, src = _peak()
    a_ms = prof["attention_ms"] / max(prof["attention_launches"], 1)
    bytes_launch = kv_bytes / args.steps / layers
    flops_launch = 4.0 * ROWS * HQ * D * (kv_bytes / args.steps / layers) / (HKV * D * 4)
    line = {
        "metric": "speculative_verify_rounds_per_s", "value": SESSIONS * 1e3 / ms, "unit": "session-rounds/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 math over an f16 KV cache", "data": "synthetic",
        "config": {"workload": "c4_spec_verify", "layers": layers, "q_heads": HQ, "kv_heads": HKV, "head_dim": D,
                   "sessions": SESSIONS, "prefix_tokens": PREFIX, "rows_per_round": ROWS,
                   "mean_context": sum(pos) / SESSIONS, "l2": f"{bytes_launch / 2**20:.0f} MiB of K/V per launch, larger than L2"},
        "roofline": {"bound": "hbm", "achieved": bytes_launch / (a_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": bytes_launch / (a_ms * 1e-3) / 1e9 / peak,
                     # ncu on a 2-layer capture of the same launch shape: 137.6 MB read + 5.3 MB written against
                     # 136.2 MB algorithmic (profiles/verify_tc_kernel_c4_small.md)
                     "traffic": bytes_launch * (137.6 + 5.3) / 136.2, "peak_source": src,
                     "kernel": ("verify_tc_kernel<32> (tcgen05)" if os.environ.get("ITK_VERIFY_TC", "1") != "0"
                                else "verify_f16_kernel<128> (mma.sync)"),
                     "bytes_per_launch": bytes_launch, "avg_launch_ms": a_ms,
                     "launches_timed": prof["attention_launches"],
                     "append_avg_launch_ms": prof["append_ms"] / max(prof["append_launches"], 1),
                     "tensor_tflops": flops_launch / (a_ms * 1e-3) / 1e12, "kv_splits": be.stats()["last_splits"]},
        "e2e": None, "cpu_baseline": None, "clocks": clocks, "gpu_launches": launches,
    }
    print(json.dumps(line), flush=True)
    be.close()
