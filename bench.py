"""Decode-attention throughput of the KV-cache hot path on N B200s (one process per GPU).

Workload (default): the long-context decode configuration - 48 layers, 64 query heads, 8 KV heads,
head dim 128, f16 KV cache, 8 resident sequences at 32768 tokens of context.  One "step" is one decode
step of the hot path: for every layer, append one RoPE'd K/V row per sequence and run GQA attention over
the whole resident cache.  At N > 1 the KV heads are sharded (8 / N per GPU, strong scaling) and each
layer ends with one all-gather of the per-head outputs over NCCL.

Prints ONE JSON line: decode steps/s (whole job), with
  roofline      - the attention kernel's algorithmic KV bytes / its CUDA-event time vs the measured HBM peak,
  e2e           - the same step through the host-buffer C-ABI call (H2D + kernels + D2H inside the timed region),
  cpu_baseline  - the CPU restatement of the reference's attention timed on this box's cores (bounded sample),
  clocks        - SM clocks and throttle reasons sampled during the timed region.
`--impl reference` times only the CPU restatement (the reference's own CPU path cannot be built here: it is Rust).
Inputs are seeded synthetic N(0,1) tensors of the configuration's shapes, generated on the device.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (layers, q_heads, kv_heads, head_dim, sequences, context)
    "c5_long_context_decode": (48, 64, 8, 128, 8, 32768),
    "c2_single_sequence_decode": (32, 32, 8, 128, 1, 4096),
}
METRIC = "decode_attention_steps_per_s"
UNIT = "steps/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c5_long_context_decode",
                    choices=sorted(WORKLOADS) + ["c4_prefix_restore", "c4_spec_verify"])
    ap.add_argument("--context", type=int, default=None, help="override the context length (smoke runs)")
    ap.add_argument("--layers", type=int, default=None, help="override the layer count (smoke runs)")
    ap.add_argument("--q-heads", type=int, default=None, help="override the query head count (shard studies)")
    ap.add_argument("--kv-heads", type=int, default=None, help="override the KV head count (shard studies)")
    ap.add_argument("--sequences", type=int, default=None, help="override the number of resident sequences")
    ap.add_argument("--no-graph", action="store_true", help="launch every layer directly instead of replaying a CUDA graph")
    ap.add_argument("--nccl-gather", action="store_true",
                    help="N > 1: gather the head outputs with an NCCL all-gather per layer instead of inside the kernel")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-units", type=int, default=None, help="(sequence, layer) units in the CPU sample")
    return ap.parse_args()


def geometry(args):
    layers, hq, hkv, d, seqs, ctx = WORKLOADS[args.workload]
    if args.context:
        ctx = args.context
    if args.layers:
        layers = args.layers
    if args.q_heads:
        hq = args.q_heads
    if args.kv_heads:
        hkv = args.kv_heads
    if args.sequences:
        seqs = args.sequences
    return layers, hq, hkv, d, seqs, ctx


def kv_bytes_per_step(layers, hkv, d, seqs, ctx_first, steps, elem=2):
    """Algorithmic KV-read bytes: visible keys x Hkv x D x 2 (K, V) x element size, summed over
    (sequence, layer), averaged over the timed steps (the context grows by one per step)."""
    total = 0
    for s in range(steps):
        total += (ctx_first + s + 1) * hkv * d * 2 * elem * layers * seqs
    return total / max(steps, 1)


# ---------------------------------------------------------------------------------------------------
# CPU restatement of the reference (the checker, here as the thing timed - the one permitted use)
# ---------------------------------------------------------------------------------------------------
def cpu_cache(hkv, d, ctx, seed=0):
    """One f32 cache of `ctx` seeded rows (a single layer of a single sequence) on the host."""
    import numpy as np

    from oracle import oracle as orc

    rng = np.random.default_rng(seed)
    cache = orc.KvCache([orc.GLOBAL], hkv, d)
    block = 4096
    for at in range(0, ctx, block):
        n = min(block, ctx - at)
        cache.append_rows(0, rng.standard_normal((n, hkv * d), dtype=np.float32),
                          rng.standard_normal((n, hkv * d), dtype=np.float32), at)
    return cache


def cpu_sample(cache, layers, hq, hkv, d, seqs, ctx, threads, units=None, seed=0):
    """Time `units` (sequence, layer) attention units of the configuration on the host cores.

    The cache is shared (read-only) by every unit; each unit has its own query.  Returns (seconds per full
    step, extrapolated from the sample; description of the sample)."""
    import numpy as np

    from oracle import oracle as orc

    if units is None:
        units = max(threads, 1)
    rng = np.random.default_rng(seed + 1)
    q = rng.standard_normal((units, hq * d), dtype=np.float32)
    _, secs = orc.attention_units([cache] * units, [0] * units, q, [ctx - 1] * units, hq, threads)
    # `threads` units run concurrently, so a step of layers * seqs units takes units-per-thread rounds
    step_seconds = secs / units * layers * seqs
    desc = (f"{units} of {layers * seqs} (sequence, layer) units per step at context {ctx} "
            f"(one shared f32 cache), {threads} host threads, extrapolated to a full step")
    return step_seconds, desc


def run_reference(args):
    """The reference arm: the CPU restatement on all host threads.  Rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    layers, hq, hkv, d, seqs, ctx = geometry(args)
    threads = os.cpu_count() or 1
    units = args.cpu_units or threads
    cache = cpu_cache(hkv, d, ctx)
    times = []
    desc = ""
    for i in range(args.warmup + args.steps):
        t, desc = cpu_sample(cache, layers, hq, hkv, d, seqs, ctx, threads, units=units, seed=i)
        if i >= args.warmup:
            times.append(t)
    step_s = statistics.mean(times)
    value = 1.0 / step_s
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "layers": layers, "q_heads": hq, "kv_heads": hkv, "head_dim": d,
                   "sequences": seqs, "context": ctx, "kv_dtype": "f32 (the reference CPU cache)"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock, power and throttle reasons through NVML (read-only) every ~20 ms."""

    REASONS = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
               "hw_power_brake_slowdown": 0x80}

    def __init__(self, index: int):
        self.index = index
        self.sm, self.reason_bits, self.power = [], 0, []
        self.max_sm = None
        self._stop = threading.Event()
        self._thread = None
        self._h = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index(index))
            self.max_sm = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._h = None

    @staticmethod
    def _physical_index(index: int) -> int:
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            parts = [p for p in vis.split(",") if p.strip()]
            if index < len(parts) and parts[index].strip().isdigit():
                return int(parts[index])
        return index

    def _loop(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.sm.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                self.reason_bits |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                self.power.append(nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0)
            except Exception:
                pass
            self._stop.wait(0.02)

    def start(self):
        if self._h is None:
            return
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()

    def stop(self) -> dict:
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=2)
        reasons = sorted(name for name, bit in self.REASONS.items() if self.reason_bits & bit)
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.max_sm,
                "reasons": reasons, "samples": len(self.sm),
                "power_w_max": max(self.power) if self.power else None}


# ---------------------------------------------------------------------------------------------------
# the CUDA arm
# ---------------------------------------------------------------------------------------------------
def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    from itak_torch_rebuild_b200 import CudaCompute, KvDtype

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch N>1 with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    layers, hq, hkv, d, seqs, ctx = geometry(args)
    if hkv % world != 0:
        raise SystemExit(f"{hkv} KV heads do not shard over {world} GPUs")
    hkv_l, hq_l = hkv // world, hq // world
    total_steps = args.warmup + args.steps
    e2e_steps = 0 if args.no_e2e else max(3, min(args.steps, 5))
    e2e_warm = 0 if args.no_e2e else 2
    headroom = total_steps + e2e_steps + e2e_warm + 24

    be = CudaCompute(layers, hq_l, hkv_l, d, n_slots=seqs, max_context=ctx + headroom, chunk_cap=1,
                     kv_dtype=KvDtype.F16, device=local_rank)
    # One non-default stream carries the kernels, the NCCL collectives and the timing events.
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    be.set_stream(stream.cuda_stream)

    # ---- prefill the resident cache with seeded N(0,1) rows, generated on the device -----------------
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)
    slots = list(range(seqs))
    chunk = min(ctx, 4096)
    kbuf = torch.empty((seqs, chunk, hkv_l * d), device=dev, dtype=torch.float32)
    vbuf = torch.empty_like(kbuf)
    # The device append takes any row count, so the prefill runs in blocks of up to 4096 rows per sequence.
    for layer in range(layers):
        at = 0
        while at < ctx:
            n = min(chunk, ctx - at)
            kb = kbuf if n == chunk else torch.empty((seqs, n, hkv_l * d), device=dev, dtype=torch.float32)
            vb = vbuf if n == chunk else torch.empty_like(kb)
            kb.normal_(generator=gen)
            vb.normal_(generator=gen)
            be.append_rows_device(layer, slots, [at] * seqs, n, kb.data_ptr(), vb.data_ptr())
            at += n
        torch.cuda.synchronize()
    del kbuf, vbuf

    # ---- per-step inputs, resident in HBM: a pool of distinct steps --------------------------------------
    pool = min(total_steps, 8)
    q_in = torch.randn((pool, layers, seqs, hq_l * d), device=dev, dtype=torch.float32, generator=gen)
    k_in = torch.randn((pool, layers, seqs, hkv_l * d), device=dev, dtype=torch.float32, generator=gen)
    v_in = torch.randn((pool, layers, seqs, hkv_l * d), device=dev, dtype=torch.float32, generator=gen)
    out = torch.empty((layers, seqs, hq_l * d), device=dev, dtype=torch.float32)
    gathered = torch.empty((layers, world, seqs, hq_l * d), device=dev, dtype=torch.float32) if world > 1 else None
    slots_c = (C.c_uint32 * seqs)(*slots)
    position = ctx

    def pos_array(p):
        return (C.c_uint64 * seqs)(*([p] * seqs))

    def device_step(step_index, p):
        i = step_index % pool
        pc = pos_array(p)
        for layer in range(layers):
            be.attention_batch_ptrs(layer, slots_c, pc, seqs, 1, q_in[i, layer].data_ptr(), k_in[i, layer].data_ptr(),
                                    v_in[i, layer].data_ptr(), out[layer].data_ptr(), device=True)
            if world > 1:
                dist.all_gather_into_tensor(gathered[layer], out[layer])

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    gather_info = {"kind": "NCCL all-gather per layer"} if world > 1 else None
    sampler = ClockSampler(local_rank) if rank == 0 else None
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    prof_steps = 0
    if args.no_graph:
        # Direct launches: one C-ABI call per layer per step, positions passed from the host.
        for w in range(args.warmup):
            device_step(w, position)
            position += 1
        barrier()
        be.profile_enable(args.steps * layers * 2 + 8)
        launches0 = be.stats()["kernel_launches"]
        if sampler:
            sampler.start()
        ctx_first = position
        barrier()
        ev0.record(stream)
        for s in range(args.steps):
            device_step(args.warmup + s, position)
            position += 1
        ev1.record(stream)
        barrier()
        elapsed_ms = ev0.elapsed_time(ev1)
        clocks = sampler.stop() if sampler else None
        prof = be.profile_read()
        be.profile_enable(0)
        prof_steps = args.steps
        launches = be.stats()["kernel_launches"] - launches0
    else:
        # One decode step (every layer: fused append + attention [+ all-gather], then the position advance) is
        # captured once per input-pool entry as a CUDA graph over device-side positions, and replayed.
        device_step(0, position)  # also brings NCCL up before any capture
        position += 1
        barrier()
        replays = args.warmup + args.steps
        fused = world > 1 and not args.nccl_gather
        slot_bytes = seqs * hq_l * d * 4
        if fused:
            # Every rank's gather buffer [layers][world][seqs][hq_l * d]; the decode kernel of rank r writes its
            # rows into slot [layer][r] of every rank's buffer.
            _, handle = be.gather_create(world, rank, layers * world * slot_bytes)
            handles = [None] * world
            dist.all_gather_object(handles, handle)
            for r in range(world):
                be.gather_open(r, handles[r])
            be.gather_reset()
            barrier()
        be.resident_begin(slots, replays)
        graphs = []
        for i in range(pool):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for layer in range(layers):
                    if fused:
                        be.resident_layer_gather(layer, q_in[i, layer].data_ptr(), k_in[i, layer].data_ptr(),
                                                 v_in[i, layer].data_ptr(), (layer * world + rank) * slot_bytes)
                    else:
                        be.resident_layer(layer, q_in[i, layer].data_ptr(), k_in[i, layer].data_ptr(),
                                          v_in[i, layer].data_ptr(), out[layer].data_ptr())
                        if world > 1:
                            dist.all_gather_into_tensor(gathered[layer], out[layer])
                be.resident_advance()
            graphs.append(g)
        torch.cuda.set_stream(stream)
        for w in range(args.warmup):
            graphs[w % pool].replay()
        barrier()
        if sampler:
            sampler.start()
        ctx_first = position + args.warmup
        barrier()
        ev0.record(stream)
        for s in range(args.steps):
            graphs[(args.warmup + s) % pool].replay()
        ev1.record(stream)
        barrier()
        elapsed_ms = ev0.elapsed_time(ev1)
        clocks = sampler.stop() if sampler else None
        be.resident_end(replays)
        position += replays
        if fused:
            gather_info = {"kind": "stores to peer memory from the decode kernel, flag per source rank",
                           "waits_timed_out": be.gather_status()}
        launches = args.steps * (layers + 1)  # per rank: one fused kernel per layer plus the position advance
        del graphs, g
        # The same steps once more as direct launches with a CUDA-event pair around every kernel: the decode
        # kernel's own duration for the roofline (identical kernel; events cannot bracket nodes of a replayed graph).
        prof_steps = min(args.steps, 8)
        be.profile_enable(prof_steps * layers * 2 + 8)
        for s in range(prof_steps):
            device_step(s, position)
            position += 1
        prof = be.profile_read()
        be.profile_enable(0)
        barrier()
    splits = be.stats()["last_splits"]
    if world > 1:
        t = torch.tensor([elapsed_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
        lt = torch.tensor([launches], device=dev, dtype=torch.int64)
        dist.all_reduce(lt, op=dist.ReduceOp.SUM)
        launches = int(lt.item())
    ms_per_step = elapsed_ms / args.steps
    value = 1e3 / ms_per_step

    # ---- roofline of the attention kernel (this rank's shard), live CUDA-event time per launch -------------
    bytes_step_total = kv_bytes_per_step(layers, hkv, d, seqs, ctx_first, args.steps)
    bytes_launch_rank = bytes_step_total / layers / world
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_src = 6650.0, "fallback (earlier measurement on this pool)"
    attn_ms = prof["attention_ms"] / max(prof["attention_launches"], 1)
    achieved = bytes_launch_rank / (attn_ms * 1e-3) / 1e9 if attn_ms > 0 else None
    # DRAM traffic per launch: ncu measured 269.24 MB read + 4.3 MB written against 268.60 MB algorithmic on a
    # context-8192 capture of this kernel (profiles/decode_f16_kernel_c5_small.md); traffic grows in proportion to
    # the keys streamed, so the full launch is that ratio times its algorithmic bytes.
    traffic = bytes_launch_rank * (269.24 + 4.3) / 268.60
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": (achieved / peak) if achieved else None, "traffic": traffic,
                "traffic_source": "ncu dram__bytes_read+write of a context-8192 capture, scaled by keys streamed",
                "peak_source": peak_src,
                "kernel": "decode_f16_kernel<128,3>", "bytes_per_launch": bytes_launch_rank,
                "avg_launch_ms": attn_ms, "launches_timed": prof["attention_launches"],
                "timed_as": "event pair around every launch" + ("" if args.no_graph else ", direct-launch pass after the graph replays"),
                "append_avg_launch_ms": prof["append_ms"] / max(prof["append_launches"], 1),
                "kv_splits": splits,
                "whole_step_kv_gbs": bytes_step_total / (ms_per_step * 1e-3) / 1e9}

    # ---- end to end through the host-buffer call: H2D of q/k/v, kernels, D2H of the result, per layer ------
    e2e = None
    if not args.no_e2e:
        hq_pin = torch.randn((layers, seqs, hq_l * d), dtype=torch.float32).pin_memory()
        hk_pin = torch.randn((layers, seqs, hkv_l * d), dtype=torch.float32).pin_memory()
        hv_pin = torch.randn((layers, seqs, hkv_l * d), dtype=torch.float32).pin_memory()
        ho_pin = torch.empty((layers, seqs, hq_l * d), dtype=torch.float32).pin_memory()

        def host_step(p):
            pc = pos_array(p)
            for layer in range(layers):
                be.attention_batch_ptrs(layer, slots_c, pc, seqs, 1, hq_pin[layer].data_ptr(), hk_pin[layer].data_ptr(),
                                        hv_pin[layer].data_ptr(), ho_pin[layer].data_ptr(), device=False)

        for _ in range(e2e_warm):
            host_step(position)
            position += 1
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            host_step(position)
            position += 1
        barrier()
        e2e_s = (time.perf_counter() - t0) / e2e_steps
        if world > 1:
            t = torch.tensor([e2e_s], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_s = float(t.item())
        h2d = layers * seqs * (hq_l + 2 * hkv_l) * d * 4 * world
        d2h = layers * seqs * hq_l * d * 4 * world
        e2e = {"value": 1.0 / e2e_s, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "steps": e2e_steps, "note": "host-buffer itk_attention_batch per layer; each rank moves its head shard"}

    # ---- CPU baseline on this box's cores (rank 0, N = 1 only) ------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        step_s, desc = cpu_sample(cpu_cache(hkv, d, ctx), layers, hq, hkv, d, seqs, ctx, threads,
                                  units=args.cpu_units or threads)
        cpu = {"value": 1.0 / step_s, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32 math over an f16 KV cache", "data": "synthetic",
            "config": {"workload": args.workload, "layers": layers, "q_heads": hq, "kv_heads": hkv, "head_dim": d,
                       "sequences": seqs, "context": ctx_first, "kv_dtype": "f16",
                       "launch": "direct" if args.no_graph else "cuda graph per step over device-side positions",
                       "parallelism": f"kv-head shards x{world}", "gather": gather_info,
                       "l2": "inputs larger than L2: every layer streams its own KV, "
                             f"{bytes_launch_rank / 2**20:.0f} MiB per launch"},
            "kv_read_gbs": bytes_step_total / (ms_per_step * 1e-3) / 1e9,
            "kv_read_frac_of_hbm_peak": bytes_step_total / world / (ms_per_step * 1e-3) / 1e9 / peak,
            "roofline": roofline, "e2e": e2e, "cpu_baseline": cpu, "clocks": clocks, "gpu_launches": launches,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        # Leave without tearing the communicator down: NCCL teardown after graph capture has been seen to wait
        # forever, and there is nothing left to release that process exit does not release.
        barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    be.close()


def main():
    args = parse_args()
    if args.workload in ("c4_prefix_restore", "c4_spec_verify"):
        # the path's other rows, one GPU, measured by bench_paths.py in the same JSON shape
        import bench_paths

        if args.impl == "reference" or args.gpus != 1:
            print(json.dumps({"impl": args.impl, "unavailable": "this workload is measured on one GPU, CUDA arm only"}))
            return
        (bench_paths.run_prefix_restore if args.workload == "c4_prefix_restore" else bench_paths.run_spec_verify)(
            args, ClockSampler)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
