"""Decode-attention throughput of the KV-cache hot path on N B200s (one process per GPU).

Workload (default): the long-context decode configuration - 48 layers, 64 query heads, 8 KV heads,
head dim 128, f16 KV cache, 8 resident sequences at 32768 tokens of context.  One "step" is one decode
step of the hot path: for every layer, append one RoPE'd K/V row per sequence and run GQA attention over
the whole resident cache.  At N > 1 the KV heads are sharded (8 / N per GPU, strong scaling) and each
layer ends with one all-gather of the per-head outputs, done by the decode kernel itself over NVLink.

Prints ONE JSON line: decode steps/s (whole job), with
  roofline      - the attention kernel's algorithmic KV bytes / its CUDA-event time vs the measured HBM peak,
  e2e           - the same step through the host-buffer C-ABI call (H2D + kernels + D2H inside the timed region),
  cpu_baseline  - the CPU restatement of the reference's attention timed on this box's cores (bounded sample),
  clocks        - SM clocks and throttle reasons sampled during the timed region,
  gather_check  - N > 1: the fused gather's buffer compared with an NCCL all-gather of the same step, every rank,
  paths         - N = 1: short measurements of the other configurations (single-sequence decode, continuous
                  batching, the f32 prefill + decode case, prefix restore, speculative verify, chunked prefill), see
                  bench_paths.py.
The `--steps` block is replayed several times (the same positions each time) until about a second has been
timed; `value` is the median block, min / max and the block count are in `blocks`.
`--impl reference` times only the CPU restatement (the reference's own CPU path cannot be built here: it is Rust).
Inputs are seeded synthetic N(0,1) tensors of the configuration's shapes, generated on the device.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import math
import os
import statistics
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
PATH_WORKLOADS = ["c1_tinyllama_f32", "c3_continuous_batching", "c4_prefix_restore", "c4_spec_verify", "c4_chunked_prefill"]
METRIC = "decode_attention_steps_per_s"
UNIT = "steps/s"
# DRAM traffic of one decode launch relative to its algorithmic KV bytes, from an ncu capture of this kernel at
# context 8192 (269.24 MB read + 4.3 MB written against 268.60 MB algorithmic); traffic grows with the keys streamed.
DECODE_TRAFFIC_RATIO = (269.24 + 4.3) / 268.60


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c5_long_context_decode", choices=sorted(WORKLOADS) + PATH_WORKLOADS)
    ap.add_argument("--context", type=int, default=None, help="override the context length (smoke runs)")
    ap.add_argument("--layers", type=int, default=None, help="override the layer count (smoke runs)")
    ap.add_argument("--q-heads", type=int, default=None, help="override the query head count (shard studies)")
    ap.add_argument("--kv-heads", type=int, default=None, help="override the KV head count (shard studies)")
    ap.add_argument("--sequences", type=int, default=None, help="override the number of resident sequences")
    ap.add_argument("--sessions", type=int, default=None, help="config 4 workloads: sessions on the shared prefix (default 16)")
    ap.add_argument("--prefix-tokens", type=int, default=None, help="config 4 workloads: length of the shared prefix (default 2048)")
    ap.add_argument("--no-graph", action="store_true", help="launch every layer directly instead of replaying a CUDA graph")
    ap.add_argument("--nccl-gather", action="store_true",
                    help="N > 1: gather the head outputs with an NCCL all-gather per layer instead of inside the kernel")
    ap.add_argument("--self-gather", action="store_true",
                    help="N = 1: run the fused-gather form of the loop with this GPU as its only rank (shard studies)")
    ap.add_argument("--blocks", type=int, default=None, help="timed repetitions of the --steps block (default: ~1 s worth)")
    ap.add_argument("--option", action="append", default=[], metavar="NAME=VALUE", help="backend option (itk_set_option)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-paths", action="store_true", help="N = 1: skip the short runs of the other configurations")
    ap.add_argument("--cpu-units", type=int, default=None, help="(sequence, layer) units in the CPU sample")
    return ap.parse_args()


def geometry(args, workload=None):
    layers, hq, hkv, d, seqs, ctx = WORKLOADS[workload or args.workload]
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


def backend_options(args):
    out = {}
    for item in args.option:
        name, _, value = item.partition("=")
        out[name] = int(value)
    return out


def kv_bytes_per_step(layers, hkv, d, seqs, ctx_first, steps, elem=2):
    """Algorithmic KV-read bytes: visible keys x Hkv x D x 2 (K, V) x element size, summed over
    (sequence, layer), averaged over the timed steps (the context grows by one per step)."""
    total = 0
    for s in range(steps):
        total += (ctx_first + s + 1) * hkv * d * 2 * elem * layers * seqs
    return total / max(steps, 1)


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (earlier measurement on this pool)"


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
    if args.workload in PATH_WORKLOADS:
        print(json.dumps({"impl": "reference", "unavailable": "the CPU leg of this workload is the cpu_baseline of its own line"}))
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


class _DevArray:
    """A device pointer dressed as a CUDA array so torch can view it."""

    def __init__(self, ptr, n):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (ptr, False), "version": 2}


class Dist:
    """Rank bookkeeping and the collectives the bench itself needs (barrier, max / sum over ranks)."""

    def __init__(self, args):
        import torch

        self.torch = torch
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={self.world}: launch N>1 with torch.distributed.run")
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.dist is not None:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def reduce(self, values, op="max", dtype=None):
        """Element-wise max (or sum) over ranks of a list of numbers."""
        if self.dist is None:
            return list(values)
        torch = self.torch
        t = torch.tensor(list(values), device=self.dev, dtype=dtype or torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX if op == "max" else self.dist.ReduceOp.SUM)
        return t.tolist()


# ---------------------------------------------------------------------------------------------------
# the CUDA arm: a resident decode loop over one geometry
# ---------------------------------------------------------------------------------------------------
def measure_decode(args, env: Dist, workload, geom, steps, warmup, *, e2e=True, cpu=True, target_ms=1100.0):
    """Build the resident cache for `geom`, time `steps` decode steps (replayed as blocks), and return the
    JSON line's dictionary (rank 0; None elsewhere)."""
    import numpy as np  # noqa: F401
    torch = env.torch
    dist = env.dist

    from itak_torch_rebuild_b200 import CudaCompute, KvDtype

    rank, world, dev = env.rank, env.world, env.dev
    layers, hq, hkv, d, seqs, ctx = geom
    if hkv % world != 0:
        raise SystemExit(f"{hkv} KV heads do not shard over {world} GPUs")
    hkv_l, hq_l = hkv // world, hq // world
    e2e_steps = max(3, min(steps, 5)) if e2e else 0
    e2e_warm = 2 if e2e else 0
    prof_steps = min(steps, 8)
    headroom = 1 + warmup + steps + prof_steps + e2e_steps + e2e_warm + 4 + 24

    be = CudaCompute(layers, hq_l, hkv_l, d, n_slots=seqs, max_context=ctx + headroom, chunk_cap=1,
                     kv_dtype=KvDtype.F16, device=env.local_rank, options=backend_options(args))
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
    pool = min(warmup + steps, 8)
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

    barrier = env.barrier
    gather_info = {"kind": "NCCL all-gather per layer"} if world > 1 else None
    gather_check = None
    sampler = ClockSampler(env.local_rank) if rank == 0 else None
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    block_ms = []
    if args.no_graph:
        # Direct launches: one C-ABI call per layer per step, positions passed from the host.
        for w in range(warmup):
            device_step(w, position)
            position += 1
        barrier()
        be.profile_enable(steps * layers * 2 + 8)
        launches0 = be.stats()["kernel_launches"]
        if sampler:
            sampler.start()
        ctx_first = position
        barrier()
        ev0.record(stream)
        for s in range(steps):
            device_step(warmup + s, position)
            position += 1
        ev1.record(stream)
        barrier()
        block_ms = [ev0.elapsed_time(ev1)]
        clocks = sampler.stop() if sampler else None
        prof = be.profile_read()
        be.profile_enable(0)
        launches = be.stats()["kernel_launches"] - launches0
    else:
        # One decode step (every layer: fused append + attention [+ all-gather], then the position advance) is
        # captured once per input-pool entry as a CUDA graph over device-side positions, and replayed.
        device_step(0, position)  # also brings NCCL up before any capture
        position += 1
        barrier()
        fused = (world > 1 and not args.nccl_gather) or (world == 1 and args.self_gather)
        slot_bytes = seqs * hq_l * d * 4
        gather_view = None
        if fused:
            # Every rank's gather buffer [layers][world][seqs][hq_l * d]; the decode kernel of rank r writes its
            # rows into slot [layer][r] of every rank's buffer.
            ptr, handle = be.gather_create(world, rank, layers * world * slot_bytes)
            if world > 1:
                handles = [None] * world
                dist.all_gather_object(handles, handle)
                for r in range(world):
                    be.gather_open(r, handles[r])
            gather_view = torch.as_tensor(_DevArray(ptr, layers * world * slot_bytes // 4), device=dev).view(
                layers, world, seqs, hq_l * d)

        def begin(n_steps):
            if fused:
                barrier()  # every rank is out of the previous loop before anybody clears its flags
                be.gather_reset()
                barrier()
            be.resident_begin(slots, n_steps)

        def capture(i, fused_form):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for layer in range(layers):
                    if fused_form:
                        be.resident_layer_gather(layer, q_in[i, layer].data_ptr(), k_in[i, layer].data_ptr(),
                                                 v_in[i, layer].data_ptr(), (layer * world + rank) * slot_bytes)
                    else:
                        be.resident_layer(layer, q_in[i, layer].data_ptr(), k_in[i, layer].data_ptr(),
                                          v_in[i, layer].data_ptr(), out[layer].data_ptr())
                        if world > 1:
                            dist.all_gather_into_tensor(gathered[layer], out[layer])
                be.resident_advance()
            return g

        begin(max(warmup, 1))
        graphs = [capture(i, fused) for i in range(pool)]
        torch.cuda.set_stream(stream)
        for w in range(warmup):
            graphs[w % pool].replay()
        barrier()
        be.resident_end(warmup)
        position += warmup
        ctx_first = position
        warm_timeouts = int(env.reduce([float(be.gather_status())])[0]) if fused else 0  # (cleared with every begin)

        def timed_block():
            begin(steps)
            barrier()
            ev0.record(stream)
            for s in range(steps):
                graphs[(warmup + s) % pool].replay()
            ev1.record(stream)
            barrier()
            be.resident_end(0)  # the next block runs the same steps again
            return ev0.elapsed_time(ev1)

        if sampler:
            sampler.start()
        first = env.reduce([timed_block()])[0]
        block_ms.append(first)
        n_blocks = args.blocks or int(min(200, max(1, math.ceil(target_ms / max(first, 1e-3)))))
        for _ in range(n_blocks - 1):
            block_ms.append(timed_block())
        clocks = sampler.stop() if sampler else None
        if fused:
            gather_info = {"kind": "stores to peer memory from the decode kernel, arrival counters per (sequence, source rank)",
                           "waits_timed_out": be.gather_status(), "waits_timed_out_in_warmup": warm_timeouts}
        launches = steps * (layers + 1)  # per rank and block: one fused kernel per layer plus the position advance

        # ---- N > 1: the fused gather's values against an NCCL all-gather of the same step, on every rank ------
        if fused and world > 1:
            begin(1)
            graphs[0].replay()
            barrier()
            got = gather_view.clone()
            be.resident_end(0)
            begin(1)
            for layer in range(layers):
                be.resident_layer(layer, q_in[0, layer].data_ptr(), k_in[0, layer].data_ptr(), v_in[0, layer].data_ptr(),
                                  out[layer].data_ptr())
                dist.all_gather_into_tensor(gathered[layer], out[layer])
            be.resident_advance()
            barrier()
            be.resident_end(0)
            scale = float(gathered.abs().max().item())
            err = float((got - gathered).abs().max().item()) / max(scale, 1e-30)
            worst = env.reduce([err])[0]
            gather_check = {"max_rel_err": worst, "tolerance": 1e-5, "ok": bool(worst <= 1e-5), "layers": layers,
                            "ranks": world, "against": "resident_layer + NCCL all_gather_into_tensor of the same step"}
        del graphs
        # The same steps once more as direct launches with a CUDA-event pair around every kernel: the decode
        # kernel's own duration for the roofline (identical kernel; events cannot bracket nodes of a replayed graph).
        be.profile_enable(prof_steps * layers * 2 + 8)
        for s in range(prof_steps):
            device_step(s, position)
            position += 1
        prof = be.profile_read()
        be.profile_enable(0)
        barrier()
    splits = be.stats()["last_splits"]
    if world > 1:
        block_ms = env.reduce(block_ms)
        launches = int(env.reduce([launches], op="sum")[0])
    elapsed_ms = statistics.median(block_ms)
    ms_per_step = elapsed_ms / steps
    value = 1e3 / ms_per_step

    # ---- roofline of the attention kernel (this rank's shard), live CUDA-event time per launch -------------
    bytes_step_total = kv_bytes_per_step(layers, hkv, d, seqs, ctx_first, steps)
    bytes_launch_rank = bytes_step_total / layers / world
    peak, peak_src = hbm_peak()
    pair_ms = prof["attention_ms"] / max(prof["attention_launches"], 1)
    pair_gbs = bytes_launch_rank / (pair_ms * 1e-3) / 1e9 if pair_ms > 0 else None
    if args.no_graph:
        attn_ms, timed_as = pair_ms, "CUDA-event pair around every launch of the timed region"
    else:
        # the timed region of a replayed step holds nothing but the decode launches, back to back, and one
        # position-advance kernel per step: its CUDA-event time over its launches is the launch duration
        attn_ms = ms_per_step / layers
        timed_as = ("CUDA events around the timed region / decode launches in it (graph replay: a step is its layers' "
                    "launches back to back plus one position-advance kernel)")
    achieved = bytes_launch_rank / (attn_ms * 1e-3) / 1e9 if attn_ms > 0 else None
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": (achieved / peak) if achieved else None, "traffic": bytes_launch_rank * DECODE_TRAFFIC_RATIO,
                "traffic_source": "ncu dram__bytes_read+write of a context-8192 capture, scaled by keys streamed",
                "peak_source": peak_src,
                "kernel": f"decode_f16_kernel<{d},{3 if d == 128 else 4}>", "bytes_per_launch": bytes_launch_rank,
                "avg_launch_ms": attn_ms, "launches_timed": steps * layers * len(block_ms), "timed_as": timed_as,
                "event_pair": {"avg_launch_ms": pair_ms, "achieved": pair_gbs, "frac": (pair_gbs / peak) if pair_gbs else None,
                               "launches_timed": prof["attention_launches"],
                               "note": "the same steps as direct launches with a CUDA-event pair around each "
                                       "(the pair itself costs a few microseconds)"},
                "append_avg_launch_ms": prof["append_ms"] / max(prof["append_launches"], 1),
                "kv_splits": splits,
                "whole_step_kv_gbs": bytes_step_total / (ms_per_step * 1e-3) / 1e9}

    # ---- end to end from host buffers: H2D of q/k/v, kernels, D2H of the result, inside the timed region ------
    e2e_rec = None
    if e2e:
        hq_pin = torch.randn((layers, seqs, hq_l * d), dtype=torch.float32).pin_memory()
        hk_pin = torch.randn((layers, seqs, hkv_l * d), dtype=torch.float32).pin_memory()
        hv_pin = torch.randn((layers, seqs, hkv_l * d), dtype=torch.float32).pin_memory()
        ho_pin = torch.empty((layers, seqs, hq_l * d), dtype=torch.float32).pin_memory()

        def per_layer_step(p):
            pc = pos_array(p)
            for layer in range(layers):
                be.attention_batch_ptrs(layer, slots_c, pc, seqs, 1, hq_pin[layer].data_ptr(), hk_pin[layer].data_ptr(),
                                        hv_pin[layer].data_ptr(), ho_pin[layer].data_ptr(), device=False)

        def whole_step(p):
            be.attention_layers_host_ptrs(slots_c, pos_array(p), seqs, 1, hq_pin.data_ptr(), hk_pin.data_ptr(),
                                          hv_pin.data_ptr(), ho_pin.data_ptr())

        def time_host(fn, n_warm, n_steps):
            nonlocal position
            for _ in range(n_warm):
                fn(position)
                position += 1
            barrier()
            t0 = time.perf_counter()
            for _ in range(n_steps):
                fn(position)
                position += 1
            barrier()
            return env.reduce([(time.perf_counter() - t0) / n_steps])[0]

        whole_s = time_host(whole_step, e2e_warm, e2e_steps)
        layer_s = time_host(per_layer_step, 1, 3)
        h2d = layers * seqs * (hq_l + 2 * hkv_l) * d * 4 * world
        d2h = layers * seqs * hq_l * d * 4 * world
        e2e_rec = {"value": 1.0 / whole_s, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                   "steps": e2e_steps,
                   "call": "itk_attention_layers_host: one call per step, pinned host q/k/v/out of all layers, returns with "
                           "the step's result on the host; "
                           + ("uploads / kernels / downloads of consecutive layers overlapped on three streams"
                              if h2d // world > (8 << 20) else
                              "a step of 8 MiB or less: three strided uploads, the step as one step of the replayable "
                              "loop, one strided download"),
                   "per_layer_call": {"value": 1.0 / layer_s, "unit": UNIT, "steps": 3,
                                      "call": "itk_attention_batch per layer (the reference's Compute::attention shape): "
                                              "H2D, kernel, D2H and a synchronisation every layer"},
                   "note": "each rank moves its head shard"}

    # ---- CPU baseline on this box's cores (rank 0, N = 1 only) ------------------------------------------------
    cpu_rec = None
    if rank == 0 and world == 1 and cpu:
        threads = os.cpu_count() or 1
        step_s, desc = cpu_sample(cpu_cache(hkv, d, ctx), layers, hq, hkv, d, seqs, ctx, threads,
                                  units=args.cpu_units or threads)
        cpu_rec = {"value": 1.0 / step_s, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc}

    if world > 1 and not args.no_graph and not args.nccl_gather:
        be.gather_close_peers()  # no rank frees its gather buffer while a peer still maps it
        barrier()
    be.close()
    torch.cuda.set_stream(torch.cuda.default_stream(dev))
    if rank != 0:
        return None if gather_check is None or gather_check["ok"] else {"gather_check": gather_check}
    return {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32 math over an f16 KV cache", "data": "synthetic",
        "config": {"workload": workload, "layers": layers, "q_heads": hq, "kv_heads": hkv, "head_dim": d,
                   "sequences": seqs, "context": ctx_first, "kv_dtype": "f16",
                   "launch": "direct" if args.no_graph else "cuda graph per step over device-side positions",
                   "parallelism": f"kv-head shards x{world}", "gather": gather_info,
                   "l2": "inputs larger than L2: every layer streams its own KV, "
                         f"{bytes_launch_rank / 2**20:.0f} MiB per launch" if bytes_launch_rank > 126e6 else
                         f"{bytes_launch_rank / 2**20:.1f} MiB per launch, {layers} layers of it between two visits of a layer"},
        "blocks": {"count": len(block_ms), "ms_median": elapsed_ms, "ms_min": min(block_ms), "ms_max": max(block_ms),
                   "note": "each block is the same --steps steps from the same positions"},
        "kv_read_gbs": bytes_step_total / (ms_per_step * 1e-3) / 1e9,
        "kv_read_frac_of_hbm_peak": bytes_step_total / world / (ms_per_step * 1e-3) / 1e9 / peak,
        "roofline": roofline, "e2e": e2e_rec, "cpu_baseline": cpu_rec, "clocks": clocks, "gather_check": gather_check,
        "gpu_launches": launches,
    }


def run_ours(args):
    env = Dist(args)
    line = None
    failed = False
    if args.workload in WORKLOADS:
        line = measure_decode(args, env, args.workload, geometry(args), args.steps, args.warmup, e2e=not args.no_e2e,
                              cpu=not args.no_cpu_baseline)
        if env.world == 1 and not args.no_paths and args.workload == "c5_long_context_decode" and not (
                args.context or args.layers or args.kv_heads or args.q_heads or args.sequences):
            # short runs of the path's other configurations, each in the shape of a bench line
            import bench_paths

            paths = {}
            c2 = measure_decode(args, env, "c2_single_sequence_decode", WORKLOADS["c2_single_sequence_decode"], 128, 3,
                                target_ms=300.0)
            paths["c2_single_sequence_decode"] = c2
            for name in PATH_WORKLOADS:
                paths[name] = bench_paths.RUNNERS[name](args, ClockSampler, short=True)
            line["paths"] = paths
    else:
        import bench_paths

        if env.world != 1:
            line = {"unavailable": "this workload is measured on one GPU"} if env.rank == 0 else None
        else:
            if args.sessions:
                bench_paths.SESSIONS = args.sessions
            if args.prefix_tokens:
                bench_paths.PREFIX = args.prefix_tokens
            line = bench_paths.RUNNERS[args.workload](args, ClockSampler, short=False)
    check = (line or {}).get("gather_check")
    if check is not None and not check["ok"]:
        failed = True
    if env.rank == 0 and line is not None:
        print(json.dumps(line), flush=True)
    if env.world > 1:
        flag = env.reduce([1.0 if failed else 0.0])[0]
        env.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        code = 1 if flag else 0
        # Orderly teardown - every graph and backend (and with them the peer mappings) is gone by now, then the
        # communicator - under a watchdog: an earlier form of this script left a captured graph holding NCCL work
        # alive when it destroyed the process group and waited forever there.  Should teardown ever stall again,
        # the line above has been printed and the process leaves after ten seconds regardless.
        watchdog = threading.Timer(10.0, lambda: os._exit(code))
        watchdog.daemon = True
        watchdog.start()
        env.dist.destroy_process_group()
        os._exit(code)
    if failed:
        raise SystemExit(1)


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
