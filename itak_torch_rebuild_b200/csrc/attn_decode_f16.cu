// GQA flash-decode over the f16 resident cache: one query row per sequence.
//
// Stands in for the reference's decode attention, i.e. gqa_attention with one
// query (crates/attention/src/attention.rs:104-215) reading an f16 cache the
// way the K6 flash f16 shader does (crates/wgpu-compute/src/kernels/k6_attention.rs:642-914):
// keys and values are upconverted exactly, all arithmetic accumulates in f32.
//
// Work split (what the reference kernels lack).  A "cell" is one
// (sequence, KV head chunk): all query heads of the GQA group share every K/V
// tile, so each cache byte crosses HBM once per step.  The launch's tiles
// (64 keys each), laid end to end over all cells, are cut into equal
// contiguous runs, one per persistent CTA - two CTAs per SM, every SM busy
// until the last tile whatever the batch's context lengths are.  A CTA whose
// run crosses a cell boundary finishes its part of the first cell and moves
// on; each part writes an (m, l, o) partial and the last CTA to arrive at a
// cell merges them (finish_unit).  Nobody waits for anybody.
// A CTA that crosses a cell boundary pays that cell's epilogue (and a fresh
// query load and pipeline refill) in the middle of its run and finishes late,
// so when the cells are alike enough that giving each its own whole number of
// CTAs lengthens no run by more than a sixteenth, the plan is cell-aligned
// instead: floor(CTAs * T_cell / total) CTAs per cell, equal runs inside it.
//
// Inside a CTA each of the 4 warps owns a private cp.async pipeline over its
// own 16-key slice of every tile: 16-byte coalesced loads into XOR-swizzled
// shared memory, STAGES tiles in flight, no CTA-wide barrier except where a
// cell ends.  The cache is head-major, so a CTA's loads walk contiguous streams.
//
// The step's new K/V row can ride along (AttnLaunch::k_new): the one warp whose
// slice holds position kv_hi - 1 converts the f32 row (round-to-nearest-even,
// the append kernel's function), stores it to the cache and drops it into its
// own staged tile, which saves the separate append launch of a decode step.
//
// Bound: HBM.  A cache element (2 B) feeds 2 * group MACs, 4 FMA/B at group 8;
// at 6.5 TB/s that is ~70% of the SM's fp32 FMA rate before counting the
// f16->f32 converts, so the dot products run on the tensor pipe instead, as
// mma.sync.m16n8k16 with M = 16 = 8 heads x {hi, lo}: the f32 query (and the
// f32 softmax weight) is split into two f16 terms that occupy the rows a GQA
// group of 8 would otherwise leave as padding.  The products are then exact to
// ~2^-22 and the accumulation is f32, so the result tracks the f32 reference
// far inside the f16-KV tolerance.  A 64-row tcgen05 tile would be 7/8 padding
// here; the tensor pipe is at ~18% load either way and never the limiter.
#include <cstdio>
#include <mutex>

#include "attn_common.cuh"
#include "kv_convert.cuh"

namespace itk {

namespace {

constexpr int kDecodeThreads = 128;
constexpr int kDecodeWarps = 4;
constexpr int kTileKeys = 64;  // keys per CTA tile = 16 per warp
// Work plan in shared memory: cum[65] tiles before each sequence, abase[65] first CTA of each sequence in the
// cell-aligned plan, then per sequence its visible keys, first storage row and slot, then the plan's mode word.
constexpr int kPlanWords = kDecodePlanWords;
constexpr int kPlanCum = 0, kPlanAbase = kMaxSeqsPerLaunch + 4, kPlanSn = 2 * (kMaxSeqsPerLaunch + 4),
              kPlanSs0 = kPlanSn + kMaxSeqsPerLaunch, kPlanSlot = kPlanSs0 + kMaxSeqsPerLaunch,
              kPlanMode = kPlanSlot + kMaxSeqsPerLaunch;  // [mode] 1 = cell-aligned plan, [mode + 1] steps done

// A walker's place in the launch's tile sequence (warp-uniform).
struct TileCursor {
    uint32_t seq, hy, tile;  // current cell (sequence, head chunk) and tile inside it
    uint32_t T;              // tiles of the current sequence
    uint32_t n;              // visible keys of the current sequence
    uint32_t s0;             // storage row of its first visible key
    uint32_t slot;
};

// The i-th sequence of the launch, from the parameters or from device-resident state.
__device__ __forceinline__ SeqDesc seq_of(const AttnLaunch& p, uint32_t i) {
    if (p.seq_dev == nullptr) return p.seq[i];
    const SeqState st = p.seq_dev[i];
    SeqDesc d;
    d.slot = st.slot;
    d.q_pos0 = st.pos;
    d.kv_hi = st.pos + 1;
    d.kv_lo = (p.layer.window != 0 && st.pos + 1 > p.layer.window) ? st.pos + 1 - p.layer.window : 0u;
    return d;
}

// Programmatic dependent launch: let the next kernel in the stream be scheduled early / wait until the
// previous one has completed and its writes are visible.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

// One plan block: sequences [s0, s1) of the batch on G CTAs.  `w` is the block's kPlanWords words (shared or global
// memory) whose per-sequence entries (kPlanSn, kPlanSs0, kPlanSlot) are already filled for the whole batch.
__device__ __forceinline__ void fill_plan_block(uint32_t* w, uint32_t s0, uint32_t s1, uint32_t HY, uint32_t G,
                                                uint32_t splits) {
    const uint32_t* sn = w + kPlanSn + s0;
    uint32_t c = 0;
    for (uint32_t s = 0; s < s1 - s0; ++s) {
        w[kPlanCum + s] = c;
        c += (sn[s] + kTileKeys - 1) / kTileKeys * HY;
    }
    w[kPlanCum + (s1 - s0)] = c;
    uint32_t worst;
    const uint32_t per = G ? (c + G - 1) / G : 0u;
    w[kPlanMode] = (G != 0 && decode_aligned_plan(sn, s1 - s0, HY, G, c, per, splits, w + kPlanAbase, &worst)) ? 1u : 0u;
}

__global__ void advance_states_kernel(SeqState* states, uint32_t n, uint32_t add, DecodePlanSpec spec, uint32_t* plan_out) {
    __shared__ uint32_t w[kDecodePlanBlocks][kPlanWords];
    const uint32_t tid = threadIdx.x;
    uint32_t pos = 0;
    if (tid < n) {
        SeqState st = states[tid];
        st.pos += add;
        pos = st.pos;
        states[tid] = st;
        for (int b = 0; b < kDecodePlanBlocks; ++b) {
            w[b][kPlanSn + tid] = pos + 1;  // global layers: positions 0..pos are visible
            w[b][kPlanSs0 + tid] = 0;
            w[b][kPlanSlot + tid] = st.slot;
        }
    }
    if (plan_out == nullptr) return;
    // (the loop's first position sits in a device word behind the blocks, not in the launch parameters: a captured
    // step is replayed by loops that begin at other positions)
    if (tid == 0)
        for (int b = 0; b < kDecodePlanBlocks; ++b) w[b][kPlanMode + 1] = pos - plan_out[kDecodePlanBlocks * kPlanWords];
    __syncthreads();
    if (tid == 0) fill_plan_block(w[0], 0, n, spec.cells_per_seq, spec.ctas, spec.splits);
    if (tid == 32 && spec.lane_ctas != 0) fill_plan_block(w[1], 0, spec.lane_split, spec.cells_per_seq, spec.lane_ctas / 2, spec.splits);
    if (tid == 63 && spec.lane_ctas != 0) fill_plan_block(w[2], spec.lane_split, n, spec.cells_per_seq, spec.lane_ctas / 2, spec.splits);
    __syncthreads();
    for (uint32_t i = tid; i < kDecodePlanBlocks * kPlanWords; i += blockDim.x) plan_out[i] = (&w[0][0])[i];
}

template <int D, int STAGES>
__host__ __device__ constexpr size_t decode_pipe_bytes() {
    return static_cast<size_t>(STAGES) * kDecodeWarps * 2 * 16 * D * 2;
}
template <int D, int STAGES>
constexpr size_t decode_smem_bytes() {
    // pipeline (its stage just consumed doubles as the warps' exchange area at a cell end) + fo[8][D]
    // + wm/wl[4][8] x2 + fm, fl + flag pad + merge weights + cumulative tile table
    return decode_pipe_bytes<D, STAGES>() +
           (kHeadsPerCta * D + 2 * kDecodeWarps * kHeadsPerCta + 2 * kHeadsPerCta + 4 +
            2 * kDecodeMaxParts * kHeadsPerCta + kHeadsPerCta + kPlanWords) * sizeof(float);
}

template <int D, int STAGES>
__global__ void __launch_bounds__(kDecodeThreads, 2) decode_f16_kernel(const __grid_constant__ AttnLaunch p) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int kRowBytes = D * 2;
    constexpr int kSliceBytes = 16 * kRowBytes;  // one warp's K (or V) slice of a tile
    constexpr int kChunksPerRow = D / 8;         // 16-byte chunks in a row
    constexpr int KS = D / 16;                   // k-steps of the QK^T product
    constexpr int NT = D / 8;                    // n-tiles of the PV product

    float* fo = reinterpret_cast<float*>(smem + decode_pipe_bytes<D, STAGES>());      // [8][D]
    float* wm = fo + kHeadsPerCta * D;                                               // [4][8]
    float* wl = wm + kDecodeWarps * kHeadsPerCta;                                    // [4][8]
    float* fm = wl + kDecodeWarps * kHeadsPerCta;                                    // [8]
    float* fl = fm + kHeadsPerCta;                                                   // [8]
    int* flag = reinterpret_cast<int*>(fl + kHeadsPerCta);
    float* wscratch = fl + kHeadsPerCta + 4;  // [2][kDecodeMaxParts][8] + [8]
    uint32_t* cum = reinterpret_cast<uint32_t*>(wscratch + 2 * kDecodeMaxParts * kHeadsPerCta + kHeadsPerCta);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t ring = p.layer.ring;
    const uint32_t HY = p.layer.kv_heads * p.gchunks;
    const bool fused = p.k_new != nullptr;

    ITK_TRACE(p, 0);
    // A launch that must wait for its predecessor before anything else (the first of a step, behind the position
    // advance) lets its own dependents start only after that wait: they may then rely on what it waited for.
    if (p.pdl == 1) pdl_wait();
    if (p.pdl != 0) pdl_launch_dependents();
    uint32_t* abase = cum + kPlanAbase;
    uint32_t* sn_all = cum + kPlanSn;      // visible keys per sequence
    uint32_t* ss0_all = cum + kPlanSs0;    // storage row of its first visible key
    uint32_t* sslot_all = cum + kPlanSlot;
    uint32_t* mode = cum + kPlanMode;      // [0] 1 = cell-aligned plan, [1] steps of the loop done (device plan only)
    // Two lanes: the first half of the grid walks sequences [0, lane_split), the second half the rest; each half
    // plans its own sequences with its own CTAs, and everything below indexes the lane's sequences from zero.
    const bool two_lanes = p.gather.lanes == 2;
    const uint32_t G = two_lanes ? gridDim.x / 2 : gridDim.x;            // CTAs of this CTA's lane
    const uint32_t glane = (two_lanes && blockIdx.x >= G) ? 1u : 0u;  // which lane this CTA serves
    const uint32_t cta = blockIdx.x - glane * G;                          // this CTA's number inside its lane
    const uint32_t seq_base = glane ? p.gather.lane_split : 0u;           // lane's first sequence in the launch
    const uint32_t n_seqs = two_lanes ? (glane ? p.n_seqs - p.gather.lane_split : p.gather.lane_split) : p.n_seqs;
    const uint32_t* sn = sn_all + seq_base;
    const uint32_t* ss0 = ss0_all + seq_base;
    const uint32_t* sslot = sslot_all + seq_base;
    const bool planned = p.plan_dev != nullptr;
    if (planned) {
        // The plan of the current positions was worked out by the kernel that advanced them: one coalesced read.
        const uint32_t* src = p.plan_dev + (two_lanes ? 1u + glane : 0u) * kPlanWords;
        for (int i = tid; i < kPlanWords; i += kDecodeThreads) cum[i] = __ldcg(src + i);
        __syncthreads();
    } else {
        if (static_cast<uint32_t>(tid) < p.n_seqs) {  // one global read per sequence, all in flight together
            const SeqDesc sd = seq_of(p, tid);
            sn_all[tid] = sd.kv_hi - sd.kv_lo;
            ss0_all[tid] = sd.kv_lo % ring;
            sslot_all[tid] = sd.slot;
        }
        __syncthreads();
        if (tid == 0) {
            // cum[s] = tiles of all cells before (lane-local) sequence s
            uint32_t c = 0;
            for (uint32_t s = 0; s < n_seqs; ++s) {
                cum[s] = c;
                c += (sn[s] + kTileKeys - 1) / kTileKeys * HY;
            }
            cum[n_seqs] = c;
            // The cell-aligned plan, if it costs at most a sixteenth more tiles per CTA than equal runs would.
            const uint32_t total = c;
            const uint32_t per = p.seq_dev ? (total + G - 1) / G : p.tiles_per_cta;
            uint32_t worst;
            mode[0] = decode_aligned_plan(sn, n_seqs, HY, G, total, per, p.splits, abase, &worst) ? 1u : 0u;
        }
        __syncthreads();
    }
    const uint32_t total = cum[n_seqs];
    const bool aligned = mode[0] != 0u;
    const uint32_t per = p.seq_dev ? (total + G - 1) / G : p.tiles_per_cta;

    auto enter_seq = [&](TileCursor& c) {
        c.n = sn[c.seq];
        c.T = (c.n + kTileKeys - 1) / kTileKeys;
        c.s0 = ss0[c.seq];
        c.slot = sslot[c.seq];
    };
    auto advance = [&](TileCursor& c) {
        if (++c.tile == c.T) {
            c.tile = 0;
            if (++c.hy == HY) {
                c.hy = 0;
                if (++c.seq < n_seqs) enter_seq(c);
            }
        }
    };
    TileCursor lc;  // load cursor, runs STAGES - 1 tiles ahead of the compute cursor
    const DecodeRun my = decode_cta_run(aligned, cta, sn, cum, abase, n_seqs, HY, per);
    const uint32_t ntiles = my.ntiles;
    const uint32_t al_parts = my.parts, al_part = my.part;  // aligned plan: CTAs sharing this CTA's cell, and which
    if (ntiles != 0) {
        lc.seq = my.seq;
        enter_seq(lc);
        lc.hy = my.hy;
        lc.tile = my.tile;
    }
    if (ntiles == 0) {
        if (p.pdl >= 2) pdl_wait();
        return;
    }
    ITK_TRACE(p, 1);
    TileCursor cc = lc;

    const uint32_t smem_base = smem_u32(smem);
    auto slice_addr = [&](uint32_t stage, int which) -> uint32_t {
        return smem_base + ((stage * kDecodeWarps + warp) * 2 + which) * kSliceBytes;
    };
    // Issue this warp's loads for the tile under the load cursor: 16 rows x kRowBytes of K and of V.  Rows past
    // the sequence's end - and the row the kernel is about to write itself - are zero-filled, not read.
    auto load_tile = [&](const TileCursor& c, uint32_t stage) {
        const uint32_t kvh = c.hy / p.gchunks;
        const size_t stream = (static_cast<size_t>(c.slot) * p.layer.kv_heads + kvh) * ring * D;
        const __half* kb = static_cast<const __half*>(p.layer.k) + stream;
        const __half* vb = static_cast<const __half*>(p.layer.v) + stream;
        const uint32_t kbuf = slice_addr(stage, 0), vbuf = slice_addr(stage, 1);
        const uint32_t row0 = c.tile * kTileKeys + warp * 16;
        const uint32_t srow0 = c.s0 + row0 >= ring ? c.s0 + row0 - ring : c.s0 + row0;
        if (row0 + 16 <= c.n - (fused ? 1u : 0u) && srow0 + 16 <= ring) {
            // The whole slice is stored rows inside the ring (every slice but a sequence's last one or two and a
            // sliding layer's wrap): this lane's copies differ by constants only.
            const int r = lane / kChunksPerRow, ch = lane % kChunksPerRow;  // first of its rows, its 16-byte chunk
            constexpr int kRowStep = 32 / kChunksPerRow;                    // rows between two copies of a lane
            const size_t goff = static_cast<size_t>(srow0 + r) * D + ch * 8;
            const __half* kg = kb + goff;
            const __half* vg = vb + goff;
#pragma unroll
            for (int i = 0; i < D / 16; ++i) {
                const int row = r + i * kRowStep;
                const uint32_t soff = row * kRowBytes + ((ch ^ (row & 7)) << 4);
                cp_async16(kbuf + soff, kg + static_cast<size_t>(i) * kRowStep * D, 16u);
                cp_async16(vbuf + soff, vg + static_cast<size_t>(i) * kRowStep * D, 16u);
            }
            return;
        }
#pragma unroll
        for (int i = 0; i < D / 16; ++i) {
            const int cid = i * 32 + lane;
            const int row = cid / kChunksPerRow, ch = cid % kChunksPerRow;
            const uint32_t kr = row0 + row;  // key index inside the sequence's visible range
            const bool valid = kr < c.n && !(fused && kr == c.n - 1);
            uint32_t srow = c.s0 + kr;  // n <= ring, so one wrap at most
            if (srow >= ring) srow -= ring;
            const size_t goff = static_cast<size_t>(valid ? srow : 0u) * D + ch * 8;
            const uint32_t soff = row * kRowBytes + ((ch ^ (row & 7)) << 4);
            cp_async16(kbuf + soff, kb + goff, valid ? 16u : 0u);
            cp_async16(vbuf + soff, vb + goff, valid ? 16u : 0u);
        }
    };

    uint32_t issued = 0;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (issued < ntiles) {
            load_tile(lc, issued % STAGES);
            advance(lc);
            ++issued;
        }
        cp_async_commit();
    }

    // The cache rows streamed above do not depend on the previous kernel; the queries, the step's new row
    // and the merge scratch do.
    ITK_TRACE(p, 2);
    if (p.pdl == 2) pdl_wait();
    ITK_TRACE(p, 3);

    // A layer's inputs exist only once every rank's heads of the previous layer have been gathered: check that the
    // peers' previous launch has arrived here.  The wait is bounded; if it runs out the kernel records that and
    // carries on (its own arithmetic does not depend on the gathered data).
    // The counters are per sequence: a CTA waits only for the sequences it works on.  With two lanes they also
    // order everything this launch shares with the previous one (split scratch, tickets, accumulators of those
    // sequences' cells): the rank's own counter is among those polled, and a cell is announced only after its merge
    // has read the scratch and reset its ticket.
    if (p.gather.n_peers != 0 && p.gather.wait_prev != 0) {
        int gave_up = 0;
        if (p.gather.stagger_ns != 0 && glane == 1 && tid == 0) {
            // lane 1 of a step's first launch: its first tiles are in flight; hold back before touching them
            unsigned long long t0, t1;
            asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t0)::"memory");
            do {
                __nanosleep(200);
                asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t1)::"memory");
            } while (t1 - t0 < p.gather.stagger_ns);
        }
        // The sequences this CTA's run touches (one in the cell-aligned plan), one polling thread per (sequence,
        // source rank).
        uint32_t last_seq = my.seq;
        if (!aligned) {
            const uint64_t end = static_cast<uint64_t>(cta) * per + ntiles - 1;
            while (last_seq + 1 < n_seqs && cum[last_seq + 1] <= end) ++last_seq;
        }
        const uint32_t n_polls = (last_seq - my.seq + 1) * p.gather.n_peers;
        const uint32_t steps_done = planned ? mode[1] : seq_of(p, 0).q_pos0 - *p.gather.base_pos;
        const uint32_t target = (steps_done * p.gather.launches_per_step + p.gather.launches_before) * p.gather.cells_per_seq;
        for (uint32_t i = tid; i < n_polls; i += kDecodeThreads) {
            const unsigned int* arrived =
                p.gather.my_flags + (seq_base + my.seq + i / p.gather.n_peers) * kMaxPeers + i % p.gather.n_peers;
            uint32_t seen = 0, spins = 0;
            for (;;) {
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(seen) : "l"(arrived) : "memory");
                if (seen >= target) break;
                if (++spins > p.gather.poll_limit) {
                    atomicOr(p.gather.err, 1u);
                    gave_up = 1;
                    break;
                }
            }
        }
        // A launch that orders itself by the counters alone must not go on without them: when a wait ran out (this
        // rank's own counter may be among those still behind, held up by the previous launch's own waits), fall back
        // to the stream order - the previous launch, whose every wait is bounded too, completes first.
        if (__syncthreads_or(gave_up) != 0 && p.pdl == 3) pdl_wait();
        ITK_TRACE(p, 14);
    }

    uint32_t qa[KS][4];
    float o[NT][4];
    float m = -INFINITY, l = 0.f;
    const float sl = p.scale * kLog2e;
    const int mi = lane >> 3, rr = lane & 7;
    bool fresh = true;
    uint32_t head0 = 0, nh = 0, kvh = 0, gc = 0;

    for (uint32_t i = 0; i < ntiles; ++i) {
        if (fresh) {
            // Entering a cell: its query fragments (row g = head g's hi term, row g + 8 = its lo term) and a
            // clean softmax state.
            kvh = cc.hy / p.gchunks;
            gc = cc.hy % p.gchunks;
            head0 = kvh * p.group + gc * kHeadsPerCta;
            nh = min(static_cast<uint32_t>(kHeadsPerCta), p.group - gc * kHeadsPerCta);
            const float* qrow = p.q + (static_cast<size_t>(seq_base + cc.seq) * p.q_heads + head0 + g) * D;
            const bool live = static_cast<uint32_t>(g) < nh;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                float2 x0 = make_float2(0.f, 0.f), x1 = make_float2(0.f, 0.f);
                if (live) {
                    x0 = *reinterpret_cast<const float2*>(qrow + 16 * ks + 2 * t);
                    x1 = *reinterpret_cast<const float2*>(qrow + 16 * ks + 8 + 2 * t);
                }
                __half h0, l0, h1, l1;
                split_half(x0.x, h0, l0);
                split_half(x0.y, h1, l1);
                qa[ks][0] = pack_half2(h0, h1);
                qa[ks][1] = pack_half2(l0, l1);
                split_half(x1.x, h0, l0);
                split_half(x1.y, h1, l1);
                qa[ks][2] = pack_half2(h0, h1);
                qa[ks][3] = pack_half2(l0, l1);
            }
#pragma unroll
            for (int j = 0; j < NT; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
            m = -INFINITY;
            l = 0.f;
            fresh = false;
        }
        cp_async_wait<STAGES - 2>();
        __syncwarp();
        if (i == 0) ITK_TRACE(p, 4);
        if (issued < ntiles) {
            load_tile(lc, issued % STAGES);
            advance(lc);
            ++issued;
        }
        cp_async_commit();

        const uint32_t row0 = cc.tile * kTileKeys + warp * 16;
        if (row0 < cc.n) {  // else this warp's slice is past the sequence's end (last tile only)
            const uint32_t stage = i % STAGES;
            const uint32_t kbuf = slice_addr(stage, 0), vbuf = slice_addr(stage, 1);

            if (fused && cc.n - 1 >= row0 && cc.n - 1 < row0 + 16) {
                // This slice holds the step's new position: cast the f32 row, keep it in the cache and put it
                // where the zero-filled row sits in the staged tile.  Lanes 0..15 take K chunks, 16..31 V chunks.
                const uint32_t row = cc.n - 1 - row0;
                const int ch = lane & 15;
                const bool is_v = lane >= 16;
                if (ch < kChunksPerRow) {
                    const float* src = (is_v ? p.v_new : p.k_new) +
                                       (static_cast<size_t>(seq_base + cc.seq) * p.layer.kv_heads + kvh) * D + ch * 8;
                    const uint4 packed = pack8(*reinterpret_cast<const float4*>(src),
                                               *reinterpret_cast<const float4*>(src + 4));
                    const uint32_t soff = row * kRowBytes + ((ch ^ (row & 7)) << 4);
                    *reinterpret_cast<uint4*>(smem + ((is_v ? vbuf : kbuf) - smem_base) + soff) = packed;
                    if (gc == 0) {
                        uint32_t srow = cc.s0 + cc.n - 1;
                        if (srow >= ring) srow -= ring;
                        const size_t stream = (static_cast<size_t>(cc.slot) * p.layer.kv_heads + kvh) * ring * D;
                        __half* dst = static_cast<__half*>(const_cast<void*>(is_v ? p.layer.v : p.layer.k)) + stream +
                                      static_cast<size_t>(srow) * D + ch * 8;
                        *reinterpret_cast<uint4*>(dst) = packed;
                    }
                }
                __syncwarp();
            }

            // S(16 x 16 keys) = Q(16 x D) * K^T
            float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            {
                const int krow = ((mi >> 1) << 3) + rr;
                const uint32_t rbase = kbuf + krow * kRowBytes;
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    uint32_t b[4];
                    ldmatrix_x4(b, rbase + (((2 * ks + (mi & 1)) ^ rr) << 4));
                    mma_16816(s[0], qa[ks], b[0], b[1]);
                    mma_16816(s[1], qa[ks], b[2], b[3]);
                }
            }
            // hi + lo, scale, mask the tail, online softmax for head g.
            float sc[2][2];
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const uint32_t kr = row0 + 8 * j + 2 * t + e;
                    float v = (s[j][e] + s[j][e + 2]) * sl;
                    v = kr < cc.n ? v : -INFINITY;
                    sc[j][e] = v;
                    mx = fmaxf(mx, v);
                }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            // The running maximum moves only when the slice's maximum exceeds it by more than 2^kRescaleStep: until
            // then the stale one is used consistently for the weights (at most 2^kRescaleStep each), their sum and
            // the accumulator, so the result is exact and the accumulator's rescale - 4 * NT multiplies per thread -
            // is skipped for almost every tile after the first few.
            constexpr float kRescaleStep = 8.f;
            const bool grow = mx > m + kRescaleStep;  // also the first slice (m = -inf; mx is finite: key row0 is valid)
            const float m_new = grow ? mx : m;
            const bool rescale = __any_sync(0xffffffffu, grow);
            const float corr = grow ? fast_exp2(m - m_new) : 1.f;
            m = m_new;
            uint32_t pa[4];
            float psum = 0.f;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float p0 = fast_exp2(sc[j][0] - m_new), p1 = fast_exp2(sc[j][1] - m_new);
                psum += p0 + p1;
                __half h0, l0, h1, l1;
                split_half(p0, h0, l0);
                split_half(p1, h1, l1);
                pa[2 * j] = pack_half2(h0, h1);
                pa[2 * j + 1] = pack_half2(l0, l1);
            }
            l = l * corr + psum;
            if (rescale) {
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    o[j][0] *= corr;
                    o[j][1] *= corr;
                    o[j][2] *= corr;
                    o[j][3] *= corr;
                }
            }
            // O(16 x D) += P(16 x 16 keys) * V(16 keys x D)
            {
                const int vrow = ((mi & 1) << 3) + rr;
                const uint32_t rbase = vbuf + vrow * kRowBytes;
#pragma unroll
                for (int jp = 0; jp < NT / 2; ++jp) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, rbase + (((2 * jp + (mi >> 1)) ^ rr) << 4));
                    mma_16816(o[2 * jp], pa, b[0], b[1]);
                    mma_16816(o[2 * jp + 1], pa, b[2], b[3]);
                }
            }
        }

        if (cc.tile + 1 == cc.T || i + 1 == ntiles) {
            // This CTA's part of the cell is complete: merge the 4 warps through shared memory, then hand the
            // (m, l, o) part to the cell's merge.
            float lq = l + __shfl_xor_sync(0xffffffffu, l, 1);
            lq += __shfl_xor_sync(0xffffffffu, lq, 2);
            if (i + 1 == ntiles) ITK_TRACE(p, 5);
            __syncthreads();  // the previous cell's epilogue is over for every thread
            if (t == 0) {
                wm[warp * kHeadsPerCta + g] = m;
                wl[warp * kHeadsPerCta + g] = lq;
            }
            {
                // The stage this tile was read from is free until the next iteration refills it (the barrier above
                // means every warp is done with it; the loads in flight target the other stages): the four warps
                // exchange whole rows through it at once (row stride D + 8 floats: conflict-free both ways).
                constexpr int RS = D + 8;
                static_assert(kDecodeWarps * kHeadsPerCta * RS * 4 <= kDecodeWarps * 2 * kSliceBytes, "exchange rows exceed a stage");
                float* big = reinterpret_cast<float*>(smem + (i % STAGES) * (kDecodeWarps * 2 * kSliceBytes));  // [4][8][RS]
                float* dst = big + (warp * kHeadsPerCta + g) * RS + 2 * t;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                    *reinterpret_cast<float2*>(dst + 8 * nt) = make_float2(o[nt][0] + o[nt][2], o[nt][1] + o[nt][3]);
                __syncthreads();
                for (int idx = tid; idx < kHeadsPerCta * D; idx += kDecodeThreads) {
                    const int h = idx / D, c = idx % D;
                    float M = -INFINITY;
#pragma unroll
                    for (int w = 0; w < kDecodeWarps; ++w) M = fmaxf(M, wm[w * kHeadsPerCta + h]);
                    float O = 0.f;
                    if (M != -INFINITY) {
#pragma unroll
                        for (int w = 0; w < kDecodeWarps; ++w) {
                            const float mw = wm[w * kHeadsPerCta + h];
                            const float a = (mw == -INFINITY) ? 0.f : fast_exp2(mw - M);
                            O += a * big[(w * kHeadsPerCta + h) * RS + c];
                        }
                    }
                    fo[idx] = O;
                }
            }
            if (tid < kHeadsPerCta) {
                float M = -INFINITY;
#pragma unroll
                for (int w = 0; w < kDecodeWarps; ++w) M = fmaxf(M, wm[w * kHeadsPerCta + tid]);
                float L = 0.f;
                if (M != -INFINITY) {
#pragma unroll
                    for (int w = 0; w < kDecodeWarps; ++w) {
                        const float mw = wm[w * kHeadsPerCta + tid];
                        L += ((mw == -INFINITY) ? 0.f : fast_exp2(mw - M)) * wl[w * kHeadsPerCta + tid];
                    }
                }
                fm[tid] = M;
                fl[tid] = L;
            }
            __syncthreads();
            // which CTAs share this cell, and which of them this one is
            if (i + 1 == ntiles) ITK_TRACE(p, 13);
            uint32_t n_parts = al_parts, part = al_part;
            if (!aligned) decode_cell_parts(cta, cum[cc.seq] + cc.hy * cc.T, cc.T, per, &n_parts, &part);
            finish_unit<kDecodeThreads, kDecodeMaxParts>(p, seq_base + cc.seq, cc.hy, n_parts, part, head0, nh, D, fo, fm,
                                                         fl, flag, wscratch);
            fresh = true;
        }
        advance(cc);
    }
    cp_async_wait<0>();
    ITK_TRACE(p, 7);
    // A launch that never waited for its predecessor does so now, so that grids complete in stream order and
    // whatever follows the loop in the stream sees all of it done.
    if (p.pdl == 3) pdl_wait();
}

constexpr int kStages128 = 3;  // 96 KiB of pipeline per CTA at D = 128, two CTAs per SM
constexpr int kStages64 = 4;   // 64 KiB at D = 64

}  // namespace

bool decode_f16_supported(uint32_t head_dim, uint32_t rows) {
    return rows == 1 && (head_dim == 128 || head_dim == 64);
}

cudaError_t configure_decode_f16() {
    cudaError_t e = cudaFuncSetAttribute(decode_f16_kernel<128, kStages128>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(decode_smem_bytes<128, kStages128>()));
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(decode_f16_kernel<64, kStages64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(decode_smem_bytes<64, kStages64>()));
}

cudaError_t launch_decode_f16(AttnLaunch p, uint32_t cta_slots, uint32_t max_parts, cudaStream_t s,
                              uint64_t* launches, uint32_t* parts_used) {
    if (p.n_seqs == 0 || p.n_seqs > static_cast<uint32_t>(kMaxSeqsPerLaunch) || p.rows != 1) return cudaErrorInvalidValue;
    const uint32_t HY = p.layer.kv_heads * p.gchunks;
    uint64_t total = 0;
    uint32_t tmax = 0;
    for (uint32_t i = 0; i < p.n_seqs; ++i) {
        const uint32_t n = p.seq[i].kv_hi - p.seq[i].kv_lo;
        if (n == 0 || n > p.layer.ring) return cudaErrorInvalidValue;
        const uint32_t T = (n + kTileKeys - 1) / kTileKeys;
        total += static_cast<uint64_t>(T) * HY;
        if (T > tmax) tmax = T;
    }
    if (total == 0 || total > 0xffffffffull) return cudaErrorInvalidValue;
    if (max_parts > kDecodeMaxParts) max_parts = kDecodeMaxParts;
    if (max_parts < 2) return cudaErrorInvalidValue;  // a cut cell needs two partial slots; the caller sizes the batch
    if (cta_slots == 0) cta_slots = 1;
    uint64_t ctas = total < cta_slots ? total : cta_slots;
    uint32_t per = static_cast<uint32_t>((total + ctas - 1) / ctas);
    while (decode_parts_for(tmax, per) > max_parts) ++per;  // fewer, longer runs when the scratch bounds the sharing
    ctas = (total + per - 1) / per;
    p.tiles_per_cta = per;
    p.splits = decode_parts_for(tmax, per);
    if (parts_used) *parts_used = p.splits;
    const dim3 grid(static_cast<unsigned int>(ctas));
    if (p.layer.head_dim == 128) {
        decode_f16_kernel<128, kStages128><<<grid, kDecodeThreads, decode_smem_bytes<128, kStages128>(), s>>>(p);
    } else if (p.layer.head_dim == 64) {
        decode_f16_kernel<64, kStages64><<<grid, kDecodeThreads, decode_smem_bytes<64, kStages64>(), s>>>(p);
    } else {
        return cudaErrorInvalidValue;
    }
    if (launches) *launches += 1;
    return cudaGetLastError();
}

cudaError_t launch_decode_f16_resident(AttnLaunch p, uint32_t ctas, uint32_t parts_stride, cudaStream_t s,
                                       uint64_t* launches) {
    if (!p.seq_dev || p.n_seqs == 0 || p.n_seqs > static_cast<uint32_t>(kMaxSeqsPerLaunch) || p.rows != 1 || ctas == 0 ||
        parts_stride < 2 || parts_stride > kDecodeMaxParts)
        return cudaErrorInvalidValue;
    p.tiles_per_cta = 0;
    p.splits = parts_stride;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(kDecodeThreads);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.pdl != 0 ? 1 : 0;
    cudaError_t e;
    if (p.layer.head_dim == 128) {
        cfg.dynamicSmemBytes = decode_smem_bytes<128, kStages128>();
        e = cudaLaunchKernelEx(&cfg, decode_f16_kernel<128, kStages128>, p);
    } else if (p.layer.head_dim == 64) {
        cfg.dynamicSmemBytes = decode_smem_bytes<64, kStages64>();
        e = cudaLaunchKernelEx(&cfg, decode_f16_kernel<64, kStages64>, p);
    } else {
        return cudaErrorInvalidValue;
    }
    if (e != cudaSuccess) return e;
    if (launches) *launches += 1;
    return cudaGetLastError();
}

cudaError_t launch_advance_states(SeqState* states, uint32_t n, uint32_t add, const DecodePlanSpec& spec, uint32_t* plan_out,
                                  cudaStream_t s, uint64_t* launches) {
    if (!states || n == 0 || n > static_cast<uint32_t>(kMaxSeqsPerLaunch)) return cudaErrorInvalidValue;
    advance_states_kernel<<<1, kMaxSeqsPerLaunch, 0, s>>>(states, n, add, spec, plan_out);
    if (launches) *launches += 1;
    return cudaGetLastError();
}

}  // namespace itk

// ---------------------------------------------------------------------------
// Decode attention for callers that must not allocate.
//
// Who this is for: code that runs where a device allocation is off the table -
// a serving loop that took all of its memory at start-up and is forbidden to
// grow, a plugin invoked from inside somebody else's runtime that owns the
// allocator, a real-time path where cudaMalloc's implicit synchronisation is
// unacceptable, or a region of work being recorded for later replay, in which
// an allocation is an error.  Such a caller already holds its cache, its
// queries and its output buffer; the only thing the split-K decode kernel
// still needs is somewhere to park the per-split partial results.  Here that
// scratch is a fixed array baked into the library image, so the call performs
// no cudaMalloc, no cudaFree and no other allocating routine.
//
// Cost and limits of that choice:
//  - the array below (about 8.1 MiB) exists on every GPU that loads this
//    library, from load until the process exits, whether or not this entry
//    point is ever used;
//  - (sequences x KV heads x head chunks) x max(splits, 2) may not exceed
//    kNoAllocCellSplits, where `splits` (at most 64) bounds how many CTAs may
//    share one (sequence, head) key range; sequences may not exceed 64,
//    head_dim is 64 or 128; anything larger is refused with ITK_ERR_CAPACITY
//    and a message;
//  - all calls share the one array and it keeps whatever the previous call
//    left.  The arrival counters are the only part that must read zero at
//    launch; every call clears them on its stream first.  Two calls whose
//    kernels can overlap on the GPU (different streams, or different host
//    threads on different streams) trample each other's partials and
//    counters: serialise them.
//
// A symbol declared `__device__` is, in host code, only a handle for the
// runtime - not an address a kernel can dereference.  The device address is
// obtained once per device with cudaGetSymbolAddress while that device is
// current, and that pointer is what the kernel receives.  The first call on a
// device performs this set-up (and the kernel's shared-memory opt-in); make
// that first call before starting any stream capture.
// ---------------------------------------------------------------------------
namespace {

constexpr size_t kNoAllocCellSplits = 2048;  // (cell, split) partial slots
constexpr size_t kNoAllocPartO = kNoAllocCellSplits * itk::kHeadsPerCta * 128 * sizeof(float);  // 8 MiB
constexpr size_t kNoAllocPartMl = kNoAllocCellSplits * itk::kHeadsPerCta * 2 * sizeof(float);   // 128 KiB
constexpr size_t kNoAllocTickets = kNoAllocCellSplits * sizeof(unsigned int);                    // 8 KiB
constexpr int kNoAllocMaxDevices = 64;

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocPartO + kNoAllocPartMl + kNoAllocTickets];

// Device address of g_noalloc_scratch per device ordinal, resolved on first use under g_noalloc_mutex (two host
// threads may make their first call on a device at the same time).
void* g_noalloc_ptr[kNoAllocMaxDevices] = {};
std::mutex g_noalloc_mutex;

int noalloc_refuse(int code, char* text, size_t text_len, const char* fmt, unsigned long long a = 0,
                   unsigned long long b = 0) {
    if (text && text_len) snprintf(text, text_len, fmt, a, b);
    return code;
}

}  // namespace

extern "C" int itk_decode_attention_noalloc(const void* k_layer, const void* v_layer, uint32_t ring,
                                            uint32_t kv_heads, uint32_t q_heads, uint32_t head_dim, uint32_t n_seqs,
                                            const uint32_t* slots, const uint32_t* kv_len, const float* d_q,
                                            float* d_out, uint32_t splits, void* cuda_stream, char* error_text,
                                            size_t error_text_len) {
    using namespace itk;
    if (error_text && error_text_len) error_text[0] = '\0';
    if (!k_layer || !v_layer || !slots || !kv_len || !d_q || !d_out)
        return noalloc_refuse(101, error_text, error_text_len, "null pointer argument");
    // the kernel moves cache rows, queries and outputs as 16-byte vectors
    if (((reinterpret_cast<uintptr_t>(k_layer) | reinterpret_cast<uintptr_t>(v_layer) | reinterpret_cast<uintptr_t>(d_q) |
          reinterpret_cast<uintptr_t>(d_out)) & 15u) != 0)
        return noalloc_refuse(101, error_text, error_text_len, "k_layer, v_layer, d_q and d_out must be 16-byte aligned");
    if (kv_heads == 0 || q_heads == 0 || ring == 0)
        return noalloc_refuse(1, error_text, error_text_len, "kv_heads, q_heads and ring must be positive");
    if (q_heads % kv_heads != 0)
        return noalloc_refuse(7, error_text, error_text_len, "%llu query heads do not divide evenly across %llu KV heads",
                              q_heads, kv_heads);
    if (head_dim != 64 && head_dim != 128)
        return noalloc_refuse(102, error_text, error_text_len, "head_dim %llu is not supported here (64 or 128)", head_dim);
    if (n_seqs == 0) return 0;
    if (n_seqs > static_cast<uint32_t>(kMaxSeqsPerLaunch))
        return noalloc_refuse(102, error_text, error_text_len,
                              "%llu sequences exceed this entry point's maximum of %llu per call", n_seqs,
                              static_cast<unsigned long long>(kMaxSeqsPerLaunch));
    const uint32_t group = q_heads / kv_heads;
    const uint32_t gchunks = (group + kHeadsPerCta - 1) / kHeadsPerCta;
    const unsigned long long cells = static_cast<unsigned long long>(n_seqs) * kv_heads * gchunks;
    uint32_t n_max = 0;
    for (uint32_t i = 0; i < n_seqs; ++i) {
        if (kv_len[i] == 0)
            return noalloc_refuse(8, error_text, error_text_len, "sequence %llu has no visible keys", i);
        if (kv_len[i] > ring)
            return noalloc_refuse(102, error_text, error_text_len, "sequence %llu holds more keys than the ring of %llu",
                                  i, ring);
        if (kv_len[i] > n_max) n_max = kv_len[i];
    }
    if (cells > kNoAllocCellSplits)
        return noalloc_refuse(102, error_text, error_text_len,
                              "%llu (sequence, head) cells exceed the built-in scratch of %llu", cells,
                              static_cast<unsigned long long>(kNoAllocCellSplits));
    if (splits > kDecodeMaxParts)
        return noalloc_refuse(102, error_text, error_text_len, "%llu splits exceed the kernel's maximum of %llu", splits,
                              static_cast<unsigned long long>(kDecodeMaxParts));
    // `splits` bounds the CTAs that may share one key range, i.e. the partial slots a cell needs; a cell can
    // always be cut in two, so 1 reserves 2.
    unsigned long long parts = splits == 0 ? kNoAllocCellSplits / cells : (splits < 2 ? 2 : splits);
    if (parts > kDecodeMaxParts) parts = kDecodeMaxParts;
    if (parts < 2 || cells * parts > kNoAllocCellSplits)
        return noalloc_refuse(102, error_text, error_text_len,
                              "cells x splits = %llu exceeds the built-in scratch of %llu partial slots; lower `splits` "
                              "or pass fewer sequences",
                              cells * (parts < 2 ? 2 : parts), static_cast<unsigned long long>(kNoAllocCellSplits));

    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices)
        return noalloc_refuse(100, error_text, error_text_len, "no usable current CUDA device");
    int sm_count = 0;
    e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess || sm_count <= 0) sm_count = 148;
    unsigned char* base = nullptr;
    {
        std::lock_guard<std::mutex> guard(g_noalloc_mutex);
        if (!g_noalloc_ptr[dev]) {
            // One-time set-up for this device: resolve the array's device address and opt the kernel in to its
            // dynamic shared memory size.  Neither allocates.
            void* ptr = nullptr;
            e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
            if (e != cudaSuccess || !ptr) {
                if (error_text && error_text_len)
                    snprintf(error_text, error_text_len, "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
                return 100;
            }
            e = configure_decode_f16();
            if (e != cudaSuccess) {
                if (error_text && error_text_len)
                    snprintf(error_text, error_text_len, "kernel attribute setup failed: %s", cudaGetErrorString(e));
                return 100;
            }
            g_noalloc_ptr[dev] = ptr;
        }
        base = static_cast<unsigned char*>(g_noalloc_ptr[dev]);
    }
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);

    AttnLaunch p{};
    p.layer.k = k_layer;
    p.layer.v = v_layer;
    p.layer.ring = ring;
    p.layer.window = 0;
    p.layer.kv_heads = kv_heads;
    p.layer.head_dim = head_dim;
    p.q = d_q;
    p.out = d_out;
    p.part_o = reinterpret_cast<float*>(base);
    p.part_ml = reinterpret_cast<float*>(base + kNoAllocPartO);
    p.tickets = reinterpret_cast<unsigned int*>(base + kNoAllocPartO + kNoAllocPartMl);
    p.q_heads = q_heads;
    p.group = group;
    p.gchunks = gchunks;
    p.rows = 1;
    p.n_seqs = n_seqs;
    p.scale = 1.0f / sqrtf(static_cast<float>(head_dim));
    for (uint32_t i = 0; i < n_seqs; ++i) p.seq[i] = SeqDesc{slots[i], kv_len[i] - 1, 0, kv_len[i]};
    // The arrival counters must read zero when the kernel starts, whatever an earlier (possibly failed)
    // call left behind.
    e = cudaMemsetAsync(p.tickets, 0, cells * sizeof(unsigned int), stream);
    if (e == cudaSuccess)
        e = launch_decode_f16(p, 2u * static_cast<uint32_t>(sm_count), static_cast<uint32_t>(parts), stream, nullptr, nullptr);
    if (e != cudaSuccess) {
        if (error_text && error_text_len)
            snprintf(error_text, error_text_len, "decode attention launch failed: %s", cudaGetErrorString(e));
        return 100;
    }
    return 0;
}
