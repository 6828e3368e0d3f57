// Multi-row causal GQA attention over the f16 resident cache on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory): the speculative verify block and chunked-prefill rows.
//
// Same contract as the mma.sync kernel next door (attn_verify_f16.cu): gqa_attention with several queries
// (crates/attention/src/attention.rs:160-213) after the block's rows were appended
// (crates/arch-llama/src/model.rs:212-228); row r sits at position q_pos0 + r and sees keys kp <= its
// position (kp > position - window on a sliding layer).
//
// One CTA (128 threads = the 128 lanes of tensor memory) owns a (sequence, KV head, block of row-head
// pairs, key split).  Per 64-key tile:
//   S = [q_hi | q_lo] * [K | K]^T   16 MMAs of M128 N64 K16.  The f32 query is carried as two f16 terms
//                                   laid side by side along the contraction dimension, so one accumulator
//                                   row receives q_hi.k + q_lo.k = the f32-grade score; the K tile is
//                                   simply addressed twice.
//   softmax                         thread i reads row i of S from tensor memory (tcgen05.ld), applies
//                                   scale and the causal / window mask, keeps a running maximum and sum,
//                                   and writes the weights as f16 hi and lo terms to a swizzled
//                                   shared-memory tile P = [p_hi | p_lo].
//   O += P * [V ; V]                8 MMAs of M128 N128 K16 accumulating in tensor memory; V is consumed
//                                   in place as an MN-major operand (no transpose in shared memory).
// The accumulator is rescaled in tensor memory only when a row's maximum grows by more than 2^8 (the
// stale maximum is used consistently for weights and sum until then, so the result is exact).
//
// A verify block has few pairs (7 rows x 4 heads = 28 in the speculative configuration) while the MMA has
// 128 rows, so the pairs are replicated R = 4, 2 or 1 times over the lane quadrants and replica r takes
// columns [r*64/R, (r+1)*64/R) of every tile: the R replicas are R interleaved key subsets with their own
// running maxima, merged at the end like key splits.  The tensor-core cost is the same, the per-thread
// softmax work drops by R.
//
// K/V tiles arrive by cp.async (16-byte, zero-filled past the split's range) in a 4-deep ring; all waits on
// the tensor core go through one mbarrier with a clock-bounded wait that raises AttnLaunch::status instead
// of spinning forever.
//
// Bound: HBM (the block's K/V stream, read once per pair block).
#include "attn_common.cuh"
#include "tcgen05.cuh"

namespace itk {

namespace {

constexpr int kTcThreads = 128;
constexpr int kTcTile = 64;   // keys per tile
constexpr int kTcStages = 4;  // K/V ring depth
constexpr int kTcD = 128;     // head dimension this kernel is built for
constexpr uint32_t kPanelQ = 128 * 128;  // bytes of a [128 rows][64 halfs] panel
constexpr uint32_t kPanelKV = 64 * 128;  // bytes of a [64 keys][64 halfs] panel
constexpr uint32_t kQBytes = 4 * kPanelQ;       // q_hi d0-63, q_hi d64-127, q_lo d0-63, q_lo d64-127
constexpr uint32_t kPBytes = 2 * kPanelQ;       // p_hi, p_lo over the tile's 64 keys
constexpr uint32_t kStageBytes = 4 * kPanelKV;  // K (2 panels) then V (2 panels)
constexpr uint32_t kTcSmemUsed = kQBytes + kPBytes + kTcStages * kStageBytes + 64;
constexpr uint32_t kTcSmemBytes = kTcSmemUsed + 1024;  // slack to align the base to 1024 bytes
constexpr uint32_t kTmemCols = 256;                    // S in columns 0-63, O in columns 128-255
constexpr uint32_t kTmemO = 128;
constexpr long long kWaitClocks = 2000000000ll;  // about a second
constexpr float kRescaleStep = 8.f;              // log2 of the growth of a row maximum that triggers a rescale
constexpr int kStageRowFloats = kTcD + 4;        // epilogue staging row (padded against bank conflicts)

__device__ __forceinline__ uint32_t panel_off(uint32_t row, uint32_t chunk) {
    return row * 128 + ((chunk ^ (row & 7)) << 4);
}

// CN = columns of a 64-key tile each thread handles = 64 / replicas; pairs per CTA = 2 * CN.
template <int CN>
__global__ void __launch_bounds__(kTcThreads, 1) verify_tc_kernel(const __grid_constant__ AttnLaunch p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    constexpr int R = kTcTile / CN;
    constexpr int PC = kTcThreads / R;
    constexpr int D = kTcD;

    unsigned char* smem =
        reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const uint32_t sbase = smem_u32(smem);
    const uint32_t qbuf = sbase, pbuf = sbase + kQBytes, kvbuf = pbuf + kPBytes;
    const uint32_t bar = kvbuf + kTcStages * kStageBytes, slot = bar + 8;
    volatile uint32_t* slot_ptr = reinterpret_cast<volatile uint32_t*>(smem + (slot - sbase));
    int* s_flag = reinterpret_cast<int*>(smem + (slot - sbase) + 4);

    const int tid = threadIdx.x, warp = tid >> 5;
    const uint32_t split = blockIdx.x, seq = blockIdx.z;
    const uint32_t gheads = min(p.group, static_cast<uint32_t>(kHeadsPerCta));
    const uint32_t pchunks = (p.rows * gheads + PC - 1) / PC;
    const uint32_t hy = blockIdx.y / pchunks, pc = blockIdx.y % pchunks;
    const SeqDesc sd = p.seq[seq];
    const uint32_t kvh = hy / p.gchunks, gc = hy % p.gchunks;
    const uint32_t head0 = kvh * p.group + gc * kHeadsPerCta;
    const uint32_t nh = min(static_cast<uint32_t>(kHeadsPerCta), p.group - gc * kHeadsPerCta);
    const uint32_t n_pairs = p.rows * nh;
    const uint32_t ring = p.layer.ring, window = p.layer.window;

    // This CTA's slice [k0, k1) of the positions [kv_lo, kv_hi) the block can see.
    const uint32_t n = sd.kv_hi - sd.kv_lo;
    uint32_t chunk = (n + p.splits - 1) / p.splits;
    chunk = (chunk + kTcTile - 1) / kTcTile * kTcTile;
    const uint32_t k0 = min(n, split * chunk);
    const uint32_t k1 = min(n, k0 + chunk);
    const uint32_t span = k1 - k0;
    const uint32_t ntiles = (span + kTcTile - 1) / kTcTile;
    const uint32_t s0 = (sd.kv_lo + k0) % ring;
    const size_t stream = (static_cast<size_t>(sd.slot) * p.layer.kv_heads + kvh) * ring * D;
    const __half* kbase = static_cast<const __half*>(p.layer.k) + stream;
    const __half* vbase = static_cast<const __half*>(p.layer.v) + stream;

    // Thread tid = tensor-memory lane tid = replica `rep` of pair `lp`; it handles tile columns [col0, col0 + CN).
    const uint32_t lp = tid % PC, rep = tid / PC, col0 = rep * CN;
    const uint32_t pair = pc * PC + lp;
    const bool live = pair < n_pairs;
    const uint32_t prow = live ? pair / nh : 0, phead = live ? pair % nh : 0;
    const uint32_t ppos = sd.q_pos0 + prow;
    uint32_t abs_lo = sd.kv_lo;
    if (window != 0 && ppos + 1 > window) abs_lo = max(abs_lo, ppos + 1 - window);
    const int64_t rel0 = static_cast<int64_t>(sd.kv_lo) + k0;
    const int64_t vis_lo = live ? static_cast<int64_t>(abs_lo) - rel0 : 0;
    const int64_t vis_hi = live ? static_cast<int64_t>(ppos) + 1 - rel0 : 0;

    auto load_tile = [&](uint32_t tile) {
        const uint32_t kst = kvbuf + (tile % kTcStages) * kStageBytes, vst = kst + 2 * kPanelKV;
        const uint32_t row0 = tile * kTcTile;
#pragma unroll
        for (int i = 0; i < kTcTile * (D / 8) / kTcThreads; ++i) {
            const int cid = i * kTcThreads + tid;
            const uint32_t row = cid / (D / 8), c = cid % (D / 8);
            const uint32_t kr = row0 + row;
            const bool valid = kr < span;
            uint32_t srow = s0 + kr;
            if (srow >= ring) srow -= ring;
            const size_t goff = static_cast<size_t>(valid ? srow : 0u) * D + c * 8;
            const uint32_t soff = (c / 8) * kPanelKV + panel_off(row, c % 8);
            cp_async16(kst + soff, kbase + goff, valid ? 16u : 0u);
            cp_async16(vst + soff, vbase + goff, valid ? 16u : 0u);
        }
    };

    // The K/V stream starts first; everything else is set up underneath it.
#pragma unroll
    for (int s = 0; s < kTcStages - 1; ++s) {
        if (static_cast<uint32_t>(s) < ntiles) load_tile(s);
        cp_async_commit();
    }

    if (tid == 0) {
        tc::mbar_init(bar, 1);
        tc::fence_mbar_init();
    }
    __syncwarp();
    if (warp == 0) {
        tc::tmem_alloc(slot, kTmemCols);
        tc::tmem_relinquish();
    }
    {   // Row tid of the query tile: hi and lo f16 terms of the pair's f32 query; row tid of P starts as zeros.
        const float* qrow = p.q + ((static_cast<size_t>(seq) * p.rows + prow) * p.q_heads + head0 + phead) * D;
#pragma unroll 4
        for (int c = 0; c < D / 8; ++c) {
            float x[8];
            if (live) {
                const float4 a = *reinterpret_cast<const float4*>(qrow + 8 * c);
                const float4 b = *reinterpret_cast<const float4*>(qrow + 8 * c + 4);
                x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
                x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) x[e] = 0.f;
            }
            uint32_t hi[4], lo[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                __half h0, l0, h1, l1;
                split_half(x[2 * e], h0, l0);
                split_half(x[2 * e + 1], h1, l1);
                hi[e] = pack_half2(h0, h1);
                lo[e] = pack_half2(l0, l1);
            }
            const uint32_t off = (c / 8) * kPanelQ + panel_off(tid, c % 8);
            *reinterpret_cast<uint4*>(smem + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
            *reinterpret_cast<uint4*>(smem + 2 * kPanelQ + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        }
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            *reinterpret_cast<uint4*>(smem + kQBytes + panel_off(tid, c)) = make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4*>(smem + kQBytes + kPanelQ + panel_off(tid, c)) = make_uint4(0u, 0u, 0u, 0u);
        }
    }


    cp_async_wait<kTcStages - 2>();  // tile 0 has landed (tiles 1 and 2 may still be in flight)
    tc::fence_proxy_async();
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = *slot_ptr;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t tS = tmem + lane_base + col0;
    const uint32_t tO = tmem + lane_base + kTmemO;

    constexpr uint32_t kIdescS = tc::instr_desc_f16(128, kTcTile, false);
    constexpr uint32_t kIdescO = tc::instr_desc_f16(128, D, true);
    auto issue_qk = [&](uint32_t tile) {  // S = [q_hi | q_lo] * [K | K]^T, 16 halfs of the contraction per MMA
        const uint32_t kst = kvbuf + (tile % kTcStages) * kStageBytes;
#pragma unroll
        for (int ks = 0; ks < 16; ++ks)
            tc::mma_f16_ss(tmem, tc::smem_desc(qbuf + (ks / 4) * kPanelQ + (ks % 4) * 32, 16, 1024),
                           tc::smem_desc(kst + ((ks % 8) / 4) * kPanelKV + (ks % 4) * 32, 16, 1024), kIdescS,
                           ks > 0 ? 1u : 0u);
    };
    auto issue_pv = [&](uint32_t tile) {  // O (+)= [p_hi | p_lo] * [V ; V], 16 keys per MMA
        const uint32_t vst = kvbuf + (tile % kTcStages) * kStageBytes + 2 * kPanelKV;
#pragma unroll
        for (int j = 0; j < 8; ++j)
            tc::mma_f16_ss(tmem + kTmemO, tc::smem_desc(pbuf + (j / 4) * kPanelQ + (j % 4) * 32, 16, 1024),
                           tc::smem_desc(vst + (j % 4) * 2048, kPanelKV, 1024), kIdescO,
                           (tile > 0 || j > 0) ? 1u : 0u);
    };
    if (tid == 0 && ntiles > 0) {
        issue_qk(0);
        tc::mma_commit(bar);
    }
    __syncwarp();

    float m_use = -INFINITY, l = 0.f;  // the maximum the weights are taken against (log2 domain), their sum
    const float sl = p.scale * kLog2e;
    uint32_t phase = 0;
    bool failed = false;
    for (uint32_t tile = 0; tile < ntiles; ++tile) {
        // S of this tile is complete, and so is every MMA issued before it: the stage of tile - 1 is free.
        const bool ok = tc::mbar_wait_bounded(bar, phase, kWaitClocks);
        phase ^= 1u;
        tc::fence_after_sync();
        if (tile + kTcStages - 1 < ntiles) load_tile(tile + kTcStages - 1);
        cp_async_commit();

        uint32_t sr[CN / 16][16];
#pragma unroll
        for (int b = 0; b < CN / 16; ++b) tc::tmem_ld16(tS + 16 * b, sr[b]);
        tc::tmem_wait_ld();
        const int64_t kr0 = static_cast<int64_t>(tile) * kTcTile + col0;
        float mx = -INFINITY;
#pragma unroll
        for (int b = 0; b < CN / 16; ++b)
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int64_t kr = kr0 + 16 * b + j;
                float v = __uint_as_float(sr[b][j]) * sl;
                v = (kr >= vis_lo && kr < vis_hi) ? v : -INFINITY;
                sr[b][j] = __float_as_uint(v);
                mx = fmaxf(mx, v);
            }
        const bool grow = mx > m_use + kRescaleStep;  // also the first visible key of the row (m_use = -inf)
        const float m_new = grow ? mx : m_use;
        const float corr = grow ? (m_use == -INFINITY ? 0.f : fast_exp2(m_use - m_new)) : 1.f;
        if (tile > 0 && __ballot_sync(0xffffffffu, grow) != 0u) {
            // Some row of this warp moves its maximum: rescale the warp's 32 accumulator rows in tensor memory
            // (every MMA into them has completed, see the wait above).
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 16) {
                uint32_t r[16];
                tc::tmem_ld16(tO + c0, r);
                tc::tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * corr);
                tc::tmem_st16(tO + c0, r);
            }
            tc::tmem_wait_st();
        }
        l *= corr;
        m_use = m_new;
        const float m_safe = (m_use == -INFINITY) ? 0.f : m_use;
#pragma unroll
        for (int jc = 0; jc < CN / 8; ++jc) {
            uint32_t hi[4], lo[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float p0 = fast_exp2(__uint_as_float(sr[jc / 2][(jc % 2) * 8 + 2 * e]) - m_safe);
                const float p1 = fast_exp2(__uint_as_float(sr[jc / 2][(jc % 2) * 8 + 2 * e + 1]) - m_safe);
                l += p0 + p1;
                __half h0, l0, h1, l1;
                split_half(p0, h0, l0);
                split_half(p1, h1, l1);
                hi[e] = pack_half2(h0, h1);
                lo[e] = pack_half2(l0, l1);
            }
            const uint32_t off = panel_off(tid, col0 / 8 + jc);
            *reinterpret_cast<uint4*>(smem + kQBytes + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
            *reinterpret_cast<uint4*>(smem + kQBytes + kPanelQ + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        }
        cp_async_wait<kTcStages - 2>();  // the next tile has landed
        tc::fence_proxy_async();
        tc::fence_before_sync();
        if (__syncthreads_or(ok ? 0 : 1)) {  // a wait ran out somewhere: every thread leaves together
            failed = true;
            break;
        }
        if (tid == 0) {
            tc::fence_after_sync();
            issue_pv(tile);
            if (tile + 1 < ntiles) issue_qk(tile + 1);  // S was read into registers by everyone before the barrier
            tc::mma_commit(bar);
        }
        __syncwarp();
    }
    if (!failed && ntiles > 0) {
        const bool ok = tc::mbar_wait_bounded(bar, phase, kWaitClocks);  // the last P * V
        if (__syncthreads_or(ok ? 0 : 1)) failed = true;
    }
    cp_async_wait<0>();
    tc::fence_after_sync();
    __syncthreads();  // nothing is in flight into shared memory any more: the K/V ring becomes staging space

    if (failed) {
        if (tid == 0 && p.status) atomicOr(p.status, 1u);
    } else {
        float* stage_o = reinterpret_cast<float*>(smem + kQBytes + kPBytes);  // [128][D + 4]
        float* stage_ml = stage_o + kTcThreads * kStageRowFloats;             // [128][2]
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 16) {
            uint32_t r[16];
            if (ntiles > 0) {
                tc::tmem_ld16(tO + c0, r);
                tc::tmem_wait_ld();
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) r[j] = 0u;
            }
            float4* dst = reinterpret_cast<float4*>(stage_o + tid * kStageRowFloats + c0);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                dst[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                     __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
        }
        stage_ml[2 * tid] = m_use;
        stage_ml[2 * tid + 1] = l;
        tc::fence_before_sync();
        __syncthreads();

        // Merge the R replicas of pair lp; this thread produces channels [rep * DW, (rep + 1) * DW).
        constexpr int DW = D / R;
        float M = -INFINITY, L = 0.f;
        float w[R];
#pragma unroll
        for (int r = 0; r < R; ++r) M = fmaxf(M, stage_ml[2 * (r * PC + lp)]);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float ms = stage_ml[2 * (r * PC + lp)];
            w[r] = (ms == -INFINITY) ? 0.f : fast_exp2(ms - M);
            L += w[r] * stage_ml[2 * (r * PC + lp) + 1];
        }
        float4 acc[DW / 4];
#pragma unroll
        for (int i = 0; i < DW / 4; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float4* src = reinterpret_cast<const float4*>(stage_o + (r * PC + lp) * kStageRowFloats + rep * DW);
#pragma unroll
            for (int i = 0; i < DW / 4; ++i) {
                const float4 v = src[i];
                acc[i].x += w[r] * v.x;
                acc[i].y += w[r] * v.y;
                acc[i].z += w[r] * v.z;
                acc[i].w += w[r] * v.w;
            }
        }

        const uint32_t HYP = p.layer.kv_heads * p.gchunks * pchunks;
        const size_t cell = static_cast<size_t>(seq) * HYP + blockIdx.y;
        if (p.splits == 1) {
            if (live) {
                float4* out4 = reinterpret_cast<float4*>(
                    p.out + ((static_cast<size_t>(seq) * p.rows + prow) * p.q_heads + head0 + phead) * D + rep * DW);
                const float inv = 1.f / L;
#pragma unroll
                for (int i = 0; i < DW / 4; ++i)
                    out4[i] = make_float4(acc[i].x * inv, acc[i].y * inv, acc[i].z * inv, acc[i].w * inv);
            }
        } else {
            if (live) {
                float4* po =
                    reinterpret_cast<float4*>(p.part_o + ((cell * p.splits + split) * PC + lp) * D + rep * DW);
#pragma unroll
                for (int i = 0; i < DW / 4; ++i) po[i] = acc[i];
                if (rep == 0) {
                    float* pml = p.part_ml + ((cell * p.splits + split) * PC + lp) * 2;
                    pml[0] = M;
                    pml[1] = L;
                }
            }
            __threadfence();
            __syncthreads();
            if (tid == 0) {
                const unsigned int ticket = atomicAdd(p.tickets + cell, 1u);
                *s_flag = (ticket == p.splits - 1) ? 1 : 0;
            }
            __syncthreads();
            if (*s_flag != 0) {  // the last CTA of the cell merges every split
                __threadfence();
                const float* all_o = p.part_o + cell * p.splits * PC * D;
                const float* all_ml = p.part_ml + cell * p.splits * PC * 2;
                const uint32_t cta_pairs = min(static_cast<uint32_t>(PC), n_pairs - pc * PC);
                for (uint32_t idx = tid; idx < cta_pairs * (D / 4); idx += kTcThreads) {
                    const uint32_t q = idx / (D / 4), d4 = idx % (D / 4);
                    float Mx = -INFINITY;
                    for (uint32_t s = 0; s < p.splits; ++s)
                        Mx = fmaxf(Mx, __ldcg(all_ml + (static_cast<size_t>(s) * PC + q) * 2));
                    float Ls = 0.f;
                    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (uint32_t s = 0; s < p.splits; ++s) {
                        const float ms = __ldcg(all_ml + (static_cast<size_t>(s) * PC + q) * 2);
                        if (ms == -INFINITY) continue;
                        const float ws = fast_exp2(ms - Mx);
                        Ls += ws * __ldcg(all_ml + (static_cast<size_t>(s) * PC + q) * 2 + 1);
                        const float4 v =
                            __ldcg(reinterpret_cast<const float4*>(all_o + (static_cast<size_t>(s) * PC + q) * D) + d4);
                        o.x += ws * v.x;
                        o.y += ws * v.y;
                        o.z += ws * v.z;
                        o.w += ws * v.w;
                    }
                    const uint32_t gp = pc * PC + q;
                    const uint32_t r = gp / nh, h = gp % nh;
                    const float inv = 1.f / Ls;
                    reinterpret_cast<float4*>(p.out + ((static_cast<size_t>(seq) * p.rows + r) * p.q_heads + head0 + h) *
                                                          D)[d4] = make_float4(o.x * inv, o.y * inv, o.z * inv, o.w * inv);
                }
                if (tid == 0) p.tickets[cell] = 0u;
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tmem, kTmemCols);
}

uint32_t tc_columns_for(uint32_t rows, uint32_t group) {
    const uint32_t pairs = rows * (group < static_cast<uint32_t>(kHeadsPerCta) ? group : kHeadsPerCta);
    return pairs <= 32 ? 16u : pairs <= 64 ? 32u : 64u;
}

}  // namespace

bool verify_tc_supported(uint32_t head_dim, uint32_t rows, uint32_t group) {
    (void)group;
    return rows >= 2 && rows <= 64 && head_dim == static_cast<uint32_t>(kTcD);
}

uint32_t verify_tc_pairs_per_cta(uint32_t rows, uint32_t group) { return 2 * tc_columns_for(rows, group); }

uint32_t verify_tc_pair_chunks(uint32_t rows, uint32_t group) {
    const uint32_t nh = group < static_cast<uint32_t>(kHeadsPerCta) ? group : kHeadsPerCta;
    const uint32_t pc = verify_tc_pairs_per_cta(rows, group);
    return (rows * nh + pc - 1) / pc;
}

cudaError_t configure_verify_tc() {
    cudaError_t e = cudaFuncSetAttribute(verify_tc_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(kTcSmemBytes));
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(verify_tc_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(kTcSmemBytes));
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(verify_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(kTcSmemBytes));
    return e;
}

cudaError_t launch_verify_tc(const AttnLaunch& p, cudaStream_t s, uint64_t* launches) {
    if (p.layer.head_dim != static_cast<uint32_t>(kTcD)) return cudaErrorInvalidValue;
    const uint32_t pchunks = verify_tc_pair_chunks(p.rows, p.group);
    const dim3 grid(p.splits, p.layer.kv_heads * p.gchunks * pchunks, p.n_seqs);
    switch (tc_columns_for(p.rows, p.group)) {
        case 16: verify_tc_kernel<16><<<grid, kTcThreads, kTcSmemBytes, s>>>(p); break;
        case 32: verify_tc_kernel<32><<<grid, kTcThreads, kTcSmemBytes, s>>>(p); break;
        default: verify_tc_kernel<64><<<grid, kTcThreads, kTcSmemBytes, s>>>(p); break;
    }
    if (launches) *launches += 1;
    return cudaGetLastError();
}

}  // namespace itk
