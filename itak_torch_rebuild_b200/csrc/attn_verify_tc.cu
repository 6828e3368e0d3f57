// Multi-row causal GQA attention over the f16 resident cache on the 5th-generation tensor cores
// (tcgen05.mma, operands and accumulators in tensor memory): the speculative verify block and
// chunked-prefill rows.
//
// Same contract as the mma.sync kernel next door (attn_verify_f16.cu): gqa_attention with several queries
// (crates/attention/src/attention.rs:160-213) after the block's rows were appended
// (crates/arch-llama/src/model.rs:212-228); row r sits at position q_pos0 + r and sees keys kp <= its
// position (kp > position - window on a sliding layer).
//
// One CTA owns a (sequence, KV head, block of row-head pairs, key split); a call of any number of rows is cut into
// such blocks, each streaming the keys up to its own last row.  Only the K/V stream lives in shared
// memory; everything else sits in the 512 columns of tensor memory:
//
//   columns   0-127  Q      row i: an f32 query as two f16 terms, [q_hi | q_lo], two halfs per column
//   columns 128-255  S      scores of a 128-key tile (f32)
//   columns 256-383  P0,P1  softmax weights of a tile as f16 (two keys per column), double buffered
//   columns 384-511  O      the output accumulator (f32)
//
// Per 128-key tile:
//   S = [q_hi | q_lo] * [K | K]^T   16 MMAs of M128 N128 K16, A from tensor memory, B = the K tile in shared
//                                   memory addressed twice: one accumulator row receives q_hi.k + q_lo.k,
//                                   the f32-grade score.
//   softmax                         thread i reads row i of S (tcgen05.ld), applies scale and the causal /
//                                   window mask, keeps a running maximum and sum, and stores the weights as
//                                   f16 hi and lo terms into P (tcgen05.st).
//   O += P * V                      8 MMAs of M128 N128 K16, A from tensor memory, B = the V tile consumed in
//                                   place as an MN-major operand (no transpose in shared memory).  The hi and
//                                   lo f16 terms of the weights sit in different ROWS (see below), so their
//                                   products are added once, at the end, instead of doubling the MMAs.
// One thread can issue a tcgen05.mma about every 64 clocks whatever its N up to 128 (measured), which is
// also what an N = 128 MMA takes to execute; hence 128-key tiles: the same 32 issues cover twice the keys of
// a 64-key tile.  S is a single buffer: the softmax threads copy their scores to registers at once and release
// it, so the next tile's scores are computed underneath the softmax.
// The accumulator is rescaled in tensor memory only when a row's maximum grows by more than 2^8 (the stale
// maximum is used consistently for weights and sum until then, so the result is exact).
//
// The CTA is warp-specialised (8 warps):
//   warps 0-3  softmax: thread i owns tensor-memory lane i;
//   warp  4    issues the score MMAs (one lane) - issuing blocks while the tensor queue is full, so it must not
//              sit in a warp that also has softmax work - and owns the tensor-memory allocation;
//   warp  7    issues the P * V MMAs (one lane): with one issuer for both kinds, its waits and fences between a
//              tile's value product and the next tile's scores left the tensor core idle a quarter of the time;
//   warp 5 streams K tiles, warp 6 V tiles, with 16-byte cp.async (zero-filled past the split's range)
//              into rings of three (K) and four (V) 32 KiB stages - a K stage is free again as soon as its
//              scores are complete, a V stage only after P * V; each copy batch reports its own completion to
//              the stage's barrier.
// With AttnLaunch::k_new set the loaders also do the block's append: tiles that hold the block's own rows take
// them from the caller's f32 rows (converted with the append kernel's function) instead of the cache, and one CTA
// per (sequence, KV head) stores them to the cache, which saves the separate append launch.
// They meet only through mbarriers: full/empty per stage, scores complete, scores consumed, weights stored, and
// one that counts completed P * V products.  Every wait is clock-bounded; a wait that runs out raises
// AttnLaunch::status and every role leaves its loop instead of spinning forever.
//
// A verify block has few pairs (7 rows x 4 heads = 28 in the speculative configuration) while the MMA has
// 128 rows.  A CTA takes PC = 32 or 64 pairs and gives each R = 128 / PC rows: row (r, pair) with r = 2 * kh + x
// handles key columns [kh * 128 / KH, (kh + 1) * 128 / KH) of every tile (KH = R / 2 interleaved key subsets
// with their own running maxima) and stores the hi (x = 0) or lo (x = 1) f16 term of its weights; the other
// columns of its P row stay zero.  All R rows of a pair hold the same query, so their scores are identical;
// their R partial outputs are merged at the end like key splits.
//
// Bound: HBM (the block's K/V stream, read once per pair block): a tile's 24 MMAs take about 1550 clocks
// against about 2500-2900 clocks of HBM time per 64 KiB tile and SM.
#include "attn_common.cuh"
#include "kv_convert.cuh"
#include "tcgen05.cuh"

namespace itk {

namespace {

constexpr int kTcSoftmaxThreads = 128;
constexpr int kTcLoaderThreads = 32;  // per stream (K, V)
constexpr int kTcThreads = kTcSoftmaxThreads + 32 + 2 * kTcLoaderThreads + 32;
constexpr int kTcMmaWarp = 4;  // issues the score MMAs and owns the tensor-memory allocation
constexpr int kTcPvWarp = 7;   // issues the P * V MMAs
constexpr int kTcTile = 128;   // keys per tile
constexpr int kTcStagesK = 3;  // K ring depth
constexpr int kTcStagesV = 4;  // V ring depth
constexpr int kTcD = 128;      // head dimension this kernel is built for
constexpr uint32_t kPanelKV = kTcTile * 128;    // bytes of a [128 keys][64 halfs] panel
constexpr uint32_t kStageBytes = 2 * kPanelKV;  // a K (or V) tile: channels 0-63, then 64-127
constexpr uint32_t kTcBarBytes = 256;
constexpr uint32_t kTcSmemUsed = (kTcStagesK + kTcStagesV) * kStageBytes + kTcBarBytes;
constexpr uint32_t kTcSmemBytes = kTcSmemUsed + 1024;  // slack to align the base to 1024 bytes
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemQ = 0, kTmemS = 128, kTmemP = 256, kTmemO = 384;
constexpr long long kWaitClocks = 2000000000ll;  // about a second
constexpr float kRescaleStep = 8.f;              // log2 of the growth of a row maximum that triggers a rescale
constexpr int kStageRowFloats = kTcD + 4;        // epilogue staging row (padded against bank conflicts)

__device__ __forceinline__ uint32_t panel_off(uint32_t row, uint32_t chunk) {
    return row * 128 + ((chunk ^ (row & 7)) << 4);
}


// Barrier among the 128 softmax threads only (hardware barrier 1; barrier 0 is __syncthreads of the whole CTA).
__device__ __forceinline__ void softmax_sync() { asm volatile("bar.sync 1, 128;\n" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive(uint32_t bar_addr) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar_addr) : "memory");
}

// The mbarrier gets one arrival (counted against its initial count) once every cp.async this thread issued before
// has written its bytes.
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar_addr) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(bar_addr) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

// Bounded wait; a wait that runs out raises the CTA's abort flag, which every role polls once per tile.
__device__ __forceinline__ bool wait_or_abort_within(uint32_t bar_addr, uint32_t parity, volatile int* abort_flag,
                                                     long long limit_clocks) {
    if (tc::mbar_wait_bounded(bar_addr, parity, limit_clocks)) return true;
    *abort_flag = 1;
    return false;
}

// Timeline stamps of CTA (0, 0, 0) (compiled in only with -DITK_DECODE_TRACE): SM clock per role and tile.
#ifdef ITK_DECODE_TRACE
#define TC_TRACE(p, slot)                                                                              \
    do {                                                                                               \
        if ((p).trace && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (slot) < 512)         \
            (p).trace[(slot)] = static_cast<unsigned long long>(clock64());                            \
    } while (0)
// ... and four wall-clock stamps of every CTA: entry, first scores issued, last value product complete, exit.
#define TC_STAMP(p, i)                                                                                         \
    do {                                                                                                       \
        if ((p).trace) {                                                                                       \
            unsigned long long t_;                                                                             \
            asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t_)::"memory");                                 \
            (p).trace[1024 + ((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 4 + (i)] = t_;  \
        }                                                                                                      \
    } while (0)
#else
#define TC_TRACE(p, slot) do { } while (0)
#define TC_STAMP(p, i) do { } while (0)
#endif

// PC = pairs per CTA (32 or 64).
template <int PC>
__global__ void __launch_bounds__(kTcThreads, 1) verify_tc_kernel(const __grid_constant__ AttnLaunch p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    constexpr int R = kTcSoftmaxThreads / PC;  // rows per pair
    constexpr int KH = R / 2;                  // key subsets
    constexpr int CN = kTcTile / KH;           // tile columns a softmax thread handles
    constexpr int D = kTcD;

    unsigned char* smem =
        reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const uint32_t kbuf = smem_u32(smem), vbuf = kbuf + kTcStagesK * kStageBytes;
    // mbarriers (8 bytes each) behind the rings
    const uint32_t bars = vbuf + kTcStagesV * kStageBytes;
    const uint32_t bar_full_k = bars;                     // [stage] the K tile's bytes are in shared memory
    const uint32_t bar_empty_k = bar_full_k + 8 * kTcStagesK;  // [stage] the scores reading it are complete
    const uint32_t bar_full_v = bar_empty_k + 8 * kTcStagesK;
    const uint32_t bar_empty_v = bar_full_v + 8 * kTcStagesV;  // [stage] the P * V reading it is complete
    const uint32_t bar_s = bar_empty_v + 8 * kTcStagesV;  // the tile's scores are complete
    const uint32_t bar_sfree = bar_s + 8;                 // every softmax thread holds its scores in registers
    const uint32_t bar_p = bar_s + 16;                    // [2] the weights of even / odd tiles are stored
    const uint32_t bar_o = bar_s + 32;                    // [2] P * V of even / odd tiles has completed
    const uint32_t bar_q = bar_o + 16;                    // Q and the zeroed P buffers are in tensor memory
    const uint32_t bar_go = bar_q + 8;                    // the query rows have arrived (and left their staging area)
    const uint32_t slot = bar_go + 8;
    volatile uint32_t* slot_ptr = reinterpret_cast<volatile uint32_t*>(smem + (slot - kbuf));
    int* s_flag = reinterpret_cast<int*>(smem + (slot - kbuf) + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + (slot - kbuf) + 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t split = blockIdx.x, seq = blockIdx.z;
    const uint32_t gheads = min(p.group, static_cast<uint32_t>(kHeadsPerCta));
    const uint32_t pchunks = (p.rows * gheads + PC - 1) / PC;
    // pair blocks are handed out last block first: under the causal bound it has the longest key range, and the
    // CTAs placed in the launch's last wave should be the short ones
    const uint32_t hy = blockIdx.y / pchunks, pc = pchunks - 1 - blockIdx.y % pchunks;
    const SeqDesc sd = p.seq[seq];
    const uint32_t kvh = hy / p.gchunks, gc = hy % p.gchunks;
    const uint32_t head0 = kvh * p.group + gc * kHeadsPerCta;
    const uint32_t nh = min(static_cast<uint32_t>(kHeadsPerCta), p.group - gc * kHeadsPerCta);
    const uint32_t n_pairs = p.rows * nh;
    const uint32_t ring = p.layer.ring, window = p.layer.window;

    // This CTA's slice [k0, k1) of the positions its pair block can see: [kv_lo, kv_hi) cut off behind the block's
    // last row (a long chunk's early row blocks do not stream the keys of its later rows).
    const uint32_t last_pair = min(n_pairs, (pc + 1u) * PC) - 1u;
    const uint32_t n = min(sd.kv_hi - sd.kv_lo, sd.q_pos0 + last_pair / nh + 1u - sd.kv_lo);
    uint32_t chunk = (n + p.splits - 1) / p.splits;
    chunk = (chunk + kTcTile - 1) / kTcTile * kTcTile;
    const uint32_t k0 = min(n, split * chunk);
    const uint32_t k1 = min(n, k0 + chunk);
    const uint32_t span = k1 - k0;
    const uint32_t ntiles = (span + kTcTile - 1) / kTcTile;

    if (tid == 0) TC_TRACE(p, 256);
    if (tid == 0) TC_STAMP(p, 0);
    // Launched as a programmatic dependent of the previous kernel in the stream (AttnLaunch::pdl): this grid's CTAs are
    // placed as SMs free up instead of after the previous grid has drained and a launch has crossed the bus; nothing
    // is read or written before the previous kernel's memory is visible.
    // pdl 1: wait for the predecessor, and only then let this grid's own dependents start (they may rely on what this
    // one waited for).  pdl 2 (the predecessor is another layer's launch of this kernel, and so is everything that
    // can still be running): the K/V loaders start streaming this layer's stored rows at once - nothing in flight
    // writes them - while every thread that touches the queries, the call's new rows, the scratch or the outputs
    // waits first.
    const bool early_kv = p.pdl == 2;
    const long long wait_clocks = p.tc_wait_kclocks != 0 ? static_cast<long long>(p.tc_wait_kclocks) << 10 : kWaitClocks;
    auto wait_or_abort = [wait_clocks](uint32_t bar_addr, uint32_t parity, volatile int* flag) {
        return wait_or_abort_within(bar_addr, parity, flag, wait_clocks);
    };
    if (p.pdl == 1) asm volatile("griddepcontrol.wait;\n" ::: "memory");
    if (p.pdl != 0) asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    // The query rows are requested first of all (each softmax warp a quarter of the CTA's PC distinct rows, lane l
    // the 16-byte chunk l of a row), so that their latency runs underneath the set-up below instead of behind the
    // opening burst of K/V tile loads.  (An early launch requests them once it has waited, after the set-up.)
    float4 q_ld[PC / 4];
    auto request_queries = [&]() {
#pragma unroll
        for (int rr = 0; rr < PC / 4; ++rr) {
            const uint32_t spair = pc * PC + warp * (PC / 4) + rr;
            q_ld[rr] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (spair < n_pairs)
                q_ld[rr] = __ldcg(reinterpret_cast<const float4*>(
                                      p.q + ((static_cast<size_t>(seq) * p.rows + spair / nh) * p.q_heads + head0 + spair % nh) *
                                                kTcD) + lane);
        }
    };
    if (warp < kTcMmaWarp && !early_kv) request_queries();
    if (tid == 0) {
        for (int s = 0; s < kTcStagesK; ++s) {
            tc::mbar_init(bar_full_k + 8 * s, kTcLoaderThreads);
            tc::mbar_init(bar_empty_k + 8 * s, 1);
        }
        for (int s = 0; s < kTcStagesV; ++s) {
            tc::mbar_init(bar_full_v + 8 * s, kTcLoaderThreads);
            tc::mbar_init(bar_empty_v + 8 * s, 1);
        }
        tc::mbar_init(bar_s, 1);
        tc::mbar_init(bar_sfree, kTcSoftmaxThreads);
        tc::mbar_init(bar_p, kTcSoftmaxThreads);
        tc::mbar_init(bar_p + 8, kTcSoftmaxThreads);
        tc::mbar_init(bar_o, 1);
        tc::mbar_init(bar_o + 8, 1);
        tc::mbar_init(bar_q, kTcSoftmaxThreads);
        tc::mbar_init(bar_go, kTcSoftmaxThreads);
        *abort_flag = 0;
        tc::fence_mbar_init();
    }
    if (warp == kTcMmaWarp) {
        tc::tmem_alloc(slot, kTmemCols);
        tc::tmem_relinquish();
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = *slot_ptr;
    if (early_kv && warp < kTcMmaWarp) {
        // Early launch: the barriers and tensor memory are set up and the loaders are already streaming; clear the
        // weight buffers while the predecessor finishes, then wait for it and only then touch the queries.
        uint32_t z[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) z[j] = 0u;
#pragma unroll 1
        for (int c = 0; c < kTcTile; c += 16) tc::tmem_st16(tmem + (static_cast<uint32_t>(warp * 32) << 16) + kTmemP + c, z);
        tc::tmem_wait_st();
        asm volatile("griddepcontrol.wait;\n" ::: "memory");
        request_queries();
    }

    if (warp > kTcMmaWarp && warp < kTcPvWarp) {
        // ---------------- loaders: warp 5 streams K, warp 6 streams V; thread lt copies 16-byte chunk c of rows
        // rg, rg + 2, ... of every tile
        const bool is_v = warp > kTcMmaWarp + 1;
        const uint32_t lt = (tid - (kTcMmaWarp + 1) * 32) % kTcLoaderThreads;
        const uint32_t c = lt % (D / 8), rg = lt / (D / 8);
        const uint32_t s0 = (sd.kv_lo + k0) % ring;
        const size_t stream = (static_cast<size_t>(sd.slot) * p.layer.kv_heads + kvh) * ring * D + c * 8;
        const __half* col = static_cast<const __half*>(is_v ? p.layer.v : p.layer.k) + stream;
        const uint32_t soff_c = (c / 8) * kPanelKV, cc = c % 8;
        const uint32_t nst = is_v ? kTcStagesV : kTcStagesK;
        const uint32_t buf = is_v ? vbuf : kbuf;
        const uint32_t bar_full = is_v ? bar_full_v : bar_full_k, bar_empty = is_v ? bar_empty_v : bar_empty_k;
        // Fused append (AttnLaunch::k_new): the block's own rows [q_pos0, q_pos0 + rows) come from the caller's f32
        // rows [n_seqs][rows][kv_heads][D]; new_rel = index of q_pos0 inside this CTA's slice.
        const float* new_base = is_v ? p.v_new : p.k_new;
        const float* new_src =
            new_base ? new_base + (static_cast<size_t>(seq) * p.rows * p.layer.kv_heads + kvh) * D + c * 8 : nullptr;
        const int64_t new_rel = static_cast<int64_t>(sd.q_pos0) - (static_cast<int64_t>(sd.kv_lo) + k0);
        // the CTAs of the LAST pair block see every row of the launch: they are the ones that store them
        const bool stores_new = gc == 0 && pc == pchunks - 1;
        // (tests of the give-up path: the first K tile lands but is never reported)
        auto withheld = [&](uint32_t tile) { return p.tc_withhold != 0 && !is_v && tile == 0; };
        bool waited = !early_kv;  // (early start) has this loader thread waited for the predecessor yet
        // Before the query rows have left their staging area (the last V stage): an ordinary launch requests only the
        // first K tile (see below); an early one fills the K ring and all V stages but the last.
        const uint32_t go_tile = early_kv ? (is_v ? static_cast<uint32_t>(kTcStagesV - 1) : 0xffffffffu) : (is_v ? 0u : 1u);
        for (uint32_t tile = 0; tile < ntiles; ++tile) {
            if (*abort_flag != 0) break;
            const uint32_t st = tile % nst;
            // Only the first K tile is requested before the query rows have arrived: a load issued together with
            // the CTAs' opening burst of hundreds of KiB each waits microseconds for its turn, and the first scores
            // need the queries.  (The last V stage also doubles as the staging area of the query rows.)
            const uint32_t row0 = tile * kTcTile;
            const bool has_new = new_src != nullptr && static_cast<int64_t>(row0) + kTcTile > new_rel;
            // The first few of the block's own rows that fall to this thread are requested before it waits for the
            // stage: they are plain (synchronous) loads, and one round trip each would otherwise sit on the path of
            // the block's last tile.
            constexpr int kPre = 4;
            float4 pre[kPre][2];
            int pre_i0 = 0;
            if (has_new && !waited) {  // the call's new rows come from the caller, and this thread may store them
                asm volatile("griddepcontrol.wait;\n" ::: "memory");
                waited = true;
            }
            if (has_new) {
                const int64_t first = new_rel - static_cast<int64_t>(row0) - rg;  // row index (rg + 2i) of the first new row
                pre_i0 = first > 0 ? static_cast<int>((first + 1) / 2) : 0;
#pragma unroll
                for (int j = 0; j < kPre; ++j) {
                    const uint32_t kr = row0 + rg + 2 * (pre_i0 + j);
                    pre[j][0] = pre[j][1] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (pre_i0 + j < kTcTile / 2 && kr < span) {
                        const float* src = new_src + static_cast<size_t>(kr - new_rel) * p.layer.kv_heads * D;
                        pre[j][0] = *reinterpret_cast<const float4*>(src);
                        pre[j][1] = *reinterpret_cast<const float4*>(src + 4);
                    }
                }
            }
            if (tile == go_tile && !wait_or_abort(bar_go, 0u, abort_flag)) break;
            if (tile >= nst && !wait_or_abort(bar_empty + 8 * st, (tile / nst - 1) & 1u, abort_flag)) break;
            const uint32_t dst = buf + st * kStageBytes;
            if (has_new) {
                // The tile holds rows of the block itself, which no append launch has stored: they are converted
                // here from the caller's f32 rows (the append kernel's conversion), dropped straight into the stage,
                // and stored to the cache by the one CTA of this (sequence, KV head) that is in charge of that.
                // This thread's rows rg + 2i of the tile: i < n_old come from the cache, n_old <= i < n_valid are the
                // block's own, the rest lie past the split and are zero-filled.
                const int n_valid = span > row0 + rg ? static_cast<int>(min(static_cast<uint32_t>(kTcTile / 2), (span - row0 - rg + 1) / 2)) : 0;
                const int n_old = min(pre_i0, n_valid);
                uint32_t nr0 = s0 + row0;
                if (nr0 >= ring) nr0 -= ring;
                if (nr0 + kTcTile <= ring) {
                    // no ring wrap inside the tile: constant offsets, as in the whole-tile path below
                    const __half* g = col + static_cast<size_t>(nr0 + rg) * D;
                    const uint32_t sb = dst + soff_c;
                    const uint32_t o0 = panel_off(rg, cc), o1 = panel_off(rg + 2, cc), o2 = panel_off(rg + 4, cc),
                                   o3 = panel_off(rg + 6, cc);
                    auto put = [&](int i, uint32_t sa, const __half* ga) {
                        if (i < n_old)
                            cp_async16(sa, ga, 16u);
                        else if (i >= n_valid)
                            cp_async16(sa, g, 0u);  // 16 zero bytes, nothing read
                    };
#pragma unroll 4
                    for (int i = 0; i < kTcTile / 8; ++i) {
                        put(4 * i, sb + 1024 * i + o0, g + (8 * i) * D);
                        put(4 * i + 1, sb + 1024 * i + o1, g + (8 * i + 2) * D);
                        put(4 * i + 2, sb + 1024 * i + o2, g + (8 * i + 4) * D);
                        put(4 * i + 3, sb + 1024 * i + o3, g + (8 * i + 6) * D);
                    }
                } else {
                    for (int i = 0; i < kTcTile / 2; ++i) {
                        if (i >= n_old && i < n_valid) continue;
                        const uint32_t row = rg + 2 * i;
                        uint32_t srow = s0 + row0 + row;
                        if (srow >= ring) srow -= ring;
                        const bool valid = i < n_old;
                        cp_async16(dst + soff_c + panel_off(row, cc), col + static_cast<size_t>(valid ? srow : 0u) * D,
                                   valid ? 16u : 0u);
                    }
                }
                for (int i = pre_i0; i < n_valid; ++i) {
                    const uint32_t row = rg + 2 * i;
                    const uint32_t kr = row0 + row;
                    uint32_t srow = s0 + kr;
                    if (srow >= ring) srow -= ring;
                    const int j = i - pre_i0;
                    float4 f0, f1;
                    if (j < kPre) {
                        // (selected by constant index so that `pre` stays in registers)
                        f0 = j == 0 ? pre[0][0] : j == 1 ? pre[1][0] : j == 2 ? pre[2][0] : pre[3][0];
                        f1 = j == 0 ? pre[0][1] : j == 1 ? pre[1][1] : j == 2 ? pre[2][1] : pre[3][1];
                    } else {
                        const float* src = new_src + static_cast<size_t>(kr - new_rel) * p.layer.kv_heads * D;
                        f0 = *reinterpret_cast<const float4*>(src);
                        f1 = *reinterpret_cast<const float4*>(src + 4);
                    }
                    const uint4 packed = pack8(f0, f1);
                    *reinterpret_cast<uint4*>(smem + (dst - kbuf) + soff_c + panel_off(row, cc)) = packed;
                    if (stores_new)
                        *reinterpret_cast<uint4*>(const_cast<__half*>(col) + static_cast<size_t>(srow) * D) = packed;
                }
                cp_async_wait_all();
                tc::fence_proxy_async();  // plain stores into the stage: visible to the tensor core before the arrival
                if (!withheld(tile)) mbar_arrive(bar_full + 8 * st);
                continue;
            }
            uint32_t sr0 = s0 + row0;
            if (sr0 >= ring) sr0 -= ring;
            if (row0 + kTcTile <= span && sr0 + kTcTile <= ring) {
                // A whole tile inside the split and inside the ring (all but a sequence's last tile and a sliding
                // layer's wrap): this thread's 64 copies differ by constants only - rows rg, rg + 2, ... are 512 bytes
                // apart in the cache, and their swizzled places repeat every four rows, 1024 bytes on - so that one
                // loader warp issues a tile in a few hundred instructions instead of a thousand.
                const __half* g = col + static_cast<size_t>(sr0 + rg) * D;
                const uint32_t sb = dst + soff_c;
                const uint32_t o0 = panel_off(rg, cc), o1 = panel_off(rg + 2, cc), o2 = panel_off(rg + 4, cc),
                               o3 = panel_off(rg + 6, cc);
#pragma unroll 4
                for (int i = 0; i < kTcTile / 8; ++i) {
                    cp_async16(sb + 1024 * i + o0, g + (8 * i) * D, 16u);
                    cp_async16(sb + 1024 * i + o1, g + (8 * i + 2) * D, 16u);
                    cp_async16(sb + 1024 * i + o2, g + (8 * i + 4) * D, 16u);
                    cp_async16(sb + 1024 * i + o3, g + (8 * i + 6) * D, 16u);
                }
            } else {
#pragma unroll 8
                for (int i = 0; i < kTcTile / 2; ++i) {
                    const uint32_t row = rg + 2 * i;
                    const uint32_t kr = row0 + row;
                    const bool valid = kr < span;
                    uint32_t srow = s0 + kr;
                    if (srow >= ring) srow -= ring;
                    cp_async16(dst + soff_c + panel_off(row, cc), col + static_cast<size_t>(valid ? srow : 0u) * D,
                               valid ? 16u : 0u);
                }
            }
            // The stage's full barrier receives this thread's arrival when the copies above have landed; nobody waits.
            if (!withheld(tile)) cp_async_arrive_noinc(bar_full + 8 * st);
            if (lt == 0) TC_TRACE(p, tile * 8 + (is_v ? 6 : 5));
        }
        cp_async_wait_all();
    } else if (warp == kTcMmaWarp) {
        // ---------------- score MMAs: one lane issues S = [q_hi | q_lo] * [K | K]^T for every tile
        // (tcgen05.commit tracks the issuing thread's MMAs).  The next tile's scores run underneath this tile's
        // softmax, as soon as every softmax thread has taken this tile's scores into registers.
        if (lane == 0 && ntiles > 0) {
            constexpr uint32_t kIdescS = tc::instr_desc_f16(128, kTcTile, false);
            if (wait_or_abort(bar_q, 0u, abort_flag)) {
                for (uint32_t tile = 0; tile < ntiles; ++tile) {
                    if (*abort_flag != 0) break;
                    if (!wait_or_abort(bar_full_k + 8 * (tile % kTcStagesK), (tile / kTcStagesK) & 1u, abort_flag)) break;
                    if (tile > 0 && !wait_or_abort(bar_sfree, (tile - 1) & 1u, abort_flag)) break;
                    tc::fence_proxy_async();  // the tile was written through the generic proxy (cp.async)
                    tc::fence_after_sync();
                    TC_TRACE(p, tile * 8 + 0);
                    if (tile == 0) TC_STAMP(p, 1);
                    const uint32_t kst = kbuf + (tile % kTcStagesK) * kStageBytes;
#pragma unroll
                    for (int ks = 0; ks < 16; ++ks)  // 16 halfs of the contraction per MMA
                        tc::mma_f16_ts(tmem + kTmemS, tmem + kTmemQ + 8 * ks,
                                       tc::smem_desc(kst + ((ks % 8) / 4) * kPanelKV + (ks % 4) * 32, 16, 1024), kIdescS,
                                       ks > 0 ? 1u : 0u);
                    tc::mma_commit(bar_empty_k + 8 * (tile % kTcStagesK));  // the K tile has been consumed
                    tc::mma_commit(bar_s);
                    TC_TRACE(p, tile * 8 + 7);
                }
            }
        }
        __syncwarp();
    } else if (warp == kTcPvWarp) {
        // ---------------- value MMAs: a second lane issues O (+)= P * V, 16 keys per MMA, as soon as a tile's weights
        // are stored and its V tile has landed; the two issuers meet only through the barriers, so a tile's value
        // product and the next tile's scores are handed to the tensor core without waiting for one another.
        if (lane == 0 && ntiles > 0) {
            constexpr uint32_t kIdescO = tc::instr_desc_f16(128, D, true);
            for (uint32_t tile = 0; tile < ntiles; ++tile) {
                if (*abort_flag != 0) break;
                if (!wait_or_abort(bar_p + 8 * (tile & 1u), (tile >> 1) & 1u, abort_flag)) break;
                if (!wait_or_abort(bar_full_v + 8 * (tile % kTcStagesV), (tile / kTcStagesV) & 1u, abort_flag)) break;
                tc::fence_proxy_async();
                tc::fence_after_sync();
                TC_TRACE(p, tile * 8 + 1);
                const uint32_t vst = vbuf + (tile % kTcStagesV) * kStageBytes;
                const uint32_t a = tmem + kTmemP + (tile & 1u) * (kTcTile / 2);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    tc::mma_f16_ts(tmem + kTmemO, a + 8 * j, tc::smem_desc(vst + j * 2048, kPanelKV, 1024), kIdescO,
                                   (tile > 0 || j > 0) ? 1u : 0u);
                tc::mma_commit(bar_empty_v + 8 * (tile % kTcStagesV));  // the V tile has been consumed
                tc::mma_commit(bar_o + 8 * (tile & 1u));
                TC_TRACE(p, tile * 8 + 2);
            }
        }
        __syncwarp();
    } else {
        // ---------------- softmax: thread tid = tensor-memory lane tid = row r = 2 * kh + x of pair lp: it handles
        // tile columns [col0, col0 + CN) in blocks of 64 and stores the hi (x = 0) or lo (x = 1) term of the weights.
        constexpr int SB = 64;
        constexpr int NSB = CN / SB;
        const uint32_t lp = tid % PC, r = tid / PC, x = r & 1u, col0 = (r >> 1) * CN;
        const uint32_t pair = pc * PC + lp;
        const bool live = pair < n_pairs;
        const uint32_t prow = live ? pair / nh : 0, phead = live ? pair % nh : 0;
        const uint32_t ppos = sd.q_pos0 + prow;
        uint32_t abs_lo = sd.kv_lo;
        if (window != 0 && ppos + 1 > window) abs_lo = max(abs_lo, ppos + 1 - window);
        // Visible keys of the row, as indices into this CTA's slice: [vis_lo, vis_hi).  Rows without a pair see
        // everything (their results are never stored), so they do not force the masked path below.
        constexpr int64_t kFar = 1ll << 30;
        const int64_t rel0 = static_cast<int64_t>(sd.kv_lo) + k0;
        const int32_t vis_lo =
            live ? static_cast<int32_t>(max(-kFar, min(kFar, static_cast<int64_t>(abs_lo) - rel0))) : -static_cast<int32_t>(kFar);
        const int32_t vis_hi =
            live ? static_cast<int32_t>(max(-kFar, min(kFar, static_cast<int64_t>(ppos) + 1 - rel0))) : static_cast<int32_t>(kFar);
        const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
        const uint32_t tO = tmem + lane_base + kTmemO;
        const uint32_t tS = tmem + lane_base + kTmemS + col0;

        {   // Row tid of Q: hi terms of the 128 channels in columns 0-63, lo terms in columns 64-127.
            // Coalesced first: a warp instruction loads one whole 512-byte row (lane l takes 16-byte chunk l), each
            // warp a quarter of the CTA's PC distinct rows, into a staging area in shared memory (chunk l of row i
            // at position l ^ (i & 31): conflict-free both ways).  Then every thread reads the row of its pair.
            unsigned char* stage_q = smem + (vbuf - kbuf) + (kTcStagesV - 1) * kStageBytes;
#pragma unroll
            for (int rr = 0; rr < PC / 4; ++rr) {
                const uint32_t srow = warp * (PC / 4) + rr;
                *reinterpret_cast<float4*>(stage_q + srow * 512 + ((lane ^ (srow & 31u)) << 4)) = q_ld[rr];
            }
            softmax_sync();
            // (a rolled loop: one-time code is kept small)
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {  // 32 channels = 16 columns of hi and 16 of lo
                uint32_t hi[16], lo[16];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float4 v4 = *reinterpret_cast<const float4*>(
                        stage_q + lp * 512 + ((static_cast<uint32_t>(8 * c + j) ^ (lp & 31u)) << 4));
                    __half h0, l0, h1, l1;
                    split_half(v4.x, h0, l0);
                    split_half(v4.y, h1, l1);
                    hi[2 * j] = pack_half2(h0, h1);
                    lo[2 * j] = pack_half2(l0, l1);
                    split_half(v4.z, h0, l0);
                    split_half(v4.w, h1, l1);
                    hi[2 * j + 1] = pack_half2(h0, h1);
                    lo[2 * j + 1] = pack_half2(l0, l1);
                }
                tc::tmem_st16(tmem + lane_base + kTmemQ + 16 * c, hi);
                tc::tmem_st16(tmem + lane_base + kTmemQ + 64 + 16 * c, lo);
            }
            if (tid == 0) TC_TRACE(p, 257);
            mbar_arrive(bar_go);  // (release) the staging area may be overwritten by the V stream
            // Both P buffers start as zeros: a row only ever writes its own columns (an early launch cleared them
            // while it waited).
            if (!early_kv) {
                uint32_t z[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) z[j] = 0u;
#pragma unroll 1
                for (int c = 0; c < kTcTile; c += 16) tc::tmem_st16(tmem + lane_base + kTmemP + c, z);
            }
            tc::tmem_wait_st();
            tc::fence_before_sync();
            mbar_arrive(bar_q);
        }

        float m_use = -INFINITY, l = 0.f;  // the maximum the weights are taken against (log2 domain), their sum
        const float sl = p.scale * kLog2e;
        bool done = ntiles > 0;  // every product into O has completed (nothing to wait for when there is no tile)
        for (uint32_t tile = 0; tile < ntiles; ++tile) {
            if (__any_sync(0xffffffffu, *abort_flag != 0)) { done = false; break; }
            // The scores of this tile are complete.
            if (!__all_sync(0xffffffffu, wait_or_abort(bar_s, tile & 1u, abort_flag))) { done = false; break; }
            tc::fence_after_sync();
            if (tid == 0) TC_TRACE(p, tile * 8 + 3);
            const int32_t kr0 = static_cast<int32_t>(tile * kTcTile + col0);
            // Tiles wholly inside every row's visible range (all but the causal edge and a window's trailing edge)
            // skip the masks.
            const bool masked = __any_sync(0xffffffffu, kr0 < vis_lo || kr0 + CN > vis_hi);
            uint32_t sr[SB / 16][16];
            // Raw scores of block sb into sr (masked ones become -inf); returns their maximum.
            auto load_block = [&](int sb) {
#pragma unroll
                for (int i = 0; i < SB / 16; ++i) tc::tmem_ld16(tS + sb * SB + 16 * i, sr[i]);
                tc::tmem_wait_ld();
                float mx = -INFINITY;
                if (masked) {
#pragma unroll
                    for (int i = 0; i < SB / 16; ++i)
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int32_t kr = kr0 + sb * SB + 16 * i + j;
                            if (kr < vis_lo || kr >= vis_hi) sr[i][j] = 0xff800000u;  // -inf
                        }
                }
#pragma unroll
                for (int i = 0; i < SB / 16; ++i)
#pragma unroll
                    for (int j = 0; j < 16; ++j) mx = fmaxf(mx, __uint_as_float(sr[i][j]));
                return mx;
            };
            float mx = load_block(0);
            if constexpr (NSB == 2) mx = fmaxf(mx, load_block(1));
            mx *= sl;  // sl > 0: the maximum of the scaled scores
            if constexpr (NSB == 1) {
                tc::fence_before_sync();
                mbar_arrive(bar_sfree);  // the scores are in registers: the next tile's may overwrite them
            }
            const bool grow = mx > m_use + kRescaleStep;  // also the first visible key of the row (m_use = -inf)
            const float m_new = grow ? mx : m_use;
            const float corr = grow ? (m_use == -INFINITY ? 0.f : fast_exp2(m_use - m_new)) : 1.f;
            if (tile > 0 && __ballot_sync(0xffffffffu, grow) != 0u) {
                // Some row of this warp moves its maximum: once the previous tile's P * V has completed, rescale
                // the warp's 32 accumulator rows in tensor memory.
                // (A parity wait is only unambiguous while the waiter is at most one phase behind: hence one barrier
                // for even and one for odd tiles - the product of tile - 3 is known complete, that of tile + 1 cannot
                // have been issued.)
                if (!__all_sync(0xffffffffu, wait_or_abort(bar_o + 8 * ((tile - 1) & 1u), ((tile - 1) >> 1) & 1u, abort_flag))) {
                    done = false;
                    break;
                }
                tc::fence_after_sync();
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 16) {
                    uint32_t o16[16];
                    tc::tmem_ld16(tO + c0, o16);
                    tc::tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 16; ++j) o16[j] = __float_as_uint(__uint_as_float(o16[j]) * corr);
                    tc::tmem_st16(tO + c0, o16);
                }
            }
            l *= corr;
            m_use = m_new;
            // The weights of this tile go where those of tile - 2 were: that tile's value product must have read
            // them (the score issuer no longer vouches for it, the two kinds of MMA come from different threads).
            if (tile >= 2) {
                if (!__all_sync(0xffffffffu, wait_or_abort(bar_o + 8 * (tile & 1u), ((tile - 2) >> 1) & 1u, abort_flag))) {
                    done = false;
                    break;
                }
                tc::fence_after_sync();
            }
            const float neg_m = (m_use == -INFINITY) ? 0.f : -m_use;
            const uint32_t tP = tmem + lane_base + kTmemP + (tile & 1u) * (kTcTile / 2) + col0 / 2;
#pragma unroll
            for (int sb = 0; sb < NSB; ++sb) {
                if constexpr (NSB == 2) {
                    load_block(sb);
                    if (sb == NSB - 1) {
                        tc::fence_before_sync();
                        mbar_arrive(bar_sfree);
                    }
                }
                // weights = 2^(score * scale - max); this row keeps their f16 hi or lo term, two keys per column
#pragma unroll
                for (int i = 0; i < SB / 16; ++i) {
                    uint32_t w8[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float p0 = fast_exp2(fmaf(__uint_as_float(sr[i][2 * e]), sl, neg_m));
                        const float p1 = fast_exp2(fmaf(__uint_as_float(sr[i][2 * e + 1]), sl, neg_m));
                        l += p0 + p1;
                        __half2 h2 = __floats2half2_rn(p0, p1);
                        if (x != 0u) {
                            const float2 hf = __half22float2(h2);
                            h2 = __floats2half2_rn(p0 - hf.x, p1 - hf.y);
                        }
                        w8[e] = *reinterpret_cast<const uint32_t*>(&h2);
                    }
                    tc::tmem_st8(tP + (sb * SB) / 2 + 8 * i, w8);
                }
            }
            tc::tmem_wait_st();
            tc::fence_before_sync();
            if (tid == 0) TC_TRACE(p, tile * 8 + 4);
            mbar_arrive(bar_p + 8 * (tile & 1u));  // weights stored
        }
        // The last two products: the scores of the last tile only vouch for those up to tile ntiles - 3.
        if (done && ntiles > 1)
            done = __all_sync(0xffffffffu, wait_or_abort(bar_o + 8 * ((ntiles - 2) & 1u), ((ntiles - 2) >> 1) & 1u, abort_flag));
        if (done)
            done = __all_sync(0xffffffffu, wait_or_abort(bar_o + 8 * ((ntiles - 1) & 1u), ((ntiles - 1) >> 1) & 1u, abort_flag));
        tc::fence_after_sync();
        if (tid == 0) TC_STAMP(p, 2);
        const bool have_o = done;
        if (x != 0u) l = 0.f;  // the hi and lo rows of a pair saw the same weights: their sum counts once
        softmax_sync();  // the rings are idle now (every tile was consumed): they become staging space

        float* stage_o = reinterpret_cast<float*>(smem);                  // [128][D + 4]
        float* stage_ml = stage_o + kTcSoftmaxThreads * kStageRowFloats;  // [128][2]
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 16) {
            uint32_t r[16];
            if (have_o) {
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
        softmax_sync();

        // Merge the R rows of pair lp; this thread produces channels [rep * DW, (rep + 1) * DW).
        const uint32_t rep = r;
        constexpr int DW = D / R;
        float M = -INFINITY, L = 0.f;
        float w[R];
#pragma unroll
        for (int rr = 0; rr < R; ++rr) M = fmaxf(M, stage_ml[2 * (rr * PC + lp)]);
#pragma unroll
        for (int rr = 0; rr < R; ++rr) {
            const float ms = stage_ml[2 * (rr * PC + lp)];
            w[rr] = (ms == -INFINITY) ? 0.f : fast_exp2(ms - M);
            L += w[rr] * stage_ml[2 * (rr * PC + lp) + 1];
        }
        float4 acc[DW / 4];
#pragma unroll
        for (int i = 0; i < DW / 4; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int rr = 0; rr < R; ++rr) {
            const float4* src = reinterpret_cast<const float4*>(stage_o + (rr * PC + lp) * kStageRowFloats + rep * DW);
#pragma unroll
            for (int i = 0; i < DW / 4; ++i) {
                const float4 v = src[i];
                acc[i].x += w[rr] * v.x;
                acc[i].y += w[rr] * v.y;
                acc[i].z += w[rr] * v.z;
                acc[i].w += w[rr] * v.w;
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
            softmax_sync();
            if (tid == 0) {
                const unsigned int ticket = atomicAdd(p.tickets + cell, 1u);
                *s_flag = (ticket == p.splits - 1) ? 1 : 0;
            }
            softmax_sync();
            if (*s_flag != 0) {  // the last CTA of the cell merges every split
                __threadfence();
                const float* all_o = p.part_o + cell * p.splits * PC * D;
                const float2* all_ml = reinterpret_cast<const float2*>(p.part_ml) + cell * p.splits * PC;
                const uint32_t cta_pairs = min(static_cast<uint32_t>(PC), n_pairs - pc * PC);
                // Every split's (max, sum) pairs come into shared memory in one round trip (the rings are idle: at
                // most 256 splits x PC x 12 bytes), the splits' weights per pair follow from them, and every output
                // is a weighted sum with all of a thread's loads of one split (two, on a 32-pair block) in flight
                // together - not one dependent round trip per split and output.
                softmax_sync();  // the staging rows above have been read by every thread
                float* w_s = reinterpret_cast<float*>(smem);                 // [splits][PC]
                float2* ml_s = reinterpret_cast<float2*>(w_s + p.splits * PC);  // [splits][PC]
                for (uint32_t i = tid; i < p.splits * PC; i += kTcSoftmaxThreads) ml_s[i] = __ldcg(all_ml + i);
                softmax_sync();
                if (static_cast<uint32_t>(tid) < cta_pairs) {
                    float Mx = -INFINITY;
                    for (uint32_t s = 0; s < p.splits; ++s) Mx = fmaxf(Mx, ml_s[s * PC + tid].x);
                    float Ls = 0.f;
                    for (uint32_t s = 0; s < p.splits; ++s) {
                        const float2 ml = ml_s[s * PC + tid];
                        const float ws = (ml.x == -INFINITY) ? 0.f : fast_exp2(ml.x - Mx);
                        w_s[s * PC + tid] = ws;
                        Ls += ws * ml.y;
                    }
                    const float inv = 1.f / Ls;
                    for (uint32_t s = 0; s < p.splits; ++s) w_s[s * PC + tid] *= inv;
                }
                softmax_sync();
                constexpr int kOut4 = PC * (D / 4) / kTcSoftmaxThreads;  // float4 outputs per thread: 8 or 16
                constexpr int kSplitBatch = kOut4 <= 8 ? 2 : 1;
                float4 o[kOut4];
#pragma unroll
                for (int i = 0; i < kOut4; ++i) o[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                for (uint32_t s0 = 0; s0 < p.splits; s0 += kSplitBatch) {
                    float4 v[kSplitBatch][kOut4];
#pragma unroll
                    for (int bb = 0; bb < kSplitBatch; ++bb) {
                        const uint32_t s = min(s0 + bb, p.splits - 1);  // a repeated split past the end weighs zero
                        const float4* src = reinterpret_cast<const float4*>(all_o + static_cast<size_t>(s) * PC * D);
#pragma unroll
                        for (int i = 0; i < kOut4; ++i) {
                            const uint32_t idx = tid + i * kTcSoftmaxThreads;
                            v[bb][i] = idx < cta_pairs * (D / 4) ? __ldcg(src + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                    }
#pragma unroll
                    for (int bb = 0; bb < kSplitBatch; ++bb) {
                        const bool real = s0 + bb < p.splits;
#pragma unroll
                        for (int i = 0; i < kOut4; ++i) {
                            const uint32_t idx = tid + i * kTcSoftmaxThreads;
                            const float ws = (real && idx < cta_pairs * (D / 4)) ? w_s[(s0 + bb) * PC + idx / (D / 4)] : 0.f;
                            o[i].x += ws * v[bb][i].x;
                            o[i].y += ws * v[bb][i].y;
                            o[i].z += ws * v[bb][i].z;
                            o[i].w += ws * v[bb][i].w;
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < kOut4; ++i) {
                    const uint32_t idx = tid + i * kTcSoftmaxThreads;
                    if (idx < cta_pairs * (D / 4)) {
                        const uint32_t q = idx / (D / 4), d4 = idx % (D / 4);
                        const uint32_t gp = pc * PC + q;
                        const uint32_t orow = gp / nh, h = gp % nh;
                        reinterpret_cast<float4*>(p.out + ((static_cast<size_t>(seq) * p.rows + orow) * p.q_heads + head0 + h) *
                                                              D)[d4] = o[i];
                    }
                }
                if (tid == 0) p.tickets[cell] = 0u;
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (tid == 0) TC_TRACE(p, 258);
    if (tid == 0) TC_STAMP(p, 3);
    if (tid == 0 && *abort_flag != 0 && p.status) atomicOr(p.status, 1u);
    if (warp == kTcMmaWarp) tc::tmem_dealloc(tmem, kTmemCols);
}

uint32_t tc_pairs_for(uint32_t rows, uint32_t group) {
    const uint32_t pairs = rows * (group < static_cast<uint32_t>(kHeadsPerCta) ? group : kHeadsPerCta);
    return pairs <= 32 ? 32u : 64u;
}

}  // namespace

bool verify_tc_supported(uint32_t head_dim, uint32_t rows, uint32_t group) {
    (void)group;
    return rows >= 2 && head_dim == static_cast<uint32_t>(kTcD);
}

uint32_t verify_tc_pairs_per_cta(uint32_t rows, uint32_t group) { return tc_pairs_for(rows, group); }

uint32_t verify_tc_pair_chunks(uint32_t rows, uint32_t group) {
    const uint32_t nh = group < static_cast<uint32_t>(kHeadsPerCta) ? group : kHeadsPerCta;
    const uint32_t pc = verify_tc_pairs_per_cta(rows, group);
    return (rows * nh + pc - 1) / pc;
}

cudaError_t configure_verify_tc() {
    cudaError_t e = cudaFuncSetAttribute(verify_tc_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
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
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kTcThreads);
    cfg.dynamicSmemBytes = kTcSmemBytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.pdl != 0 ? 1 : 0;
    const cudaError_t e = tc_pairs_for(p.rows, p.group) == 32 ? cudaLaunchKernelEx(&cfg, verify_tc_kernel<32>, p)
                                                              : cudaLaunchKernelEx(&cfg, verify_tc_kernel<64>, p);
    if (e != cudaSuccess) return e;
    if (launches) *launches += 1;
    return cudaGetLastError();
}

}  // namespace itk
