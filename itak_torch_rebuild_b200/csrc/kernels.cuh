// Device-side contracts shared by the hot-path kernels and their launchers.
//
// HBM layout of the resident cache (one slab for K, one for V, per backend):
//
//   layer l  ->  [slot][kv_head][row][D]      row = position % ring_l
//
// i.e. HEAD-MAJOR inside a slot: all rows of one (slot, kv head) are one
// contiguous stream of ring_l * D elements.  A decode CTA owns one
// (sequence, kv head, split) and therefore streams one contiguous byte range;
// a KV-head shard for another GPU is a contiguous slice; appends, snapshots and
// restores are the vectorised transposes between this layout and the
// position-major `[position][kv_head][D]` rows the callers speak.
// ring_l is max_context on a global layer and window + chunk_cap on a sliding
// layer: a chunk appended before its attention never evicts a row one of its
// own queries still sees, and rows discarded by a speculative rewind never sit
// on a row that a later query or view can reach.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace itk {

constexpr int kMaxSeqsPerLaunch = 64;  // sequences described in one launch's parameters
constexpr int kHeadsPerCta = 8;        // query heads of one GQA group handled by one CTA
constexpr int kMaxLayersPerLaunch = 64;

// One sequence of an attention / append launch.
struct SeqDesc {
    uint32_t slot;    // resident sequence index
    uint32_t q_pos0;  // absolute position of the first query (and first appended) row
    uint32_t kv_lo;   // first absolute position any row of this launch may see
    uint32_t kv_hi;   // one past the last position (q_pos0 + rows)
};

// Device-resident form of a decode step's sequence list: the kernels derive kv_lo / kv_hi from the position,
// and a one-block kernel advances the positions, so a captured step can be replayed without host updates.
struct SeqState {
    uint32_t slot;
    uint32_t pos;  // position of the step's query = position its new row is stored at
};

struct LayerView {
    const void* k;      // layer base of the K slab (element type by dtype)
    const void* v;      // layer base of the V slab
    uint32_t ring;      // rows per (slot, head) stream
    uint32_t window;    // 0 = global layer, else the attention window
    uint32_t kv_heads;  // heads resident in this backend
    uint32_t head_dim;
};

constexpr int kMaxPeers = 8;  // GPUs of one box

// The per-layer gather of head outputs done by the decode kernel itself: the CTA that writes a cell's final
// output stores it into the same place of every rank's gather buffer (plain stores to peer-mapped memory over
// NVLink) and then bumps entry [sequence][my_rank] of every rank's counter array, so a consumer on rank j knows that
// rank r has delivered c cells of a sequence (cells_per_seq per launch) once counters_j[sequence][r] >= c.
//
// Lanes.  A layer's inputs for one sequence depend on the previous layer's gathered outputs of THAT sequence only, so
// the batch can run as two halves ("lanes": sequences [0, lane_split) and [lane_split, n_seqs)) that are out of phase
// with each other: while one lane's outputs cross NVLink and the next layer waits for them, the other lane streams
// its cache.  With lanes == 2 the first half of the grid's CTAs serves lane 0 and the second half lane 1 (one CTA of
// each per SM), and a CTA waits only for the previous launch's cells of the sequences it works on itself.
struct GatherTarget {
    uint32_t n_peers;                    // 0 = outputs go to AttnLaunch::out only
    uint32_t my_rank;
    float* peer_out[kMaxPeers];          // this rank's [n_seqs][q_heads][D] slot inside every rank's buffer
    unsigned int* peer_flags[kMaxPeers]; // every rank's counter array ([kMaxSeqsPerLaunch][kMaxPeers] entries)
    const unsigned int* my_flags;        // the local flag array, written by the peers
    unsigned int* err;                   // local word: bit 0 = a bounded wait ran out
    const uint32_t* base_pos;            // device word: position of sequence 0 when the loop began
    uint32_t launches_per_step;          // decode launches of one step of the loop
    uint32_t launches_before;            // decode launches of this step that precede this one
    uint32_t lanes;                      // 1, or 2 = the two-lane schedule described above
    uint32_t lane_split;                 // first sequence of lane 1
    uint32_t cells_per_seq;              // cells every rank delivers per sequence and launch
    uint32_t stagger_ns;                 // (first launch of a step, two lanes) lane 1 holds back this long after its
                                         // CTAs start - about half of what a lane takes to stream - which puts the two
                                         // lanes out of phase for the rest of the step; 0 = no hold
    uint32_t wait_prev;                  // 1 = before using its inputs, check that every peer's previous launch arrived
    uint32_t local_only;                 // 1 = the only "peer" is this GPU itself (a single-GPU loop run in lanes): the
                                         // outputs and counters need device scope only
    uint32_t poll_limit;                 // polls of one arrival flag before the wait gives up and records that
};

struct AttnLaunch {
    LayerView layer;
    const float* q;          // [n_seqs][rows][q_heads][D]
    float* out;              // [n_seqs][rows][q_heads][D]
    float* part_o;           // [unit][hy][split][8][D] unnormalised partial outputs
    float* part_ml;          // [unit][hy][split][8][2] running max (log2 domain) and sum
    unsigned int* tickets;   // [unit][hy] arrival counters, zero between launches
    float* acc_o;            // decode kernel, optional: [unit][hy][8][D] sums of the parts' outputs, each scaled by
    float* acc_l;            // 2^max of its part, and [unit][hy][8] of their weight sums, added to with reductions
    unsigned int* acc_flag;  // in L2; [unit][hy] raised when a part's maximum is outside the range that makes such
                             // sums safe, which sends the cell's merge down the exact path.  All zero between launches.
    uint32_t q_heads;
    uint32_t group;          // q_heads / kv_heads
    uint32_t gchunks;        // ceil(group / 8): head chunks per kv head
    uint32_t rows;           // query rows per sequence
    uint32_t n_seqs;
    uint32_t splits;         // partial slots per cell in the scratch: the CTAs along a key range (general and
                             // verify kernels) or the most CTAs that can share one cell (decode kernel)
    uint32_t tiles_per_cta;  // decode kernel: 64-key tiles each persistent CTA walks
    const float* k_new;      // decode and tcgen05 multi-row kernels: when set, the launch's new K rows
    const float* v_new;      // [n_seqs][rows][kv_heads][D] (f32); the kernel stores them at positions q_pos0.. itself
                             // instead of a separate append launch
    uint32_t pdl;            // decode and tcgen05 multi-row kernels launched as a programmatic dependent of the previous kernel in the
                             // stream: 0 = no, 1 = wait for it before anything else, 2 = wait only after the first
                             // K/V tile loads are in flight (nothing the predecessor writes is read before the wait),
                             // (tcgen05 multi-row kernel: its K/V loaders stream the layer's stored rows before the
                             // wait; the backend grants it only behind launches of the same kernel on other layers),
                             // 3 = (decode kernel, two lanes) never wait for the predecessor before working - the
                             // lane's arrival counters order everything that is shared with it - and wait for it just
                             // before the CTA exits, so that grids still complete in stream order
    GatherTarget gather;     // decode kernel (replayable loop): fused all-gather of the outputs
    const SeqState* seq_dev; // decode kernel: when set, sequences come from device memory instead of `seq`, and
                             // tiles_per_cta is derived in the kernel from the grid size
    const uint32_t* plan_dev; // decode kernel, with seq_dev: the work plan of the current positions, worked out once
                             // per step by the kernel that advances them (kDecodePlanBlocks blocks of kDecodePlanWords
                             // words: whole batch, lane 0, lane 1); null = every CTA works it out itself
    unsigned int* status;    // device word the kernels OR error bits into (bit 0: a bounded wait on the tensor
                             // core ran out in the tcgen05 multi-row kernel); may be null
    uint32_t tc_wait_kclocks;  // tcgen05 multi-row kernel: limit of every bounded wait in units of 1024 SM clocks
                               // (0 = the default of about a second)
    uint32_t tc_withhold;      // tcgen05 multi-row kernel, tests of the give-up path only: 1 = the K loader never
                               // reports the first tile, so the first wait for it runs out and every role leaves
    float scale;             // score scale, 1/sqrt(D) by default
#ifdef ITK_DECODE_TRACE
    unsigned long long* trace;  // timeline build only: [cta][16] %globaltimer stamps of the decode kernel's phases
#endif
    SeqDesc seq[kMaxSeqsPerLaunch];
};

// Timeline stamps of the decode kernel (compiled in only with -DITK_DECODE_TRACE; thread 0 of each CTA).
#ifdef ITK_DECODE_TRACE
#define ITK_TRACE(p, i)                                                                     \
    do {                                                                                    \
        if ((p).trace && threadIdx.x == 0) {                                                \
            unsigned long long t_;                                                          \
            asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t_)::"memory");              \
            (p).trace[blockIdx.x * 16 + (i)] = t_;                                           \
        }                                                                                   \
    } while (0)
#else
#define ITK_TRACE(p, i) do { } while (0)
#endif

struct AppendLaunch {
    void* k;  // layer base of the K slab
    void* v;
    const float* k_src;  // [n_seqs][rows][kv_heads][D]
    const float* v_src;
    uint32_t ring, kv_heads, head_dim, rows, n_seqs;
    SeqDesc seq[kMaxSeqsPerLaunch];
};

// Attention preparation (per-head RMSNorm and rotary rotation of the Q and K rows of one call).
struct PrepLaunch {
    const float* q_in;       // [n_seqs][rows][q_heads][D]
    const float* k_in;       // [n_seqs][rows][kv_heads][D]
    float* q_out;            // same shapes; may not alias the inputs
    float* k_out;
    const float* q_w;        // [D] RMSNorm weight of the Q head rows, or null: no norm
    const float* k_w;        // [D] ... of the K head rows, or null
    const double* inv_freq;  // [rotary_dim / 2] base^(-2i / rotary_dim); null when rotary_dim == 0
    float eps;
    uint32_t rotary_dim;     // 0 = no rotation; even, <= head_dim
    uint32_t pairing;        // 0 = adjacent pairs (2i, 2i + 1), 1 = half split (i, i + rotary_dim / 2)
    uint32_t q_heads, kv_heads, head_dim, rows, n_seqs;
    uint32_t pos0[kMaxSeqsPerLaunch];  // absolute position of each sequence's first row
};

// One layer of a snapshot gather / restore scatter.
struct CopyLayer {
    unsigned long long slab_off;  // element offset of this layer inside the K (= V) slab
    unsigned long long snap_k;    // element offset of the layer's K block inside the snapshot buffer
    unsigned long long snap_v;    // ... and of its V block
    uint32_t ring;
    uint32_t first_pos;  // absolute position of the block's first row
    uint32_t rows;
    uint32_t _pad;
};

struct CopyLaunch {
    void* k_slab;
    void* v_slab;
    void* snap;          // snapshot buffer (element type = cache element type)
    uint32_t slot, kv_heads, head_dim, n_layers;
    uint32_t elem_bytes;
    uint32_t to_snapshot;  // 1 = gather slab -> snapshot, 0 = scatter snapshot -> slab
    unsigned long long total_vec;  // work items over all layers, K and V (an item = 8 rows of one vector column)
    unsigned long long vec_prefix[kMaxLayersPerLaunch + 1];  // running K work-item counts per layer
    CopyLayer layer[kMaxLayersPerLaunch];
};

// ---- launchers (defined next to their kernels) -------------------------------
// Every launcher returns the CUDA error of the launch and adds the number of
// kernels it launched to *launches.

cudaError_t launch_append(const AppendLaunch& p, bool f16, cudaStream_t s, uint64_t* launches);
// f32 -> cache element type, flat (used to import f32 snapshot rows).
cudaError_t launch_convert(const float* src, void* dst, size_t n, bool f16, cudaStream_t s, uint64_t* launches);
// Flash-decode over an f16 cache, rows == 1, head_dim 64 or 128 (tensor-core path).  `p` carries everything
// but the work partition, which the launcher derives for `cta_slots` resident CTAs; at most `max_parts` CTAs
// may share one (sequence, head) cell (bounds the scratch: cells * max_parts partial slots).  The number of
// partial slots per cell actually used is returned through *parts_used.
cudaError_t launch_decode_f16(AttnLaunch p, uint32_t cta_slots, uint32_t max_parts, cudaStream_t s,
                              uint64_t* launches, uint32_t* parts_used);
constexpr uint32_t kDecodeMaxParts = 64;
// The same kernel over device-resident sequence states (p.seq_dev, p.n_seqs set by the caller): `ctas` CTAs,
// `parts_stride` partial slots per cell.  Nothing in the launch depends on host-side positions.
cudaError_t launch_decode_f16_resident(AttnLaunch p, uint32_t ctas, uint32_t parts_stride, cudaStream_t s,
                                       uint64_t* launches);
// pdl != 0 launches with programmatic stream serialization (see AttnLaunch::pdl).
// The decode kernel's work plan as device words (AttnLaunch::plan_dev): per block the running tile counts, the
// aligned plan's first CTAs, every sequence's visible keys / first storage row / slot, and [mode, steps done].
constexpr int kDecodePlanWords = 2 * (kMaxSeqsPerLaunch + 4) + 3 * kMaxSeqsPerLaunch + 4;
constexpr int kDecodePlanBlocks = 3;  // 0 = the whole batch on `ctas` CTAs, 1 and 2 = the lanes on lane_ctas / 2 each
struct DecodePlanSpec {
    uint32_t cells_per_seq;  // KV heads x head chunks
    uint32_t ctas;           // CTAs of a launch without lanes
    uint32_t lane_ctas;      // CTAs of a two-lane launch (both lanes), 0 = no lanes
    uint32_t lane_split;     // first sequence of lane 1
    uint32_t splits;         // partial slots per cell
};
// (behind the blocks, plan_out holds one more word: the position of sequence 0 when the loop began, written by the host)
// pos += add for the first n states (global layers only: a sequence sees positions 0..pos), then the plans of the new
// positions into plan_out (may be null: positions only).
cudaError_t launch_advance_states(SeqState* states, uint32_t n, uint32_t add, const DecodePlanSpec& spec, uint32_t* plan_out,
                                  cudaStream_t s, uint64_t* launches);
// The decode kernel's cell-aligned plan: every cell (sequence s has `cells_per_seq` of them, each of
// tiles(keys[s]) 64-key tiles) gets floor(G * T / total) CTAs of its own and equal runs inside it.  Returns
// whether that plan is taken - every cell gets at least one CTA, no cell needs more than `splits` parts and the
// longest run exceeds `per` (the equal-run length of the unaligned plan) by at most a sixteenth - and fills
// first_cta[0..n_seqs] (first CTA of each sequence's cells), *worst (longest run in tiles).  Evaluated by the kernel
// and, identically, by the host when it sizes the grid.
__host__ __device__ inline bool decode_aligned_plan(const uint32_t* keys, uint32_t n_seqs, uint32_t cells_per_seq,
                                                    uint32_t G, uint32_t total, uint32_t per, uint32_t splits,
                                                    uint32_t* first_cta, uint32_t* worst) {
    bool ok = total >= G && G > 0;
    uint32_t b = 0, w = 0;
    for (uint32_t s = 0; s < n_seqs && ok; ++s) {
        const uint32_t T = (keys[s] + 63u) / 64u;
        const uint32_t ns = static_cast<uint32_t>(static_cast<unsigned long long>(T) * G / total);  // CTAs per cell
        if (ns == 0) {
            ok = false;
            break;
        }
        const uint32_t run = (T + ns - 1) / ns;
        if ((T + run - 1) / run > splits) ok = false;  // more parts than the scratch has slots per cell
        if (run > w) w = run;
        first_cta[s] = b;
        b += ns * cells_per_seq;
    }
    first_cta[n_seqs] = b;
    *worst = w;
    const uint32_t slack = per / 16u > 1u ? per / 16u : 1u;
    return ok && w <= per + slack;
}
// Where a CTA of the decode kernel starts and how far it walks.  `cum[s]` = tiles of all cells before sequence s
// (cum[n_seqs] = total), `first_cta` from decode_aligned_plan, `per` = tiles per CTA of the equal-run plan.
// ntiles == 0: the CTA has nothing to do.  parts / part (how many CTAs share the first cell, and which of them
// this is) are filled for the aligned plan only; in the equal-run plan a cell's parts follow from decode_cell_parts.
struct DecodeRun {
    uint32_t seq, hy, tile, ntiles, parts, part;
};
__host__ __device__ inline DecodeRun decode_cta_run(bool aligned, uint32_t cta, const uint32_t* keys, const uint32_t* cum,
                                                    const uint32_t* first_cta, uint32_t n_seqs, uint32_t cells_per_seq,
                                                    uint32_t per) {
    DecodeRun r{0, 0, 0, 0, 0, 0};
    if (aligned) {
        if (cta >= first_cta[n_seqs]) return r;
        uint32_t s = 0;
        while (first_cta[s + 1] <= cta) ++s;
        const uint32_t T = (keys[s] + 63u) / 64u;
        const uint32_t ns = (first_cta[s + 1] - first_cta[s]) / cells_per_seq;
        const uint32_t at = cta - first_cta[s];
        const uint32_t run = (T + ns - 1) / ns;
        r.seq = s;
        r.hy = at / ns;
        r.part = at % ns;
        r.parts = (T + run - 1) / run;
        r.tile = r.part * run;
        if (r.tile < T) r.ntiles = (run < T - r.tile) ? run : T - r.tile;
        return r;
    }
    const uint32_t total = cum[n_seqs];
    const uint64_t g0 = static_cast<uint64_t>(cta) * per;
    if (g0 >= total) return r;
    r.ntiles = static_cast<uint32_t>((total < g0 + per ? total : g0 + per) - g0);
    uint32_t s = 0;
    while (s + 1 < n_seqs && cum[s + 1] <= g0) ++s;
    const uint32_t T = (keys[s] + 63u) / 64u;
    const uint32_t at = static_cast<uint32_t>(g0) - cum[s];
    r.seq = s;
    r.hy = at / T;
    r.tile = at % T;
    return r;
}
// Equal-run plan: the CTAs that share cell (seq, hy) of T tiles, and which of them `cta` is.
__host__ __device__ inline void decode_cell_parts(uint32_t cta, uint32_t cell_first_tile, uint32_t T, uint32_t per,
                                                  uint32_t* parts, uint32_t* part) {
    const uint32_t first = cell_first_tile / per, last = (cell_first_tile + T - 1) / per;
    *parts = last - first + 1;
    *part = cta - first;
}
// Most CTAs that can share a cell of T tiles when every CTA walks `per` tiles.
inline uint32_t decode_parts_for(uint32_t T, uint32_t per) { return (T + per - 2) / per + 1; }
bool decode_f16_supported(uint32_t head_dim, uint32_t rows);
// Multi-row causal attention over an f16 cache (chunked prefill / speculative verify).
cudaError_t launch_verify_f16(const AttnLaunch& p, cudaStream_t s, uint64_t* launches);
bool verify_f16_supported(uint32_t head_dim, uint32_t rows, uint32_t group);
// The same contract on the tcgen05 tensor cores (head_dim 128): accumulators in tensor memory, one CTA per SM.
// A cell of its scratch is a (sequence, head chunk, block of verify_tc_pairs_per_cta row-head pairs).
cudaError_t launch_verify_tc(const AttnLaunch& p, cudaStream_t s, uint64_t* launches);
bool verify_tc_supported(uint32_t head_dim, uint32_t rows, uint32_t group);
uint32_t verify_tc_pairs_per_cta(uint32_t rows, uint32_t group);
uint32_t verify_tc_pair_chunks(uint32_t rows, uint32_t group);
cudaError_t configure_verify_tc();
// Attention over an f32 cache on the tensor cores (three-term tf32 products), head_dim 64 or 128, any number of rows.
// With AttnLaunch::k_new / v_new set it stores the call's new rows itself (no append launch).
// A cell of its scratch is a (sequence, head chunk, block of attn_f32_pairs_per_cta row-head pairs).
cudaError_t launch_attn_f32(const AttnLaunch& p, cudaStream_t s, uint64_t* launches);
bool attn_f32_supported(uint32_t head_dim, uint32_t rows);
uint32_t attn_f32_pairs_per_cta(uint32_t rows, uint32_t group);
uint32_t attn_f32_pair_chunks(uint32_t rows, uint32_t group);
uint32_t attn_f32_max_parts();  // most parts one block's key range is cut into
cudaError_t configure_attn_f32();
// General kernel: any head_dim <= 256, any rows, f32 or f16 cache (CUDA cores, f32 math).
cudaError_t launch_attn_general(const AttnLaunch& p, bool f16, cudaStream_t s, uint64_t* launches);
cudaError_t launch_snapshot_copy(const CopyLaunch& p, cudaStream_t s, uint64_t* launches);
cudaError_t launch_prep(const PrepLaunch& p, cudaStream_t s, uint64_t* launches);
// One-time per-device kernel attribute setup (dynamic shared memory opt-in).
cudaError_t configure_kernels();

}  // namespace itk
