// Host side of the C ABI (include/itak_cuda_compute.h): the resident cache's
// bookkeeping, every refusal in the reference's order and wording, and the
// dispatch of the hot-path kernels.  The arithmetic lives in the kernels; this
// file never touches a cache element on the CPU.
//
// State mirrored from the reference:
//   - per (slot, layer) `appended`: KvCache's position counter
//     (crates/attention/src/cache.rs:114-116, 407-415);
//   - per slot one live checkpoint (cache id, serial, per-layer bases, round
//     bound): crates/attention/src/cache.rs:229-321, 606-833;
//   - the attention step's position cross-check against the caller's
//     Cache::position(): crates/cpu-compute/src/cpu.rs:558-581.
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "../../include/itak_cuda_compute.h"
#include "itkv_codec.hpp"
#include "kernels.cuh"

namespace itk {
cudaError_t configure_decode_f16();
cudaError_t configure_verify_f16();
cudaError_t configure_verify_tc();
uint32_t verify_pair_chunks(uint32_t rows, uint32_t group);
}

#ifdef ITK_DECODE_TRACE
extern "C" int itk_debug_trace_buffer(void** dev_ptr, uint64_t* bytes);
#endif

namespace {

using itk::AppendLaunch;
using itk::AttnLaunch;
#ifdef ITK_DECODE_TRACE
// Timeline build only: [layer][512 CTAs][16] stamps, allocated on request.
static unsigned long long* g_trace = nullptr;
#endif
using itk::CopyLaunch;
using itk::SeqDesc;

std::string g_create_error;
std::atomic<uint64_t> g_next_cache_id{1};  // crates/attention/src/cache.rs:32

std::string zu(uint64_t v) { return std::to_string(v); }

struct SlotState {
    uint64_t id = 0;
    bool built = false;  // the reference builds its KV state lazily at the first forward
    std::vector<uint64_t> appended;
    bool live = false;
    uint64_t next_serial = 0;
    uint64_t live_serial = 0;
    uint64_t max_round = 0;
    std::vector<uint64_t> bases;
};

constexpr size_t kPartCellSplits = 148 * 64;  // (cell, split) partials the scratch holds
constexpr size_t kGatherHeader = 4096, kGatherErr = 2048, kGatherBase = 2176;  // layout of a gather buffer's header

}  // namespace

struct itk_snapshot {
    int device = 0;
    bool f16 = false;
    uint32_t kv_heads = 0, head_dim = 0;
    std::vector<uint32_t> window;  // per layer, 0 = global
    uint64_t token_count = 0;
    std::vector<uint64_t> first, rows;  // per layer
    std::vector<uint64_t> k_off, v_off;  // element offsets inside `data`
    uint64_t total_elems = 0;
    void* data = nullptr;
};

struct itk_backend {
    itk_config cfg{};
    std::vector<uint32_t> window, ring;
    std::vector<size_t> layer_off;  // element offset of each layer inside a slab
    size_t slab_elems = 0;
    bool f16 = false;
    uint32_t elem_bytes = 4;
    uint32_t group = 1, gchunks = 1;
    void* k_slab = nullptr;
    void* v_slab = nullptr;
    cudaStream_t own_stream = nullptr, stream = nullptr;
    float* part_o = nullptr;
    float* part_ml = nullptr;
    unsigned int* tickets = nullptr;
    float* acc_o = nullptr;  // fused-sum accumulators of the resident decode loop: [ticket_cells][8][head_dim], [..][8]
    float* acc_l = nullptr;
    unsigned int* acc_flag = nullptr;
    bool fused_sum = true;   // option decode_fused_sum = 0: cells shared by many CTAs are merged from the stored parts
    size_t ticket_cells = 0;
    float *d_q = nullptr, *d_k = nullptr, *d_v = nullptr, *d_out = nullptr;
    size_t stage_rows = 0;
    void* gather_buf = nullptr;
    size_t gather_bytes = 0;
    std::vector<SlotState> slots;
    mutable std::string err;
    itk_stats stats{};
    int sm_count = 148;
    int forced_splits = 0;
    int forced_ctas = 0;         // option decode_ctas: persistent CTAs of the decode kernel (default 2 per SM)
    uint32_t tc_wait_kclocks = 0;  // option tc_wait_kclocks: bound of the tcgen05 kernel's waits (0 = default)
    bool tc_withhold = false;      // option tc_withhold_first_tile: tests of the give-up path
    uint64_t fw_loop_bytes = 8ull << 20;  // option layers_host_decode_loop: decode steps from host buffers that upload no more run as one step of the replayable loop
    uint64_t fw_bulk_bytes = 1ull << 20;  // option layers_host_bulk_bytes: forwards that upload no more take the bulk path
    bool separate_append = false;  // option separate_append = 1: decode steps launch the append kernel separately
    bool force_general = false;  // option force_general = 1: multi-row launches take the CUDA-core kernel (A/B checks)
    bool verify_tc = true;       // option verify_tc = 0: multi-row launches take the mma.sync kernel instead of tcgen05
    unsigned int* d_status = nullptr;  // device word kernels OR error bits into
    unsigned int* h_status = nullptr;  // pinned host copy read after a synchronisation
    bool status_pending = false;       // a kernel that can raise d_status was launched since the last check
    // resident decode loop (device-side sequence states, replayable)
    itk::SeqState* d_states = nullptr;
    bool res_active = false;
    std::vector<uint32_t> res_slots;
    uint64_t res_max_steps = 0;
    uint32_t res_ctas = 0, res_parts = 0;
    uint32_t res_launches_in_step = 0;
    // two-lane schedule of the loop's gathering launches (see GatherTarget): 1 = off
    uint32_t res_lanes = 1, res_lane_split = 0, res_lane_ctas = 0;
    int lanes_mode = 1;        // option decode_lanes: 0 = never, 1 = when a launch is short enough to gain, 2 = whenever possible
    int lane_stagger = 100;    // option decode_lane_stagger: how far lane 1 of a step's first launch starts behind lane 0,
                               // in per cent of the time lane 0 needs to stream its keys (0 = together)
    uint64_t res_lane0_tiles = 0;  // 64-key tiles of lane 0 in one launch when the loop began
    // The uninterrupted run of tcgen05 multi-row launches at the end of the stream's queue: the layers they cover.
    // A further launch on a layer outside it may stream its stored K/V before its predecessor completes (nothing that
    // can still be running writes that layer's cache); any other queued work that writes the cache ends the run.
    uint64_t tc_chain_mask = 0;
    bool tc_chain_live = false;
    unsigned char* lane_hdr = nullptr;  // arrival counters of a single-GPU loop run in lanes (a gather header without data)
    uint32_t* d_plan = nullptr;  // the decode kernel's work plan of the loop's current positions (device words)
    itk::DecodePlanSpec res_spec{};
    bool res_planned = false;    // the plan is kept on the device (all layers global)
    // fused gather: one allocation per rank = [kGatherHeader bytes: arrival counters [64 sequences][8 ranks], status word
    // @kGatherErr, loop base position @kGatherBase][data]
    unsigned char* gth_local = nullptr;
    unsigned char* gth_peer[itk::kMaxPeers] = {};
    bool gth_attached[itk::kMaxPeers] = {};  // the caller's mapping (itk_gather_attach): not closed by the backend
    uint32_t gth_world = 0, gth_rank = 0;
    uint64_t gth_bytes = 0;
    uint32_t gth_poll_limit = 200000;  // option gather_poll_limit: polls of a peer's arrival flag before giving up
    int res_prev_layer = -1;  // layer of the loop's previous launch on the stream, -1 = something else
    bool use_pdl = true;      // option pdl = 0 turns programmatic dependent launch off
    // attention preparation (per-head RMSNorm + rotary rotation), configured per layer
    struct LayerPrep {
        bool set = false;
        float* q_w = nullptr;       // device [head_dim] or null
        float* k_w = nullptr;
        double* inv_freq = nullptr; // device [rotary_dim / 2] or null
        float eps = 0.f;
        uint32_t rotary_dim = 0, pairing = 0;
    };
    std::vector<LayerPrep> prep;
    float *d_qp = nullptr, *d_kp = nullptr;  // prepared rows, stage_rows each (allocated with the first config)
    // whole-forward host call: per-layer staging on the device, two copy streams and per-layer events (lazy)
    float *fw_q = nullptr, *fw_k = nullptr, *fw_v = nullptr, *fw_out = nullptr;
    size_t fw_rows = 0;  // rows (sequences x rows per sequence) each layer's staging holds
    cudaStream_t fw_in = nullptr, fw_outs = nullptr;
    std::vector<cudaEvent_t> fw_ev_in, fw_ev_k;
    cudaEvent_t fw_ev_prev = nullptr;
    // profiling: event pairs (start, stop) tagged 0 = attention, 1 = append, 2 = snapshot gather / restore scatter
    std::vector<cudaEvent_t> prof_events;
    std::vector<int> prof_tags;
    size_t prof_used = 0;
    double prof_copy_ms = 0.0;
    uint64_t prof_copy_launches = 0;

    int fail(int code, std::string msg) const {
        err = std::move(msg);
        return code;
    }
    int cuda_fail(cudaError_t e, const char* what) const {
        return fail(ITK_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
    }
    size_t row_len() const { return static_cast<size_t>(cfg.kv_heads) * cfg.head_dim; }
    size_t q_width() const { return static_cast<size_t>(cfg.q_heads) * cfg.head_dim; }
    uint64_t stored(uint32_t layer, uint64_t appended) const {
        return window[layer] ? (appended < window[layer] ? appended : window[layer]) : appended;
    }
    void* layer_ptr(void* slab, uint32_t layer) const {
        return static_cast<unsigned char*>(slab) + layer_off[layer] * elem_bytes;
    }
};

namespace {

#define ITK_CUDA(b, call, what)                                \
    do {                                                       \
        cudaError_t e_ = (call);                               \
        if (e_ != cudaSuccess) return (b)->cuda_fail(e_, what); \
    } while (0)

int check_slot(const itk_backend* b, uint32_t slot) {
    if (slot >= b->cfg.n_slots)
        return b->fail(ITK_ERR_INVALID_SLOT, "slot " + zu(slot) + " out of range, backend has " + zu(b->cfg.n_slots) + " slots");
    return ITK_OK;
}
int check_layer(const itk_backend* b, uint32_t layer) {
    if (layer >= b->cfg.n_layers)
        return b->fail(ITK_ERR_INVALID_LAYER,
                       "layer " + zu(layer) + " out of range, cache has " + zu(b->cfg.n_layers) + " layers");
    return ITK_OK;
}

// KV splits for a decode launch: minimise waves x (tiles per CTA + fixed cost)
// over the CTA slots the device offers (2 resident CTAs per SM).
uint32_t choose_splits(const itk_backend* b, uint64_t cells, uint64_t n_max, uint32_t tile, uint64_t scratch_mult = 1,
                       uint32_t ctas_per_sm = 2, uint32_t min_tiles = 4) {
    if (b->forced_splits > 0) {
        uint64_t s = static_cast<uint64_t>(b->forced_splits);
        const uint64_t by_len = (n_max + tile - 1) / tile;
        if (s > by_len) s = by_len;
        if (s * cells * scratch_mult > kPartCellSplits) s = kPartCellSplits / (cells * scratch_mult);
        if (s > 256) s = 256;
        return static_cast<uint32_t>(s < 1 ? 1 : s);
    }
    const uint64_t slots = static_cast<uint64_t>(b->sm_count) * ctas_per_sm;
    uint64_t max_s = (n_max + min_tiles * tile - 1) / (min_tiles * tile);  // at least min_tiles tiles per CTA
    if (max_s < 1) max_s = 1;
    if (max_s > 256) max_s = 256;
    if (cells == 0) return 1;
    if (max_s * cells * scratch_mult > kPartCellSplits) max_s = kPartCellSplits / (cells * scratch_mult);
    if (max_s < 1) max_s = 1;
    uint64_t best = 1;
    double best_cost = 1e300;
    for (uint64_t s = 1; s <= max_s; ++s) {
        const uint64_t ctas = cells * s;
        const uint64_t waves = (ctas + slots - 1) / slots;
        const uint64_t per = (n_max + s - 1) / s;
        const uint64_t tiles = (per + tile - 1) / tile;
        const double cost = static_cast<double>(waves) * (static_cast<double>(tiles) + 3.0);
        if (cost < best_cost - 1e-9) {
            best_cost = cost;
            best = s;
        }
    }
    return static_cast<uint32_t>(best);
}

// How a decode batch of `n_seqs` sequences with `cells_per_seq` (KV head x head chunk) cells each is cut into
// launches so that the split scratch (kPartCellSplits partial slots) is never overrun: stream-K can cut any cell in
// two, so every cell of a launch needs at least two slots.  *seqs_per_launch = sequences one launch may carry,
// *parts_per_cell = partial slots each of its cells then owns (2..kDecodeMaxParts).  False when even one sequence
// does not fit.
bool decode_batch_limits(uint32_t n_seqs, uint32_t cells_per_seq, uint32_t* seqs_per_launch, uint32_t* parts_per_cell) {
    if (n_seqs == 0 || cells_per_seq == 0 || 2ull * cells_per_seq > kPartCellSplits) return false;
    uint64_t fit = kPartCellSplits / (2ull * cells_per_seq);
    if (fit > static_cast<uint64_t>(itk::kMaxSeqsPerLaunch)) fit = itk::kMaxSeqsPerLaunch;
    if (fit > n_seqs) fit = n_seqs;
    uint64_t parts = kPartCellSplits / (fit * cells_per_seq);
    if (parts > itk::kDecodeMaxParts) parts = itk::kDecodeMaxParts;
    *seqs_per_launch = static_cast<uint32_t>(fit);
    *parts_per_cell = static_cast<uint32_t>(parts);
    return true;
}

// Event pair around one kernel launch while profiling is on; returns the pair's index or -1.
long prof_begin(itk_backend* b, int tag) {
    if (b->prof_used + 2 > b->prof_events.size()) return -1;
    const long at = static_cast<long>(b->prof_used);
    b->prof_used += 2;
    b->prof_tags[at / 2] = tag;
    cudaEventRecord(b->prof_events[at], b->stream);
    return at;
}
void prof_end(itk_backend* b, long at) {
    if (at >= 0) cudaEventRecord(b->prof_events[at + 1], b->stream);
}

void fill_layer_view(const itk_backend* b, uint32_t layer, itk::LayerView* v) {
    v->k = b->layer_ptr(b->k_slab, layer);
    v->v = b->layer_ptr(b->v_slab, layer);
    v->ring = b->ring[layer];
    v->window = b->window[layer];
    v->kv_heads = b->cfg.kv_heads;
    v->head_dim = b->cfg.head_dim;
}

// Launch the append kernel for `n` sequences (device sources).
int run_append(itk_backend* b, uint32_t layer, uint32_t n, const SeqDesc* seqs, uint32_t rows, const float* d_k,
               const float* d_v) {
    b->tc_chain_live = false;
    for (uint32_t at = 0; at < n; at += itk::kMaxSeqsPerLaunch) {
        const uint32_t m = (n - at < static_cast<uint32_t>(itk::kMaxSeqsPerLaunch)) ? n - at : itk::kMaxSeqsPerLaunch;
        AppendLaunch p{};
        p.k = b->layer_ptr(b->k_slab, layer);
        p.v = b->layer_ptr(b->v_slab, layer);
        p.k_src = d_k + static_cast<size_t>(at) * rows * b->row_len();
        p.v_src = d_v + static_cast<size_t>(at) * rows * b->row_len();
        p.ring = b->ring[layer];
        p.kv_heads = b->cfg.kv_heads;
        p.head_dim = b->cfg.head_dim;
        p.rows = rows;
        p.n_seqs = m;
        for (uint32_t i = 0; i < m; ++i) p.seq[i] = seqs[at + i];
        const long ev = prof_begin(b, 1);
        ITK_CUDA(b, itk::launch_append(p, b->f16, b->stream, &b->stats.kernel_launches), "append launch");
        prof_end(b, ev);
    }
    return ITK_OK;
}

// The kernels' error word: queued for download before a synchronisation that follows a launch able to raise it,
// and turned into a named refusal afterwards (the word is cleared so that later calls start clean).
void queue_status_read(itk_backend* b) {
    if (b->status_pending)
        cudaMemcpyAsync(b->h_status, b->d_status, sizeof(unsigned int), cudaMemcpyDeviceToHost, b->stream);
}
int check_status(itk_backend* b) {
    if (!b->status_pending) return ITK_OK;
    b->status_pending = false;
    if (*b->h_status == 0u) return ITK_OK;
    *b->h_status = 0u;
    cudaMemsetAsync(b->d_status, 0, sizeof(unsigned int), b->stream);
    return b->fail(ITK_ERR_CUDA, "a bounded wait on the tensor core ran out in the multi-row attention kernel; "
                                 "the launch's outputs are not valid");
}

// Launch attention for `n` sequences of `rows` rows each (device q / out).
// `d_k_new` / `d_v_new` (device f32 [n][rows][kv_heads*D], may be null): the launch's new rows for the decode or
// the tcgen05 multi-row kernel to store itself (see decode_fuses_append, verify_fuses_append).
int run_attention(itk_backend* b, uint32_t layer, uint32_t n, const SeqDesc* seqs, uint32_t rows, const float* d_q,
                  float* d_out, const float* d_k_new = nullptr, const float* d_v_new = nullptr) {
    const uint32_t D = b->cfg.head_dim;
    const uint32_t HY = b->cfg.kv_heads * b->gchunks;
    const bool decode = b->f16 && itk::decode_f16_supported(D, rows);
    const bool verify_tc = b->f16 && !decode && !b->force_general && b->verify_tc &&
                           itk::verify_tc_supported(D, rows, b->group);
    const bool verify = !verify_tc && b->f16 && !decode && !b->force_general &&
                        itk::verify_f16_supported(D, rows, b->group);
    const bool f32_tc = !b->f16 && !b->force_general && itk::attn_f32_supported(D, rows);
    const uint32_t f32_pairs = f32_tc ? itk::attn_f32_pairs_per_cta(rows, b->group) : 0u;
    // grid.z carries n_seqs * rows (general kernel) and is limited to 65535
    uint32_t per_launch = itk::kMaxSeqsPerLaunch;
    while (per_launch > 1 && static_cast<uint64_t>(per_launch) * rows > 65535) per_launch >>= 1;
    if (static_cast<uint64_t>(rows) > 65535)
        return b->fail(ITK_ERR_CAPACITY, "attention: " + zu(rows) + " rows exceed one launch's 65535-row limit");
    if (decode) {
        uint32_t fit = 0, parts = 0;
        if (!decode_batch_limits(n, HY, &fit, &parts))
            return b->fail(ITK_ERR_CAPACITY, "attention: " + zu(HY) + " head cells per sequence exceed the split scratch of " +
                                                 zu(kPartCellSplits) + " partial slots");
        if (per_launch > fit) per_launch = fit;
    }
    for (uint32_t at = 0; at < n; at += per_launch) {
        const uint32_t m = (n - at < per_launch) ? n - at : per_launch;
        AttnLaunch p{};
        fill_layer_view(b, layer, &p.layer);
        p.q = d_q + static_cast<size_t>(at) * rows * b->q_width();
        p.out = d_out + static_cast<size_t>(at) * rows * b->q_width();
        p.part_o = b->part_o;
        p.part_ml = b->part_ml;
        p.tickets = b->tickets;
        p.status = b->d_status;
        p.q_heads = b->cfg.q_heads;
        p.group = b->group;
        p.gchunks = b->gchunks;
        p.rows = rows;
        p.n_seqs = m;
        p.scale = 1.0f / sqrtf(static_cast<float>(D));
        uint64_t n_max = 0, keys = 0;
        for (uint32_t i = 0; i < m; ++i) {
            p.seq[i] = seqs[at + i];
            const uint64_t span = p.seq[i].kv_hi - p.seq[i].kv_lo;
            if (span > n_max) n_max = span;
            keys += span;  // every stored row the launch can see is streamed once per KV head
        }
        // A "cell" is one (unit, head chunk) whose splits are merged: a (sequence, row) for the decode and
        // general kernels, a (sequence, block of 32 row-head pairs) for the verify kernel, which needs four
        // times the scratch per (cell, split).
        const uint64_t cells = verify_tc ? static_cast<uint64_t>(m) * HY * itk::verify_tc_pair_chunks(rows, b->group)
                               : verify  ? static_cast<uint64_t>(m) * HY * itk::verify_pair_chunks(rows, b->group)
                               : f32_tc  ? static_cast<uint64_t>(m) * HY * itk::attn_f32_pair_chunks(rows, b->group)
                                         : static_cast<uint64_t>(m) * rows * HY;
        if (cells > b->ticket_cells)
            return b->fail(ITK_ERR_CAPACITY, "attention: " + zu(cells) + " (row, head) cells exceed the scratch of " +
                                                 zu(b->ticket_cells));
        b->stats.kv_bytes_read += keys * b->cfg.kv_heads * D * 2ull * b->elem_bytes;
        const long ev = prof_begin(b, 0);
        if (!verify_tc) b->tc_chain_live = false;
        if (decode) {
            if (d_k_new) {
                p.k_new = d_k_new + static_cast<size_t>(at) * b->row_len();
                p.v_new = d_v_new + static_cast<size_t>(at) * b->row_len();
            }
            uint64_t max_parts = kPartCellSplits / cells;
            if (max_parts > itk::kDecodeMaxParts) max_parts = itk::kDecodeMaxParts;
            const uint32_t ctas = b->forced_ctas > 0 ? static_cast<uint32_t>(b->forced_ctas)
                                                     : 2u * static_cast<uint32_t>(b->sm_count);
            uint32_t parts = 0;
            ITK_CUDA(b, itk::launch_decode_f16(p, ctas, static_cast<uint32_t>(max_parts), b->stream,
                                               &b->stats.kernel_launches, &parts),
                     "decode attention launch");
            b->stats.last_splits = parts;
            prof_end(b, ev);
            continue;
        }
        if (verify_tc) {
            // one CTA per SM; a partial slot holds verify_tc_pairs_per_cta rows instead of 8
            p.splits = choose_splits(b, cells, n_max, 64, itk::verify_tc_pairs_per_cta(rows, b->group) / 8, 1);
            b->stats.last_splits = p.splits;
            if (d_k_new) {
                p.k_new = d_k_new + static_cast<size_t>(at) * rows * b->row_len();
                p.v_new = d_v_new + static_cast<size_t>(at) * rows * b->row_len();
            }
            b->status_pending = true;
            p.tc_wait_kclocks = b->tc_wait_kclocks;
            p.tc_withhold = b->tc_withhold ? 1u : 0u;
            // behind an unbroken run of this kernel's launches on other layers, the K/V stream may start early
            const bool early = b->use_pdl && b->tc_chain_live && layer < 64 && ((b->tc_chain_mask >> layer) & 1ull) == 0 &&
                               b->prof_events.empty();
            p.pdl = !b->use_pdl ? 0u : (early ? 2u : 1u);
            if (!early) b->tc_chain_mask = 0;
            b->tc_chain_live = layer < 64;
            if (layer < 64) b->tc_chain_mask |= 1ull << layer;
#ifdef ITK_DECODE_TRACE
            p.trace = g_trace;
#endif
            ITK_CUDA(b, itk::launch_verify_tc(p, b->stream, &b->stats.kernel_launches), "tensor-core attention launch");
            prof_end(b, ev);
            continue;
        }
        if (f32_tc) {
            // a slot of its scratch holds f32_pairs rows instead of 8; a decode block's CTAs may take a single 32-key
            // tile each (the launch is latency-bound), a prefill block's at least four.  A block whose causal range
            // is shorter than the longest one takes fewer parts (the kernel cuts every range into parts of one size).
            // Under the causal bound a block of a long chunk walks, on average, the stored history plus half the
            // chunk: the CTA count that fills the machine is estimated from that share of the cells.
            uint64_t busy_cells = cells;
            if (f32_pairs == 64 && n_max > 0) {
                const uint64_t mean = n_max > rows / 2 ? n_max - rows / 2 : 1;
                busy_cells = (cells * mean + n_max - 1) / n_max;
                if (busy_cells < 1) busy_cells = 1;
            }
            p.splits = choose_splits(b, busy_cells, n_max, 32, 0, D == 64 ? 4 : 2, f32_pairs == 16 ? 1 : 4);
            while (p.splits > 1 && static_cast<uint64_t>(p.splits) * cells * (f32_pairs / 8) > kPartCellSplits) --p.splits;
            if (p.splits > itk::attn_f32_max_parts()) p.splits = itk::attn_f32_max_parts();
            b->stats.last_splits = p.splits;
            if (d_k_new) {
                p.k_new = d_k_new + static_cast<size_t>(at) * rows * b->row_len();
                p.v_new = d_v_new + static_cast<size_t>(at) * rows * b->row_len();
            }
            ITK_CUDA(b, itk::launch_attn_f32(p, b->stream, &b->stats.kernel_launches), "f32 attention launch");
            prof_end(b, ev);
            continue;
        }
        p.splits = choose_splits(b, cells, n_max, verify ? 64 : 128, verify ? 4 : 1);
        b->stats.last_splits = p.splits;
        if (verify)
            ITK_CUDA(b, itk::launch_verify_f16(p, b->stream, &b->stats.kernel_launches), "verify attention launch");
        else
            ITK_CUDA(b, itk::launch_attn_general(p, b->f16, b->stream, &b->stats.kernel_launches),
                     "attention launch");
        prof_end(b, ev);
    }
    return ITK_OK;
}

// A decode step (one row per sequence, f16 cache, head_dim 64 or 128) lets the attention kernel store the new
// row itself; the option separate_append = 1 keeps the two-launch form for A/B checks.
bool decode_fuses_append(const itk_backend* b, uint32_t rows) {
    return b->f16 && !b->separate_append && (b->cfg.head_dim % 8 == 0) && itk::decode_f16_supported(b->cfg.head_dim, rows);
}

// So does the tcgen05 multi-row kernel for a short block (its loader warps convert the block's rows on their way
// into the staged tiles and store them).  A long chunk's rows are most of what its tiles hold, and converting them
// in the two loader warps of every CTA that reads them costs far more than the append kernel's launch: from
// kVerifyFuseMaxRows rows on, the rows are appended first and every tile comes from the cache.
constexpr uint32_t kVerifyFuseMaxRows = 64;
bool verify_fuses_append(const itk_backend* b, uint32_t rows) {
    return b->f16 && !b->separate_append && !b->force_general && b->verify_tc && rows > 1 && rows <= kVerifyFuseMaxRows &&
           itk::verify_tc_supported(b->cfg.head_dim, rows, b->group);
}

// Shared validation of one attention step; fills `seqs`.  Mirrors
// crates/cpu-compute/src/cpu.rs:558-581 (position cross-check) and
// crates/attention/src/cache.rs:445-471 (checkpoint range) before anything moves.
int validate_step(itk_backend* b, uint32_t layer, uint32_t n_seqs, const uint32_t* slots, const uint64_t* positions,
                  uint32_t rows, std::vector<SeqDesc>* seqs) {
    if (int rc = check_layer(b, layer)) return rc;
    if (n_seqs == 0 || rows == 0) return b->fail(ITK_ERR_INVALID_ARGUMENT, "attention: zero sequences or zero rows");
    if (rows > b->cfg.chunk_cap)
        return b->fail(ITK_ERR_CAPACITY, "attention: " + zu(rows) + " rows exceed the backend's chunk cap of " +
                                             zu(b->cfg.chunk_cap) + "; forward in chunks");
    if (n_seqs > b->cfg.n_slots)
        return b->fail(ITK_ERR_INVALID_ARGUMENT, "attention: more sequences than slots");
    seqs->resize(n_seqs);
    for (uint32_t i = 0; i < n_seqs; ++i) {
        if (int rc = check_slot(b, slots[i])) return rc;
        for (uint32_t j = 0; j < i; ++j)
            if (slots[j] == slots[i])
                return b->fail(ITK_ERR_INVALID_ARGUMENT, "attention: slot " + zu(slots[i]) + " listed twice");
        const SlotState& st = b->slots[slots[i]];
        const uint64_t appended = st.appended[layer];
        const uint64_t start = positions[i];
        if (appended != start)
            return b->fail(ITK_ERR_STEP_FAILED,
                           "attention: KV state for layer " + zu(layer) + " is at position " + zu(appended) +
                               " but the sequence cache is at position " + zu(start) +
                               ": the two disagree, so attending would read the wrong history. Pair one Cache with "
                               "one slot per sequence, or call itk_reset when a sequence is abandoned");
        if (st.live) {
            const uint64_t limit = st.bases[layer] + st.max_round;
            if (start + rows > limit) {
                const uint64_t bad = start > limit ? start : limit;
                return b->fail(ITK_ERR_CHECKPOINT_RANGE_EXCEEDED,
                               "attention: layer " + zu(layer) + " append at position " + zu(bad) +
                                   " is outside the live checkpoint's saved range (first unsaved position " + zu(limit) +
                                   "); refusing so a later rewind cannot meet a slot it cannot restore");
            }
        }
        if (b->window[layer] == 0 && start + rows > b->ring[layer])
            return b->fail(ITK_ERR_CAPACITY, "attention: position " + zu(start + rows) + " is past the slot's context "
                                             "capacity of " + zu(b->ring[layer]) + " positions");
        if (start + rows > 0xfffffff0ull) return b->fail(ITK_ERR_CAPACITY, "attention: position exceeds 32 bits");
        SeqDesc d;
        d.slot = slots[i];
        d.q_pos0 = static_cast<uint32_t>(start);
        d.kv_hi = static_cast<uint32_t>(start + rows);
        d.kv_lo = 0;
        if (b->window[layer] && start + 1 > b->window[layer]) d.kv_lo = static_cast<uint32_t>(start + 1 - b->window[layer]);
        (*seqs)[i] = d;
    }
    return ITK_OK;
}

// The device buffers of a call must start on 16-byte boundaries (the kernels move them as 16-byte vectors):
// a named refusal instead of a misaligned-address fault.
template <typename... P>
int check_device_alignment(itk_backend* b, const char* what, P... ptrs) {
    const uintptr_t all = (... | reinterpret_cast<uintptr_t>(ptrs));
    if ((all & 15u) != 0)
        return b->fail(ITK_ERR_INVALID_ARGUMENT, std::string(what) + ": device buffers must be 16-byte aligned");
    return ITK_OK;
}

// And the tensor-core kernel of an f32 cache, for any number of rows (the append is a plain copy there).
bool f32_fuses_append(const itk_backend* b, uint32_t rows) {
    return !b->f16 && !b->separate_append && !b->force_general && itk::attn_f32_supported(b->cfg.head_dim, rows);
}

int step_device(itk_backend* b, uint32_t layer, uint32_t n_seqs, const uint32_t* slots, const uint64_t* positions,
                uint32_t rows, const float* d_q, const float* d_k, const float* d_v, float* d_out) {
    std::vector<SeqDesc> seqs;
    if (int rc = validate_step(b, layer, n_seqs, slots, positions, rows, &seqs)) return rc;
    const bool fuse = decode_fuses_append(b, rows) || verify_fuses_append(b, rows) || f32_fuses_append(b, rows);
    if (!fuse)
        if (int rc = run_append(b, layer, n_seqs, seqs.data(), rows, d_k, d_v)) return rc;
    // The positions move only once the launch that stores the rows (the fused kernels) has been queued: a refused
    // or failed launch leaves the slot where it was (the reference validates before any state moves,
    // crates/cpu-compute/src/cpu.rs:558-581).
    if (int rc = run_attention(b, layer, n_seqs, seqs.data(), rows, d_q, d_out, fuse ? d_k : nullptr, fuse ? d_v : nullptr))
        return rc;
    for (uint32_t i = 0; i < n_seqs; ++i) {
        SlotState& st = b->slots[slots[i]];
        st.appended[layer] += rows;
        st.built = true;
    }
    b->stats.rows_appended += static_cast<uint64_t>(n_seqs) * rows;
    b->stats.attention_calls += 1;
    return ITK_OK;
}

int ensure_gather(itk_backend* b, size_t bytes) {
    if (bytes <= b->gather_bytes) return ITK_OK;
    if (b->gather_buf) cudaFree(b->gather_buf);
    b->gather_buf = nullptr;
    b->gather_bytes = 0;
    ITK_CUDA(b, cudaMalloc(&b->gather_buf, bytes), "gather buffer allocation");
    b->gather_bytes = bytes;
    return ITK_OK;
}

// Gather or scatter layers [l0, l1) of one slot between the slabs and `snap_base`.
int run_copy(itk_backend* b, uint32_t slot, void* snap_base, const std::vector<uint32_t>& layers,
             const std::vector<uint64_t>& first, const std::vector<uint64_t>& rows, const std::vector<uint64_t>& k_off,
             const std::vector<uint64_t>& v_off, bool to_snapshot) {
    b->tc_chain_live = false;
    const uint32_t row_bytes = b->cfg.head_dim * b->elem_bytes;
    const uint32_t vb = (row_bytes % 16 == 0) ? 16 : b->elem_bytes;
    const uint64_t units_per_row = static_cast<uint64_t>(b->cfg.kv_heads) * (row_bytes / vb);
    for (size_t at = 0; at < layers.size(); at += itk::kMaxLayersPerLaunch) {
        const size_t m = (layers.size() - at < static_cast<size_t>(itk::kMaxLayersPerLaunch)) ? layers.size() - at
                                                                                               : itk::kMaxLayersPerLaunch;
        CopyLaunch p{};
        p.k_slab = b->k_slab;
        p.v_slab = b->v_slab;
        p.snap = snap_base;
        p.slot = slot;
        p.kv_heads = b->cfg.kv_heads;
        p.head_dim = b->cfg.head_dim;
        p.n_layers = static_cast<uint32_t>(m);
        p.elem_bytes = b->elem_bytes;
        p.to_snapshot = to_snapshot ? 1 : 0;
        p.vec_prefix[0] = 0;
        for (size_t i = 0; i < m; ++i) {
            const uint32_t l = layers[at + i];
            p.layer[i].slab_off = b->layer_off[l];
            p.layer[i].snap_k = k_off[at + i];
            p.layer[i].snap_v = v_off[at + i];
            p.layer[i].ring = b->ring[l];
            p.layer[i].first_pos = static_cast<uint32_t>(first[at + i]);
            p.layer[i].rows = static_cast<uint32_t>(rows[at + i]);
            p.vec_prefix[i + 1] = p.vec_prefix[i] + ((rows[at + i] + 7) / 8) * units_per_row;  // 8-row work items
        }
        p.total_vec = 2 * p.vec_prefix[m];
        const long ev = prof_begin(b, 2);
        ITK_CUDA(b, itk::launch_snapshot_copy(p, b->stream, &b->stats.kernel_launches), "snapshot copy launch");
        prof_end(b, ev);
    }
    return ITK_OK;
}

void drop_slot(itk_backend* b, uint32_t slot) {
    SlotState& st = b->slots[slot];
    st.id = g_next_cache_id.fetch_add(1);
    st.built = false;
    st.appended.assign(b->cfg.n_layers, 0);
    st.live = false;
    st.next_serial = 0;
    st.bases.clear();
}

// crates/attention/src/cache.rs:719-728
int check_live(const itk_backend* b, const SlotState& st, const itk_checkpoint* cp) {
    if (st.live && st.live_serial == cp->serial && cp->id == st.id) return ITK_OK;
    return b->fail(ITK_ERR_STALE_CHECKPOINT, "checkpoint " + zu(cp->serial) +
                                                 " is not this cache's live checkpoint (already released or foreign)");
}

}  // namespace

extern "C" {

int itk_backend_create(const itk_config* cfg, itk_backend** out) {
    auto refuse = [](int code, std::string msg) {
        g_create_error = std::move(msg);
        return code;
    };
    if (!cfg || !out) return refuse(ITK_ERR_INVALID_ARGUMENT, "null config or output pointer");
    if (cfg->n_layers == 0) return refuse(ITK_ERR_ZERO_DIMENSION, "layer pattern must be positive, got 0");
    if (cfg->kv_heads == 0) return refuse(ITK_ERR_ZERO_DIMENSION, "num_kv_heads must be positive, got 0");
    if (cfg->head_dim == 0) return refuse(ITK_ERR_ZERO_DIMENSION, "head_dim must be positive, got 0");
    if (cfg->q_heads == 0) return refuse(ITK_ERR_ZERO_DIMENSION, "num_q_heads must be positive, got 0");
    if (cfg->q_heads % cfg->kv_heads != 0)
        return refuse(ITK_ERR_NON_DIVISIBLE_HEADS, zu(cfg->q_heads) + " query heads do not divide evenly across " +
                                                       zu(cfg->kv_heads) + " KV heads");
    if (cfg->n_slots == 0) return refuse(ITK_ERR_ZERO_DIMENSION, "n_slots must be positive, got 0");
    if (cfg->max_context == 0) return refuse(ITK_ERR_ZERO_DIMENSION, "max_context must be positive, got 0");
    if (cfg->chunk_cap == 0) return refuse(ITK_ERR_ZERO_DIMENSION, "chunk_cap must be positive, got 0");
    if (cfg->kv_dtype != ITK_KV_F32 && cfg->kv_dtype != ITK_KV_F16)
        return refuse(ITK_ERR_INVALID_ARGUMENT, "kv_dtype must be ITK_KV_F32 or ITK_KV_F16");
    if (cfg->head_dim > 256) return refuse(ITK_ERR_CAPACITY, "head_dim above 256 is not supported");

    itk_backend* b = new (std::nothrow) itk_backend();
    if (!b) return refuse(ITK_ERR_CUDA, "out of host memory");
    b->cfg = *cfg;
    b->cfg.layer_window = nullptr;
    b->f16 = cfg->kv_dtype == ITK_KV_F16;
    b->elem_bytes = b->f16 ? 2 : 4;
    b->group = cfg->q_heads / cfg->kv_heads;
    b->gchunks = (b->group + itk::kHeadsPerCta - 1) / itk::kHeadsPerCta;
    const uint64_t row = static_cast<uint64_t>(cfg->kv_heads) * cfg->head_dim;
    uint64_t total = 0;
    for (uint32_t l = 0; l < cfg->n_layers; ++l) {
        const uint32_t w = cfg->layer_window ? cfg->layer_window[l] : 0;
        uint64_t ring = w ? static_cast<uint64_t>(w) + cfg->chunk_cap : cfg->max_context;
        if (ring > 0xfffffff0ull) {
            delete b;
            return refuse(ITK_ERR_SIZE_OVERFLOW, "windowed layer storage: element count overflows");
        }
        b->window.push_back(w);
        b->ring.push_back(static_cast<uint32_t>(ring));
        b->layer_off.push_back(total);
        uint64_t layer_elems;
        if (__builtin_mul_overflow(ring * cfg->n_slots, row, &layer_elems) ||
            __builtin_add_overflow(total, layer_elems, &total) || total > (1ull << 46)) {
            delete b;
            return refuse(ITK_ERR_SIZE_OVERFLOW, "kv storage: element count overflows");
        }
    }
    b->slab_elems = total;

    auto cuda_refuse = [&](cudaError_t e, const char* what) {
        std::string msg = std::string(what) + ": " + cudaGetErrorString(e);
        itk_backend_destroy(b);
        return refuse(ITK_ERR_CUDA, msg);
    };
    cudaError_t e = cudaSetDevice(cfg->device);
    if (e != cudaSuccess) return cuda_refuse(e, "cudaSetDevice");
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, cfg->device);
    if (e != cudaSuccess) return cuda_refuse(e, "cudaGetDeviceProperties");
    if (prop.major != 10)
        return cuda_refuse(cudaErrorNoKernelImageForDevice, "this library carries sm_100a kernels only");
    b->sm_count = prop.multiProcessorCount;
    e = itk::configure_decode_f16();
    if (e == cudaSuccess) e = itk::configure_verify_f16();
    if (e == cudaSuccess) e = itk::configure_verify_tc();
    if (e == cudaSuccess) e = itk::configure_attn_f32();
    if (e != cudaSuccess) return cuda_refuse(e, "kernel attribute setup");
    e = cudaStreamCreateWithFlags(&b->own_stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) return cuda_refuse(e, "cudaStreamCreate");
    b->stream = b->own_stream;
    e = cudaMalloc(&b->k_slab, total * b->elem_bytes);
    if (e != cudaSuccess) return cuda_refuse(e, "K slab allocation");
    e = cudaMalloc(&b->v_slab, total * b->elem_bytes);
    if (e != cudaSuccess) return cuda_refuse(e, "V slab allocation");
    // Windowed rings start zero-filled like the reference's (cache.rs:139); global rows are written before read.
    for (uint32_t l = 0; l < cfg->n_layers; ++l)
        if (b->window[l]) {
            const size_t bytes = static_cast<size_t>(b->ring[l]) * cfg->n_slots * row * b->elem_bytes;
            cudaMemsetAsync(b->layer_ptr(b->k_slab, l), 0, bytes, b->stream);
            cudaMemsetAsync(b->layer_ptr(b->v_slab, l), 0, bytes, b->stream);
        }
    const uint32_t HY = cfg->kv_heads * b->gchunks;
    b->ticket_cells = static_cast<size_t>(cfg->n_slots) * cfg->chunk_cap * HY;
    if (b->ticket_cells < 64u * HY) b->ticket_cells = 64u * HY;
    e = cudaMalloc(&b->tickets, b->ticket_cells * sizeof(unsigned int));
    if (e != cudaSuccess) return cuda_refuse(e, "ticket allocation");
    cudaMemsetAsync(b->tickets, 0, b->ticket_cells * sizeof(unsigned int), b->stream);
    {
        const size_t ao = b->ticket_cells * itk::kHeadsPerCta * cfg->head_dim * sizeof(float);
        const size_t al = b->ticket_cells * itk::kHeadsPerCta * sizeof(float);
        if (cudaMalloc(&b->acc_o, ao) == cudaSuccess && cudaMalloc(&b->acc_l, al) == cudaSuccess &&
            cudaMalloc(&b->acc_flag, b->ticket_cells * sizeof(unsigned int)) == cudaSuccess) {
            cudaMemsetAsync(b->acc_o, 0, ao, b->stream);
            cudaMemsetAsync(b->acc_l, 0, al, b->stream);
            cudaMemsetAsync(b->acc_flag, 0, b->ticket_cells * sizeof(unsigned int), b->stream);
        } else {
            return cuda_refuse(cudaErrorMemoryAllocation, "fused-sum accumulator allocation");
        }
    }
    e = cudaMalloc(&b->part_o, kPartCellSplits * itk::kHeadsPerCta * cfg->head_dim * sizeof(float));
    if (e != cudaSuccess) return cuda_refuse(e, "partial-output scratch allocation");
    e = cudaMalloc(&b->part_ml, kPartCellSplits * itk::kHeadsPerCta * 2 * sizeof(float));
    if (e != cudaSuccess) return cuda_refuse(e, "partial-stat scratch allocation");
    b->stage_rows = static_cast<size_t>(cfg->n_slots) * cfg->chunk_cap;
    if (b->stage_rows < 64) b->stage_rows = 64;
    e = cudaMalloc(&b->d_q, b->stage_rows * b->q_width() * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&b->d_out, b->stage_rows * b->q_width() * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&b->d_k, b->stage_rows * b->row_len() * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&b->d_v, b->stage_rows * b->row_len() * sizeof(float));
    if (e != cudaSuccess) return cuda_refuse(e, "staging allocation");
    e = cudaMalloc(&b->d_states, itk::kMaxSeqsPerLaunch * sizeof(itk::SeqState));
    if (e != cudaSuccess) return cuda_refuse(e, "sequence-state allocation");
    e = cudaMalloc(&b->d_plan, (itk::kDecodePlanBlocks * itk::kDecodePlanWords + 4) * sizeof(uint32_t));
    if (e != cudaSuccess) return cuda_refuse(e, "plan allocation");
    e = cudaMalloc(&b->lane_hdr, kGatherHeader);
    if (e != cudaSuccess) return cuda_refuse(e, "lane counter allocation");
    cudaMemsetAsync(b->lane_hdr, 0, kGatherHeader, b->stream);
    e = cudaMalloc(&b->d_status, sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMallocHost(&b->h_status, sizeof(unsigned int));
    if (e != cudaSuccess) return cuda_refuse(e, "status word allocation");
    *b->h_status = 0u;
    cudaMemsetAsync(b->d_status, 0, sizeof(unsigned int), b->stream);
    e = cudaStreamSynchronize(b->stream);
    if (e != cudaSuccess) return cuda_refuse(e, "initialisation");
    b->slots.resize(cfg->n_slots);
    for (uint32_t s = 0; s < cfg->n_slots; ++s) drop_slot(b, s);
    *out = b;
    return ITK_OK;
}

void itk_backend_destroy(itk_backend* b) {
    if (!b) return;
    cudaSetDevice(b->cfg.device);
    if (b->stream) cudaStreamSynchronize(b->stream);
    cudaFree(b->k_slab);
    cudaFree(b->v_slab);
    cudaFree(b->tickets);
    cudaFree(b->acc_o);
    cudaFree(b->acc_l);
    cudaFree(b->acc_flag);
    for (auto& lp : b->prep) {
        cudaFree(lp.q_w);
        cudaFree(lp.k_w);
        cudaFree(lp.inv_freq);
    }
    cudaFree(b->d_qp);
    cudaFree(b->d_kp);
    cudaFree(b->part_o);
    cudaFree(b->part_ml);
    cudaFree(b->d_q);
    cudaFree(b->d_k);
    cudaFree(b->d_v);
    cudaFree(b->d_out);
    cudaFree(b->gather_buf);
    cudaFree(b->d_states);
    cudaFree(b->d_plan);
    cudaFree(b->lane_hdr);
    cudaFree(b->d_status);
    if (b->h_status) cudaFreeHost(b->h_status);
    for (uint32_t j = 0; j < itk::kMaxPeers; ++j)
        if (b->gth_peer[j] && j != b->gth_rank && !b->gth_attached[j]) cudaIpcCloseMemHandle(b->gth_peer[j]);
    cudaFree(b->gth_local);
    for (cudaEvent_t e : b->prof_events) cudaEventDestroy(e);
    cudaFree(b->fw_q);
    cudaFree(b->fw_k);
    cudaFree(b->fw_v);
    cudaFree(b->fw_out);
    for (cudaEvent_t e : b->fw_ev_in) cudaEventDestroy(e);
    for (cudaEvent_t e : b->fw_ev_k) cudaEventDestroy(e);
    if (b->fw_ev_prev) cudaEventDestroy(b->fw_ev_prev);
    if (b->fw_in) cudaStreamDestroy(b->fw_in);
    if (b->fw_outs) cudaStreamDestroy(b->fw_outs);
    if (b->own_stream) cudaStreamDestroy(b->own_stream);
    delete b;
}

const char* itk_last_error(const itk_backend* b) { return b ? b->err.c_str() : g_create_error.c_str(); }

int itk_set_stream(itk_backend* b, void* cuda_stream) {
    if (!b) return ITK_ERR_INVALID_ARGUMENT;
    b->stream = cuda_stream ? static_cast<cudaStream_t>(cuda_stream) : b->own_stream;
    return ITK_OK;
}

int itk_set_option(itk_backend* b, const char* name, int64_t value) {
    if (!b || !name) return ITK_ERR_INVALID_ARGUMENT;
    const std::string key(name);
    if (b->res_active) return b->fail(ITK_ERR_INVALID_ARGUMENT, "set_option: not while a resident loop is active");
    auto flag = [&](bool* field) {
        *field = value != 0;
        return ITK_OK;
    };
    if (key == "decode_splits" || key == "decode_ctas") {
        if (value < 0 || value > 4096) return b->fail(ITK_ERR_INVALID_ARGUMENT, "set_option: " + key + " must be 0..4096");
        (key == "decode_splits" ? b->forced_splits : b->forced_ctas) = static_cast<int>(value);
        return ITK_OK;
    }
    if (key == "decode_lanes") {
        if (value < 0 || value > 2) return b->fail(ITK_ERR_INVALID_ARGUMENT, "set_option: decode_lanes is 0, 1 or 2");
        b->lanes_mode = static_cast<int>(value);
        return ITK_OK;
    }
    if (key == "decode_lane_stagger") {
        if (value < 0 || value > 400) return b->fail(ITK_ERR_INVALID_ARGUMENT, "set_option: decode_lane_stagger is 0..400 (per cent)");
        b->lane_stagger = static_cast<int>(value);
        return ITK_OK;
    }
    if (key == "pdl") return flag(&b->use_pdl);
    if (key == "decode_fused_sum") return flag(&b->fused_sum);
    if (key == "separate_append") return flag(&b->separate_append);
    if (key == "force_general") return flag(&b->force_general);
    if (key == "verify_tc") return flag(&b->verify_tc);
    if (key == "gather_poll_limit") {
        if (value < 1 || value > 100000000) return b->fail(ITK_ERR_INVALID_ARGUMENT, "set_option: gather_poll_limit must be 1..1e8");
        b->gth_poll_limit = static_cast<uint32_t>(value);
        return ITK_OK;
    }
    if (key == "tc_wait_kclocks") {
        if (value < 0 || value > (1ll << 22)) return b->fail(ITK_ERR_INVALID_ARGUMENT, "set_option: tc_wait_kclocks must be 0..2^22");
        b->tc_wait_kclocks = static_cast<uint32_t>(value);
        return ITK_OK;
    }
    if (key == "tc_withhold_first_tile") return flag(&b->tc_withhold);
    if (key == "layers_host_decode_loop") {
        if (value < 0 || value > (1ll << 40)) return b->fail(ITK_ERR_INVALID_ARGUMENT, "set_option: layers_host_decode_loop must be 0..2^40");
        b->fw_loop_bytes = static_cast<uint64_t>(value);
        return ITK_OK;
    }
    if (key == "layers_host_bulk_bytes") {
        if (value < 0 || value > (1ll << 40)) return b->fail(ITK_ERR_INVALID_ARGUMENT, "set_option: layers_host_bulk_bytes must be 0..2^40");
        b->fw_bulk_bytes = static_cast<uint64_t>(value);
        return ITK_OK;
    }
    return b->fail(ITK_ERR_INVALID_ARGUMENT, "set_option: unknown option '" + key + "'");
}

int itk_synchronize(itk_backend* b) {
    if (!b) return ITK_ERR_INVALID_ARGUMENT;
    cudaSetDevice(b->cfg.device);
    queue_status_read(b);
    ITK_CUDA(b, cudaStreamSynchronize(b->stream), "synchronize");
    return check_status(b);
}

int itk_get_stats(const itk_backend* b, itk_stats* out) {
    if (!b || !out) return ITK_ERR_INVALID_ARGUMENT;
    *out = b->stats;
    return ITK_OK;
}

int itk_decode_plan(const uint32_t* keys, uint32_t n_seqs, uint32_t cells_per_seq, uint32_t ctas, uint32_t splits,
                    uint32_t* aligned, uint32_t* runs) {
    if (!keys || !aligned || !runs || n_seqs == 0 || n_seqs > static_cast<uint32_t>(itk::kMaxSeqsPerLaunch) ||
        cells_per_seq == 0 || ctas == 0)
        return ITK_ERR_INVALID_ARGUMENT;
    std::vector<uint32_t> cum(n_seqs + 1), first(n_seqs + 1);
    uint64_t total = 0;
    for (uint32_t s = 0; s < n_seqs; ++s) {
        if (keys[s] == 0) return ITK_ERR_INVALID_ARGUMENT;
        cum[s] = static_cast<uint32_t>(total);
        total += static_cast<uint64_t>((keys[s] + 63u) / 64u) * cells_per_seq;
        if (total > 0xffffffffull) return ITK_ERR_INVALID_ARGUMENT;
    }
    cum[n_seqs] = static_cast<uint32_t>(total);
    const uint32_t per = static_cast<uint32_t>((total + ctas - 1) / ctas);
    uint32_t worst = 0;
    const bool al = itk::decode_aligned_plan(keys, n_seqs, cells_per_seq, ctas, static_cast<uint32_t>(total), per, splits,
                                             first.data(), &worst);
    *aligned = al ? 1u : 0u;
    for (uint32_t c = 0; c < ctas; ++c) {
        itk::DecodeRun r = itk::decode_cta_run(al, c, keys, cum.data(), first.data(), n_seqs, cells_per_seq, per);
        if (!al && r.ntiles != 0) {
            const uint32_t T = (keys[r.seq] + 63u) / 64u;
            itk::decode_cell_parts(c, cum[r.seq] + r.hy * T, T, per, &r.parts, &r.part);
        }
        uint32_t* o = runs + 6ull * c;
        o[0] = r.seq;
        o[1] = r.hy;
        o[2] = r.tile;
        o[3] = r.ntiles;
        o[4] = r.parts;
        o[5] = r.part;
    }
    return ITK_OK;
}

int itk_decode_batch_limits(uint32_t n_seqs, uint32_t cells_per_seq, uint32_t* seqs_per_launch, uint32_t* parts_per_cell,
                            uint64_t* scratch_slots) {
    if (!seqs_per_launch || !parts_per_cell || !scratch_slots) return ITK_ERR_INVALID_ARGUMENT;
    *scratch_slots = kPartCellSplits;
    return decode_batch_limits(n_seqs, cells_per_seq, seqs_per_launch, parts_per_cell) ? ITK_OK : ITK_ERR_CAPACITY;
}

int itk_resident_begin(itk_backend* b, uint32_t n_seqs, const uint32_t* slots, uint64_t max_steps) {
    if (!b || !slots) return ITK_ERR_INVALID_ARGUMENT;
    cudaSetDevice(b->cfg.device);
    if (b->res_active) return b->fail(ITK_ERR_INVALID_ARGUMENT, "resident loop: already active; end it first");
    if (!(b->f16 && itk::decode_f16_supported(b->cfg.head_dim, 1)))
        return b->fail(ITK_ERR_INVALID_ARGUMENT, "resident loop: needs an f16 cache with head_dim 64 or 128");
    if (n_seqs == 0 || n_seqs > static_cast<uint32_t>(itk::kMaxSeqsPerLaunch) || max_steps == 0)
        return b->fail(ITK_ERR_INVALID_ARGUMENT, "resident loop: 1..64 sequences and at least one step");
    std::vector<itk::SeqState> states(n_seqs);
    const uint32_t HY = b->cfg.kv_heads * b->gchunks;
    for (uint32_t i = 0; i < n_seqs; ++i) {
        if (int rc = check_slot(b, slots[i])) return rc;
        for (uint32_t j = 0; j < i; ++j)
            if (slots[j] == slots[i])
                return b->fail(ITK_ERR_INVALID_ARGUMENT, "resident loop: slot " + zu(slots[i]) + " listed twice");
        const SlotState& st = b->slots[slots[i]];
        const uint64_t pos = st.appended[0];
        for (uint32_t l = 0; l < b->cfg.n_layers; ++l) {
            if (st.appended[l] != pos)
                return b->fail(ITK_ERR_INCOHERENT_CACHE, "resident loop: layer 0 has appended " + zu(pos) +
                                                             " positions but layer " + zu(l) + " has appended " +
                                                             zu(st.appended[l]));
            if (b->window[l] == 0 && pos + max_steps > b->ring[l])
                return b->fail(ITK_ERR_CAPACITY, "resident loop: position " + zu(pos + max_steps) +
                                                     " is past the slot's context capacity of " + zu(b->ring[l]));
            if (st.live && pos + max_steps > st.bases[l] + st.max_round)
                return b->fail(ITK_ERR_CHECKPOINT_RANGE_EXCEEDED,
                               "resident loop: layer " + zu(l) + " append at position " + zu(st.bases[l] + st.max_round) +
                                   " is outside the live checkpoint's saved range");
        }
        if (pos + max_steps > 0xfffffff0ull) return b->fail(ITK_ERR_CAPACITY, "resident loop: position exceeds 32 bits");
        states[i].slot = slots[i];
        states[i].pos = static_cast<uint32_t>(pos);
    }
    // One grid for every layer and every step of the loop: the largest one (at most two CTAs per SM) that keeps
    // each cell within the scratch's partial slots on every layer, at the first and at the last step.
    const uint64_t cells = static_cast<uint64_t>(n_seqs) * HY;
    uint64_t cap = kPartCellSplits / cells;
    if (cap > itk::kDecodeMaxParts) cap = itk::kDecodeMaxParts;
    if (cap < 2 || cells > b->ticket_cells) return b->fail(ITK_ERR_CAPACITY, "resident loop: too many (sequence, head) cells");
    // per layer: (largest cell, all cells) in tiles at the first and last step
    auto tiles_at = [&](uint32_t l, uint64_t extra, uint64_t* tmax, uint64_t* total) {
        *tmax = 0;
        *total = 0;
        for (uint32_t i = 0; i < n_seqs; ++i) {
            uint64_t n = static_cast<uint64_t>(states[i].pos) + 1 + extra;
            if (b->window[l] && n > b->window[l]) n = b->window[l];
            const uint64_t t = (n + 63) / 64;
            if (t > *tmax) *tmax = t;
            *total += t * HY;
        }
    };
    uint64_t ctas = b->forced_ctas > 0 ? static_cast<uint64_t>(b->forced_ctas) : 2ull * b->sm_count;
    auto fits = [&](uint64_t g) {
        for (uint32_t l = 0; l < b->cfg.n_layers; ++l) {
            uint64_t ts, tots, te, tote;
            tiles_at(l, 0, &ts, &tots);
            tiles_at(l, max_steps - 1, &te, &tote);
            const uint32_t ps = static_cast<uint32_t>((tots + g - 1) / g), pe = static_cast<uint32_t>((tote + g - 1) / g);
            if (itk::decode_parts_for(static_cast<uint32_t>(ts), ps) > cap ||
                itk::decode_parts_for(static_cast<uint32_t>(te), pe) > cap ||
                itk::decode_parts_for(static_cast<uint32_t>(te), ps) > cap)
                return false;
        }
        return true;
    };
    while (ctas > 1 && !fits(ctas)) --ctas;
    // With dependent launch the next layer's CTAs move in as this layer's move out, and the CTAs that merge a
    // cell (one per cell) move out last: the CTAs that inherit their places start late, finish late and become the
    // next mergers.  When the plan is cell-aligned, leave one place per cell unused if that lengthens the runs by
    // less than a twelfth, so that every CTA of the next layer finds a place before the merges begin.
    if (b->use_pdl && b->forced_ctas <= 0 && cells < ctas) {
        std::vector<uint32_t> keys(n_seqs), first(n_seqs + 1);
        auto plan = [&](uint64_t g, uint32_t* worst, uint32_t* used) {
            uint64_t total = 0;
            for (uint32_t i = 0; i < n_seqs; ++i) {
                uint64_t n = static_cast<uint64_t>(states[i].pos) + 1;
                if (b->window[0] && n > b->window[0]) n = b->window[0];
                keys[i] = static_cast<uint32_t>(n);
                total += (n + 63) / 64 * HY;
            }
            const uint32_t per = static_cast<uint32_t>((total + g - 1) / g);
            const bool ok = itk::decode_aligned_plan(keys.data(), n_seqs, HY, static_cast<uint32_t>(g),
                                                     static_cast<uint32_t>(total), per, static_cast<uint32_t>(cap),
                                                     first.data(), worst);
            *used = first[n_seqs];
            return ok;
        };
        uint32_t w0 = 0, u0 = 0, w1 = 0, u1 = 0;
        if (plan(ctas, &w0, &u0) && ctas - u0 < cells && plan(ctas - cells, &w1, &u1) && fits(ctas - cells) &&
            12ull * w1 <= 13ull * w0)
            ctas -= cells;
    }
    // Two lanes for the gathering launches: cut the batch where the tiles of layer 0 balance best, give each half one
    // CTA per SM, and take the schedule only if every cell of either lane stays within the scratch's partial slots on
    // every layer at the first and the last step - and, unless asked for regardless, only when a launch is short
    // enough (at most kLaneTilesPerCta tiles per CTA) for the hand-over between layers to matter.
    uint32_t lanes = 1, lane_split = 0;
    const uint32_t lane_ctas = 2u * static_cast<uint32_t>(b->sm_count);
    if (b->lanes_mode != 0 && n_seqs >= 2 && b->forced_ctas <= 0) {
        constexpr uint64_t kLaneTilesPerCta = 96;
        auto lane_tiles = [&](uint32_t l, uint32_t s0, uint32_t s1, uint64_t extra, uint64_t* tmax, uint64_t* total) {
            *tmax = 0;
            *total = 0;
            for (uint32_t i = s0; i < s1; ++i) {
                uint64_t n = static_cast<uint64_t>(states[i].pos) + 1 + extra;
                if (b->window[l] && n > b->window[l]) n = b->window[l];
                const uint64_t t = (n + 63) / 64;
                if (t > *tmax) *tmax = t;
                *total += t * HY;
            }
        };
        uint64_t tm, whole, best_gap = ~0ull;
        lane_tiles(0, 0, n_seqs, 0, &tm, &whole);
        for (uint32_t s = 1; s < n_seqs; ++s) {
            uint64_t left;
            lane_tiles(0, 0, s, 0, &tm, &left);
            const uint64_t gap = 2 * left > whole ? 2 * left - whole : whole - 2 * left;
            if (gap < best_gap) {
                best_gap = gap;
                lane_split = s;
            }
        }
        bool ok = b->lanes_mode == 2 || whole <= kLaneTilesPerCta * lane_ctas;
        const uint64_t g = lane_ctas / 2;
        for (uint32_t l = 0; l < b->cfg.n_layers && ok; ++l)
            for (int half = 0; half < 2 && ok; ++half) {
                const uint32_t s0 = half ? lane_split : 0, s1 = half ? n_seqs : lane_split;
                uint64_t ts, tots, te, tote;
                lane_tiles(l, s0, s1, 0, &ts, &tots);
                lane_tiles(l, s0, s1, max_steps - 1, &te, &tote);
                const uint32_t ps = static_cast<uint32_t>((tots + g - 1) / g), pe = static_cast<uint32_t>((tote + g - 1) / g);
                ok = itk::decode_parts_for(static_cast<uint32_t>(ts), ps) <= cap &&
                     itk::decode_parts_for(static_cast<uint32_t>(te), pe) <= cap &&
                     itk::decode_parts_for(static_cast<uint32_t>(te), ps) <= cap;
            }
        if (ok) {
            lanes = 2;
            lane_tiles(0, 0, lane_split, 0, &tm, &b->res_lane0_tiles);
        }
    }
    // The plan of the current positions lives on the device (worked out by the kernel that moves the positions) when
    // every layer sees the same keys, i.e. all layers are global; otherwise every CTA derives its own.
    bool all_global = true;
    for (uint32_t l = 0; l < b->cfg.n_layers; ++l) all_global = all_global && b->window[l] == 0;
    b->res_planned = all_global;
    b->res_spec.cells_per_seq = HY;
    b->res_spec.ctas = static_cast<uint32_t>(ctas);
    b->res_spec.lane_ctas = lanes == 2 ? lane_ctas : 0u;
    b->res_spec.lane_split = lane_split;
    b->res_spec.splits = static_cast<uint32_t>(cap);
    ITK_CUDA(b, cudaMemcpyAsync(b->d_states, states.data(), n_seqs * sizeof(itk::SeqState), cudaMemcpyHostToDevice,
                                b->stream), "sequence-state upload");
    ITK_CUDA(b, cudaMemcpyAsync(b->d_plan + itk::kDecodePlanBlocks * itk::kDecodePlanWords, &states[0].pos, sizeof(uint32_t),
                                cudaMemcpyHostToDevice, b->stream), "loop base position upload");
    if (lanes == 2) {  // the counters a single-GPU loop's lanes order themselves by start from zero with the loop
        ITK_CUDA(b, cudaMemsetAsync(b->lane_hdr, 0, kGatherErr + 64, b->stream), "lane counter clear");
        ITK_CUDA(b, cudaMemcpyAsync(b->lane_hdr + kGatherBase, &states[0].pos, sizeof(uint32_t), cudaMemcpyHostToDevice,
                                    b->stream), "loop base position upload");
    }
    ITK_CUDA(b, itk::launch_advance_states(b->d_states, n_seqs, 0, b->res_spec, all_global ? b->d_plan : nullptr, b->stream,
                                           &b->stats.kernel_launches), "plan launch");
    ITK_CUDA(b, cudaStreamSynchronize(b->stream), "sequence-state upload");
#ifdef ITK_DECODE_TRACE
    if (!g_trace) {  // timeline build: allocate before any capture begins; the caller reads it back through
        void* ptr;   // itk_debug_trace_buffer
        uint64_t bytes;
        itk_debug_trace_buffer(&ptr, &bytes);
    }
#endif
    b->res_active = true;
    b->res_slots.assign(slots, slots + n_seqs);
    b->res_max_steps = max_steps;
    b->res_ctas = static_cast<uint32_t>(ctas);
    b->res_parts = static_cast<uint32_t>(cap);
    b->res_lanes = lanes;
    b->res_lane_split = lane_split;
    b->res_lane_ctas = lane_ctas;
    b->res_prev_layer = -1;
    b->res_launches_in_step = 0;
    if (b->gth_local) {
        ITK_CUDA(b, cudaMemcpyAsync(b->gth_local + kGatherBase, &states[0].pos, sizeof(uint32_t), cudaMemcpyHostToDevice, b->stream),
                 "gather base position upload");
        ITK_CUDA(b, cudaStreamSynchronize(b->stream), "gather base position upload");
    }
    return ITK_OK;
}

#ifdef ITK_DECODE_TRACE
extern "C" int itk_debug_trace_buffer(void** dev_ptr, uint64_t* bytes) {
    const size_t n = 64ull * 512 * 16 * sizeof(unsigned long long);
    if (!g_trace) {
        if (cudaMalloc(&g_trace, n) != cudaSuccess) return ITK_ERR_CUDA;
        cudaMemset(g_trace, 0, n);
    }
    *dev_ptr = g_trace;
    *bytes = n;
    return ITK_OK;
}
#endif

static int resident_layer_impl(itk_backend* b, uint32_t layer, const float* d_q, const float* d_k, const float* d_v,
                               float* d_out, bool gather, uint64_t gather_offset_bytes) {
    if (!b->res_active) return b->fail(ITK_ERR_INVALID_ARGUMENT, "resident loop: not active");
    if (int rc = check_device_alignment(b, "resident loop", d_q, d_k, d_v, d_out)) return rc;  // (a null d_out is aligned)
    if (int rc = check_layer(b, layer)) return rc;
    b->tc_chain_live = false;
    AttnLaunch p{};
    bool two_lanes = false;
    fill_layer_view(b, layer, &p.layer);
    p.q = d_q;
    p.out = d_out;
    p.part_o = b->part_o;
    p.part_ml = b->part_ml;
    p.tickets = b->tickets;
    p.q_heads = b->cfg.q_heads;
    p.group = b->group;
    p.gchunks = b->gchunks;
    p.rows = 1;
    p.n_seqs = static_cast<uint32_t>(b->res_slots.size());
    p.scale = 1.0f / sqrtf(static_cast<float>(b->cfg.head_dim));
    p.k_new = d_k;
    p.v_new = d_v;
    p.seq_dev = b->d_states;
    p.plan_dev = b->res_planned ? b->d_plan : nullptr;
    if (b->fused_sum) {
        p.acc_o = b->acc_o;
        p.acc_l = b->acc_l;
        p.acc_flag = b->acc_flag;
    }
#ifdef ITK_DECODE_TRACE
    p.trace = g_trace ? g_trace + static_cast<size_t>(layer % 64) * 512 * 16 : nullptr;
#endif
    if (gather) {
        if (!b->gth_local) return b->fail(ITK_ERR_INVALID_ARGUMENT, "fused gather: no gather buffer (itk_gather_create)");
        const uint64_t slot_bytes = static_cast<uint64_t>(p.n_seqs) * b->q_width() * sizeof(float);
        if (gather_offset_bytes % 16 != 0 || gather_offset_bytes + slot_bytes > b->gth_bytes)
            return b->fail(ITK_ERR_INVALID_ARGUMENT, "fused gather: offset " + zu(gather_offset_bytes) +
                                                         " is misaligned or past the buffer of " + zu(b->gth_bytes) + " bytes");
        p.gather.n_peers = b->gth_world;
        p.gather.my_rank = b->gth_rank;
        for (uint32_t j = 0; j < b->gth_world; ++j) {
            if (!b->gth_peer[j]) return b->fail(ITK_ERR_INVALID_ARGUMENT, "fused gather: rank " + zu(j) + " is not open");
            p.gather.peer_out[j] = reinterpret_cast<float*>(b->gth_peer[j] + kGatherHeader + gather_offset_bytes);
            p.gather.peer_flags[j] = reinterpret_cast<unsigned int*>(b->gth_peer[j]);
        }
        p.gather.my_flags = reinterpret_cast<const unsigned int*>(b->gth_local);
        p.gather.err = reinterpret_cast<unsigned int*>(b->gth_local + kGatherErr);
        p.gather.base_pos = reinterpret_cast<const uint32_t*>(b->gth_local + kGatherBase);
    } else if (b->res_lanes == 2 && b->use_pdl) {
        // A single-GPU loop on a short launch runs in lanes too: the outputs go to the caller's buffer through the
        // gather's store path with this GPU as the only rank, and the arrival counters are the backend's own.
        p.out = nullptr;
        p.gather.n_peers = 1;
        p.gather.my_rank = 0;
        p.gather.local_only = 1;
        p.gather.peer_out[0] = d_out;
        p.gather.peer_flags[0] = reinterpret_cast<unsigned int*>(b->lane_hdr);
        p.gather.my_flags = reinterpret_cast<const unsigned int*>(b->lane_hdr);
        p.gather.err = reinterpret_cast<unsigned int*>(b->lane_hdr + kGatherErr);
        p.gather.base_pos = reinterpret_cast<const uint32_t*>(b->lane_hdr + kGatherBase);
    }
    if (p.gather.n_peers != 0) {
        p.gather.launches_per_step = b->cfg.n_layers;
        p.gather.launches_before = b->res_launches_in_step;
        const uint32_t HY = b->cfg.kv_heads * b->gchunks;
        two_lanes = b->res_lanes == 2;
        p.gather.lanes = two_lanes ? 2u : 1u;
        p.gather.lane_split = two_lanes ? b->res_lane_split : 0u;
        p.gather.cells_per_seq = HY;
        p.gather.stagger_ns = 0;
        if (two_lanes && b->lane_stagger > 0 && b->use_pdl && b->res_launches_in_step == 0) {
            // what lane 0 needs to stream its keys once, at about 6.5 TB/s = 6500 bytes per nanosecond
            const double lane0_bytes = static_cast<double>(b->res_lane0_tiles) * 64.0 * b->cfg.head_dim * 2.0 * 2.0;
            p.gather.stagger_ns = static_cast<uint32_t>(lane0_bytes / 6500.0 * b->lane_stagger / 100.0);
            if (p.gather.stagger_ns > 200000u) p.gather.stagger_ns = 200000u;
        }
        p.gather.wait_prev = 1u;
        p.gather.poll_limit = b->gth_poll_limit;
    }
    // Early K/V loads are safe behind another layer's decode kernel; behind anything else (the position advance,
    // the same layer) the kernel waits first.  A two-lane launch behind another layer's does not wait for it at all
    // before working: its lanes' arrival counters order what the two launches share.
    const bool behind_other_layer = b->res_prev_layer >= 0 && static_cast<uint32_t>(b->res_prev_layer) != layer;
    p.pdl = !b->use_pdl ? 0u : (behind_other_layer ? (two_lanes ? 3u : 2u) : 1u);
    ITK_CUDA(b, itk::launch_decode_f16_resident(p, two_lanes ? b->res_lane_ctas : b->res_ctas, b->res_parts, b->stream,
                                                &b->stats.kernel_launches),
             "resident decode launch");
    b->res_prev_layer = static_cast<int>(layer);
    b->res_launches_in_step += 1;
    return ITK_OK;
}

int itk_resident_layer(itk_backend* b, uint32_t layer, const float* d_q, const float* d_k, const float* d_v,
                       float* d_out) {
    if (!b || !d_q || !d_k || !d_v || !d_out) return ITK_ERR_INVALID_ARGUMENT;
    return resident_layer_impl(b, layer, d_q, d_k, d_v, d_out, false, 0);
}

int itk_resident_layer_gather(itk_backend* b, uint32_t layer, const float* d_q, const float* d_k, const float* d_v,
                              uint64_t gather_offset_bytes) {
    if (!b || !d_q || !d_k || !d_v) return ITK_ERR_INVALID_ARGUMENT;
    return resident_layer_impl(b, layer, d_q, d_k, d_v, nullptr, true, gather_offset_bytes);
}

int itk_gather_create(itk_backend* b, uint32_t world, uint32_t rank, uint64_t data_bytes, void** local_data,
                      uint8_t* handle64) {
    if (!b || !local_data || !handle64) return ITK_ERR_INVALID_ARGUMENT;
    cudaSetDevice(b->cfg.device);
    if (b->gth_local) return b->fail(ITK_ERR_INVALID_ARGUMENT, "fused gather: buffer already created");
    if (world < 1 || world > itk::kMaxPeers || rank >= world || data_bytes == 0)
        return b->fail(ITK_ERR_INVALID_ARGUMENT, "fused gather: 1..8 ranks, rank < world, non-empty buffer");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    void* ptr = nullptr;
    ITK_CUDA(b, cudaMalloc(&ptr, kGatherHeader + data_bytes), "gather buffer allocation");
    ITK_CUDA(b, cudaMemset(ptr, 0, kGatherHeader + data_bytes), "gather buffer clear");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
    if (e != cudaSuccess) {
        cudaFree(ptr);
        return b->cuda_fail(e, "cudaIpcGetMemHandle");
    }
    std::memcpy(handle64, &h, 64);
    b->gth_local = static_cast<unsigned char*>(ptr);
    b->gth_world = world;
    b->gth_rank = rank;
    b->gth_bytes = data_bytes;
    b->gth_peer[rank] = b->gth_local;
    *local_data = b->gth_local + kGatherHeader;
    return ITK_OK;
}

int itk_gather_open(itk_backend* b, uint32_t peer_rank, const uint8_t* handle64) {
    if (!b || !handle64) return ITK_ERR_INVALID_ARGUMENT;
    cudaSetDevice(b->cfg.device);
    if (!b->gth_local || peer_rank >= b->gth_world)
        return b->fail(ITK_ERR_INVALID_ARGUMENT, "fused gather: create the local buffer first; rank must be < world");
    if (peer_rank == b->gth_rank || b->gth_peer[peer_rank]) return ITK_OK;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle64, 64);
    void* ptr = nullptr;
    ITK_CUDA(b, cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
    b->gth_peer[peer_rank] = static_cast<unsigned char*>(ptr);
    return ITK_OK;
}

int itk_gather_attach(itk_backend* b, uint32_t peer_rank, void* peer_local_data) {
    if (!b || !peer_local_data) return ITK_ERR_INVALID_ARGUMENT;
    if (!b->gth_local || peer_rank >= b->gth_world)
        return b->fail(ITK_ERR_INVALID_ARGUMENT, "fused gather: create the local buffer first; rank must be < world");
    if (peer_rank == b->gth_rank) return ITK_OK;
    if (b->gth_peer[peer_rank]) return b->fail(ITK_ERR_INVALID_ARGUMENT, "fused gather: rank " + zu(peer_rank) + " is already open");
    b->gth_peer[peer_rank] = static_cast<unsigned char*>(peer_local_data) - kGatherHeader;  // the header sits before the data
    b->gth_attached[peer_rank] = true;
    return ITK_OK;
}

int itk_gather_close_peers(itk_backend* b) {
    if (!b) return ITK_ERR_INVALID_ARGUMENT;
    cudaSetDevice(b->cfg.device);
    if (b->res_active) return b->fail(ITK_ERR_INVALID_ARGUMENT, "fused gather: end the resident loop first");
    if (b->stream) ITK_CUDA(b, cudaStreamSynchronize(b->stream), "gather close");
    for (uint32_t j = 0; j < itk::kMaxPeers; ++j) {
        if (j == b->gth_rank || !b->gth_peer[j]) continue;
        if (!b->gth_attached[j]) cudaIpcCloseMemHandle(b->gth_peer[j]);
        b->gth_peer[j] = nullptr;
        b->gth_attached[j] = false;
    }
    return ITK_OK;
}

int itk_gather_reset(itk_backend* b) {
    if (!b) return ITK_ERR_INVALID_ARGUMENT;
    cudaSetDevice(b->cfg.device);
    if (!b->gth_local) return b->fail(ITK_ERR_INVALID_ARGUMENT, "fused gather: no gather buffer");
    ITK_CUDA(b, cudaMemsetAsync(b->gth_local, 0, kGatherErr + 64, b->stream), "gather flag clear");
    ITK_CUDA(b, cudaStreamSynchronize(b->stream), "gather flag clear");
    return ITK_OK;
}

int itk_gather_status(itk_backend* b, uint32_t* error_bits) {
    if (!b || !error_bits) return ITK_ERR_INVALID_ARGUMENT;
    cudaSetDevice(b->cfg.device);
    if (!b->gth_local) return b->fail(ITK_ERR_INVALID_ARGUMENT, "fused gather: no gather buffer");
    ITK_CUDA(b, cudaStreamSynchronize(b->stream), "gather status");
    ITK_CUDA(b, cudaMemcpy(error_bits, b->gth_local + kGatherErr, sizeof(uint32_t), cudaMemcpyDeviceToHost), "gather status");
    return ITK_OK;
}

int itk_resident_advance(itk_backend* b) {
    if (!b) return ITK_ERR_INVALID_ARGUMENT;
    if (!b->res_active) return b->fail(ITK_ERR_INVALID_ARGUMENT, "resident loop: not active");
    ITK_CUDA(b, itk::launch_advance_states(b->d_states, static_cast<uint32_t>(b->res_slots.size()), 1, b->res_spec,
                                           b->res_planned ? b->d_plan : nullptr, b->stream, &b->stats.kernel_launches),
             "state advance launch");
    b->res_prev_layer = -1;
    b->res_launches_in_step = 0;
    return ITK_OK;
}

int itk_resident_end(itk_backend* b, uint64_t steps_done) {
    if (!b) return ITK_ERR_INVALID_ARGUMENT;
    if (!b->res_active) return b->fail(ITK_ERR_INVALID_ARGUMENT, "resident loop: not active");
    if (steps_done > b->res_max_steps)
        return b->fail(ITK_ERR_INVALID_ARGUMENT, "resident loop: " + zu(steps_done) + " steps reported, " +
                                                     zu(b->res_max_steps) + " were reserved");
    for (uint32_t slot : b->res_slots) {
        SlotState& st = b->slots[slot];
        for (uint32_t l = 0; l < b->cfg.n_layers; ++l) st.appended[l] += steps_done;
        if (steps_done) st.built = true;
    }
    b->stats.rows_appended += steps_done * b->res_slots.size() * b->cfg.n_layers;
    b->stats.attention_calls += steps_done * b->cfg.n_layers;
    b->res_active = false;
    return ITK_OK;
}

int itk_profile_enable(itk_backend* b, uint32_t capacity) {
    if (!b) return ITK_ERR_INVALID_ARGUMENT;
    cudaSetDevice(b->cfg.device);
    for (cudaEvent_t e : b->prof_events) cudaEventDestroy(e);
    b->prof_events.clear();
    b->prof_tags.assign(capacity, 0);
    b->prof_used = 0;
    for (uint32_t i = 0; i < 2 * capacity; ++i) {
        cudaEvent_t e;
        ITK_CUDA(b, cudaEventCreate(&e), "profile event creation");
        b->prof_events.push_back(e);
    }
    return ITK_OK;
}

int itk_profile_read(itk_backend* b, double* attention_ms, uint64_t* attention_launches, double* append_ms,
                     uint64_t* append_launches) {
    if (!b) return ITK_ERR_INVALID_ARGUMENT;
    cudaSetDevice(b->cfg.device);
    ITK_CUDA(b, cudaStreamSynchronize(b->stream), "profile read");
    double ms[3] = {0.0, 0.0, 0.0};
    uint64_t n[3] = {0, 0, 0};
    for (size_t at = 0; at + 1 < b->prof_used; at += 2) {
        float t = 0.f;
        ITK_CUDA(b, cudaEventElapsedTime(&t, b->prof_events[at], b->prof_events[at + 1]), "profile read");
        const int tag = b->prof_tags[at / 2];
        ms[tag] += t;
        n[tag] += 1;
    }
    if (attention_ms) *attention_ms = ms[0];
    if (attention_launches) *attention_launches = n[0];
    if (append_ms) *append_ms = ms[1];
    if (append_launches) *append_launches = n[1];
    b->prof_copy_ms = ms[2];
    b->prof_copy_launches = n[2];
    b->prof_used = 0;
    return ITK_OK;
}

int itk_profile_read_copy(itk_backend* b, double* copy_ms, uint64_t* copy_launches) {
    if (!b) return ITK_ERR_INVALID_ARGUMENT;
    if (copy_ms) *copy_ms = b->prof_copy_ms;
    if (copy_launches) *copy_launches = b->prof_copy_launches;
    return ITK_OK;
}

int itk_attention_batch_device(itk_backend* b, uint32_t layer, uint32_t n_seqs, const uint32_t* slots,
                               const uint64_t* positions, uint32_t rows, const float* d_q, const float* d_k,
                               const float* d_v, float* d_out) {
    if (!b || !slots || !positions || !d_q || !d_k || !d_v || !d_out) return ITK_ERR_INVALID_ARGUMENT;
    if (int rc = check_device_alignment(b, "attention", d_q, d_k, d_v, d_out)) return rc;
    cudaSetDevice(b->cfg.device);
    return step_device(b, layer, n_seqs, slots, positions, rows, d_q, d_k, d_v, d_out);
}

int itk_attention_batch(itk_backend* b, uint32_t layer, uint32_t n_seqs, const uint32_t* slots,
                        const uint64_t* positions, uint32_t rows, const float* q, const float* k, const float* v,
                        float* out) {
    if (!b || !slots || !positions || !q || !k || !v || !out) return ITK_ERR_INVALID_ARGUMENT;
    cudaSetDevice(b->cfg.device);
    std::vector<SeqDesc> seqs;
    if (int rc = validate_step(b, layer, n_seqs, slots, positions, rows, &seqs)) return rc;
    const size_t total_rows = static_cast<size_t>(n_seqs) * rows;
    if (total_rows > b->stage_rows)
        return b->fail(ITK_ERR_CAPACITY, "attention: " + zu(total_rows) + " rows exceed the staging capacity of " +
                                             zu(b->stage_rows));
    const size_t qb = total_rows * b->q_width() * sizeof(float), kb = total_rows * b->row_len() * sizeof(float);
    ITK_CUDA(b, cudaMemcpyAsync(b->d_k, k, kb, cudaMemcpyHostToDevice, b->stream), "k upload");
    ITK_CUDA(b, cudaMemcpyAsync(b->d_v, v, kb, cudaMemcpyHostToDevice, b->stream), "v upload");
    ITK_CUDA(b, cudaMemcpyAsync(b->d_q, q, qb, cudaMemcpyHostToDevice, b->stream), "q upload");
    if (int rc = step_device(b, layer, n_seqs, slots, positions, rows, b->d_q, b->d_k, b->d_v, b->d_out)) return rc;
    ITK_CUDA(b, cudaMemcpyAsync(out, b->d_out, qb, cudaMemcpyDeviceToHost, b->stream), "output download");
    queue_status_read(b);
    ITK_CUDA(b, cudaStreamSynchronize(b->stream), "attention");
    return check_status(b);
}

int itk_attention_layers_host(itk_backend* b, uint32_t n_seqs, const uint32_t* slots, const uint64_t* positions,
                              uint32_t rows, const float* q, const float* k, const float* v, float* out) {
    if (!b || !slots || !positions || !q || !k || !v || !out) return ITK_ERR_INVALID_ARGUMENT;
    cudaSetDevice(b->cfg.device);
    const uint32_t L = b->cfg.n_layers;
    // Every layer is validated before anything is queued: a refusal leaves all layers where they were.
    std::vector<SeqDesc> seqs;
    for (uint32_t l = 0; l < L; ++l)
        if (int rc = validate_step(b, l, n_seqs, slots, positions, rows, &seqs)) return rc;
    const size_t total_rows = static_cast<size_t>(n_seqs) * rows;
    if (total_rows > b->stage_rows)
        return b->fail(ITK_ERR_CAPACITY, "attention: " + zu(total_rows) + " rows exceed the staging capacity of " +
                                             zu(b->stage_rows));
    if (b->fw_rows < total_rows) {  // first use (or a larger batch): per-layer staging, copy streams, events
        ITK_CUDA(b, cudaStreamSynchronize(b->stream), "forward staging");
        cudaFree(b->fw_q);
        cudaFree(b->fw_k);
        cudaFree(b->fw_v);
        cudaFree(b->fw_out);
        b->fw_q = b->fw_k = b->fw_v = b->fw_out = nullptr;
        b->fw_rows = 0;
        const size_t rows_cap = b->stage_rows;
        ITK_CUDA(b, cudaMalloc(&b->fw_q, L * rows_cap * b->q_width() * sizeof(float)), "forward staging allocation");
        ITK_CUDA(b, cudaMalloc(&b->fw_out, L * rows_cap * b->q_width() * sizeof(float)), "forward staging allocation");
        ITK_CUDA(b, cudaMalloc(&b->fw_k, L * rows_cap * b->row_len() * sizeof(float)), "forward staging allocation");
        ITK_CUDA(b, cudaMalloc(&b->fw_v, L * rows_cap * b->row_len() * sizeof(float)), "forward staging allocation");
        b->fw_rows = rows_cap;
        if (!b->fw_in) ITK_CUDA(b, cudaStreamCreateWithFlags(&b->fw_in, cudaStreamNonBlocking), "copy stream");
        if (!b->fw_outs) ITK_CUDA(b, cudaStreamCreateWithFlags(&b->fw_outs, cudaStreamNonBlocking), "copy stream");
        if (!b->fw_ev_prev) ITK_CUDA(b, cudaEventCreateWithFlags(&b->fw_ev_prev, cudaEventDisableTiming), "event");
        while (b->fw_ev_in.size() < L) {
            cudaEvent_t a, c;
            ITK_CUDA(b, cudaEventCreateWithFlags(&a, cudaEventDisableTiming), "event");
            b->fw_ev_in.push_back(a);
            ITK_CUDA(b, cudaEventCreateWithFlags(&c, cudaEventDisableTiming), "event");
            b->fw_ev_k.push_back(c);
        }
    }
    const size_t qn = total_rows * b->q_width(), kn = total_rows * b->row_len();
    const size_t qs = b->fw_rows * b->q_width(), ks = b->fw_rows * b->row_len();  // per-layer staging strides
    const size_t f = sizeof(float);
    if (rows == 1 && b->f16 && itk::decode_f16_supported(b->cfg.head_dim, 1) && !b->res_active &&
        static_cast<uint64_t>(L) * (qn + 2 * kn) * f <= b->fw_loop_bytes) {
        // A decode step from host buffers: every layer's rows go up in three strided copies and the step runs as one
        // step of the replayable loop - positions on the device, each layer's launch a programmatic dependent of the
        // one before, two lanes on short launches - instead of as ordinary per-layer launches behind per-layer copies
        // (whose fixed cost exceeds a short layer's kernel time, above all with one process per GPU on a shared host).
        // A step that moves more than fw_loop_bytes gains more from copies that overlap the kernels.
        ITK_CUDA(b, cudaMemcpy2DAsync(b->fw_q, qs * f, q, qn * f, qn * f, L, cudaMemcpyHostToDevice, b->stream), "q upload");
        ITK_CUDA(b, cudaMemcpy2DAsync(b->fw_k, ks * f, k, kn * f, kn * f, L, cudaMemcpyHostToDevice, b->stream), "k upload");
        ITK_CUDA(b, cudaMemcpy2DAsync(b->fw_v, ks * f, v, kn * f, kn * f, L, cudaMemcpyHostToDevice, b->stream), "v upload");
        int rc = itk_resident_begin(b, n_seqs, slots, 1);
        if (rc == ITK_OK) {
            for (uint32_t l = 0; l < L && rc == ITK_OK; ++l)
                rc = resident_layer_impl(b, l, b->fw_q + l * qs, b->fw_k + l * ks, b->fw_v + l * ks, b->fw_out + l * qs, false, 0);
            const int rc_end = itk_resident_end(b, rc == ITK_OK ? 1 : 0);
            if (rc != ITK_OK) return rc;
            if (rc_end != ITK_OK) return rc_end;
        } else {
            // the loop's own limits (its scratch, a live checkpoint's range): the step runs as ordinary launches
            for (uint32_t l = 0; l < L; ++l)
                if (int rc2 = step_device(b, l, n_seqs, slots, positions, rows, b->fw_q + l * qs, b->fw_k + l * ks,
                                          b->fw_v + l * ks, b->fw_out + l * qs))
                    return rc2;
        }
        ITK_CUDA(b, cudaMemcpy2DAsync(out, qn * f, b->fw_out, qs * f, qn * f, L, cudaMemcpyDeviceToHost, b->stream),
                 "output download");
        queue_status_read(b);
        ITK_CUDA(b, cudaStreamSynchronize(b->stream), "forward");
        return check_status(b);
    }
    if (static_cast<uint64_t>(L) * (qn + 2 * kn) * sizeof(float) <= b->fw_bulk_bytes) {
        // A small forward (a decode step of a few sequences): the per-layer copies' fixed cost would outweigh what
        // their overlap with the kernels hides.  Every layer's rows go up in three strided copies, the layers'
        // launches follow back to back, one strided copy brings all results down.
        ITK_CUDA(b, cudaMemcpy2DAsync(b->fw_q, qs * f, q, qn * f, qn * f, L, cudaMemcpyHostToDevice, b->stream), "q upload");
        ITK_CUDA(b, cudaMemcpy2DAsync(b->fw_k, ks * f, k, kn * f, kn * f, L, cudaMemcpyHostToDevice, b->stream), "k upload");
        ITK_CUDA(b, cudaMemcpy2DAsync(b->fw_v, ks * f, v, kn * f, kn * f, L, cudaMemcpyHostToDevice, b->stream), "v upload");
        for (uint32_t l = 0; l < L; ++l)
            if (int rc = step_device(b, l, n_seqs, slots, positions, rows, b->fw_q + l * qs, b->fw_k + l * ks,
                                     b->fw_v + l * ks, b->fw_out + l * qs))
                return rc;
        ITK_CUDA(b, cudaMemcpy2DAsync(out, qn * f, b->fw_out, qs * f, qn * f, L, cudaMemcpyDeviceToHost, b->stream),
                 "output download");
        queue_status_read(b);
        ITK_CUDA(b, cudaStreamSynchronize(b->stream), "forward");
        return check_status(b);
    }
    // The uploads start once everything already queued on the backend's stream (an earlier forward's kernels,
    // which read the same staging) has run.
    ITK_CUDA(b, cudaEventRecord(b->fw_ev_prev, b->stream), "forward");
    ITK_CUDA(b, cudaStreamWaitEvent(b->fw_in, b->fw_ev_prev, 0), "forward");
    // Three streams: layer l's rows go up on the first while layer l - 1 computes on the backend's stream and
    // layer l - 2's result comes down on the third.
    for (uint32_t l = 0; l < L; ++l) {
        ITK_CUDA(b, cudaMemcpyAsync(b->fw_q + l * qs, q + l * qn, qn * sizeof(float), cudaMemcpyHostToDevice, b->fw_in), "q upload");
        ITK_CUDA(b, cudaMemcpyAsync(b->fw_k + l * ks, k + l * kn, kn * sizeof(float), cudaMemcpyHostToDevice, b->fw_in), "k upload");
        ITK_CUDA(b, cudaMemcpyAsync(b->fw_v + l * ks, v + l * kn, kn * sizeof(float), cudaMemcpyHostToDevice, b->fw_in), "v upload");
        ITK_CUDA(b, cudaEventRecord(b->fw_ev_in[l], b->fw_in), "forward");
    }
    for (uint32_t l = 0; l < L; ++l) {
        ITK_CUDA(b, cudaStreamWaitEvent(b->stream, b->fw_ev_in[l], 0), "forward");
        if (int rc = step_device(b, l, n_seqs, slots, positions, rows, b->fw_q + l * qs, b->fw_k + l * ks, b->fw_v + l * ks,
                                 b->fw_out + l * qs))
            return rc;
        ITK_CUDA(b, cudaEventRecord(b->fw_ev_k[l], b->stream), "forward");
        ITK_CUDA(b, cudaStreamWaitEvent(b->fw_outs, b->fw_ev_k[l], 0), "forward");
        ITK_CUDA(b, cudaMemcpyAsync(out + l * qn, b->fw_out + l * qs, qn * sizeof(float), cudaMemcpyDeviceToHost, b->fw_outs),
                 "output download");
    }
    queue_status_read(b);
    ITK_CUDA(b, cudaStreamSynchronize(b->fw_outs), "forward");
    ITK_CUDA(b, cudaStreamSynchronize(b->stream), "forward");
    return check_status(b);
}

int itk_layer_prep_set(itk_backend* b, uint32_t layer, const itk_prep_config* cfg) {
    if (!b || !cfg) return ITK_ERR_INVALID_ARGUMENT;
    cudaSetDevice(b->cfg.device);
    if (int rc = check_layer(b, layer)) return rc;
    const uint32_t D = b->cfg.head_dim;
    if (D > 256) return b->fail(ITK_ERR_CAPACITY, "attention preparation: head_dim " + zu(D) + " exceeds 256");
    // crates/torch-math/src/norm.rs:34-40, rope_interleaved.rs:72-95: the same refusals, by name
    if ((cfg->q_norm_weight || cfg->k_norm_weight) && !(std::isfinite(cfg->norm_eps) && cfg->norm_eps > 0.f))
        return b->fail(ITK_ERR_STEP_FAILED, "rms_norm: eps must be finite and > 0");
    if (cfg->rotary_dim != 0) {
        if (D < 2 || D % 2 != 0) return b->fail(ITK_ERR_STEP_FAILED, "rope: head_dim must be even and >= 2");
        if (cfg->rotary_dim < 2 || cfg->rotary_dim % 2 != 0 || cfg->rotary_dim > D)
            return b->fail(ITK_ERR_STEP_FAILED, "rope: rotary_dim must be even, >= 2, and <= head_dim");
        if (!std::isfinite(cfg->rope_base) || cfg->rope_base <= 1.0f)
            return b->fail(ITK_ERR_STEP_FAILED, "rope: base must be finite and > 1");
        if (cfg->pairing > 1) return b->fail(ITK_ERR_INVALID_ARGUMENT, "rope: pairing is 0 (adjacent) or 1 (half split)");
    }
    if (b->prep.empty()) b->prep.resize(b->cfg.n_layers);
    if (!b->d_qp) {
        ITK_CUDA(b, cudaMalloc(&b->d_qp, b->stage_rows * b->q_width() * sizeof(float)), "prepared-row staging");
        ITK_CUDA(b, cudaMalloc(&b->d_kp, b->stage_rows * b->row_len() * sizeof(float)), "prepared-row staging");
    }
    itk_backend::LayerPrep next;
    auto upload = [&](const float* host, float** dev) -> int {
        if (!host) return ITK_OK;
        ITK_CUDA(b, cudaMalloc(dev, D * sizeof(float)), "norm weight allocation");
        ITK_CUDA(b, cudaMemcpy(*dev, host, D * sizeof(float), cudaMemcpyHostToDevice), "norm weight upload");
        return ITK_OK;
    };
    int rc = upload(cfg->q_norm_weight, &next.q_w);
    if (rc == ITK_OK) rc = upload(cfg->k_norm_weight, &next.k_w);
    if (rc == ITK_OK && cfg->rotary_dim != 0) {
        // base^(-2i / rotary_dim) in f64, the CPU reference's own expression
        std::vector<double> inv(cfg->rotary_dim / 2);
        for (uint32_t i = 0; i < cfg->rotary_dim / 2; ++i)
            inv[i] = std::pow(static_cast<double>(cfg->rope_base),
                              -static_cast<double>(2 * i) / static_cast<double>(cfg->rotary_dim));
        cudaError_t e = cudaMalloc(&next.inv_freq, inv.size() * sizeof(double));
        if (e == cudaSuccess)
            e = cudaMemcpy(next.inv_freq, inv.data(), inv.size() * sizeof(double), cudaMemcpyHostToDevice);
        if (e != cudaSuccess) rc = b->cuda_fail(e, "inverse-frequency table upload");
    }
    if (rc != ITK_OK) {
        cudaFree(next.q_w);
        cudaFree(next.k_w);
        cudaFree(next.inv_freq);
        return rc;
    }
    next.set = true;
    next.eps = cfg->norm_eps;
    next.rotary_dim = cfg->rotary_dim;
    next.pairing = cfg->pairing;
    itk_backend::LayerPrep& cur = b->prep[layer];
    ITK_CUDA(b, cudaStreamSynchronize(b->stream), "attention preparation");  // nothing in flight reads the old tables
    cudaFree(cur.q_w);
    cudaFree(cur.k_w);
    cudaFree(cur.inv_freq);
    cur = next;
    return ITK_OK;
}

// Prepares the call's Q and K rows (device f32) into the backend's staging, then runs the ordinary step on them.
static int step_prepared(itk_backend* b, uint32_t layer, uint32_t n_seqs, const uint32_t* slots,
                         const uint64_t* positions, uint32_t rows, const float* d_q, const float* d_k,
                         const float* d_v, float* d_out) {
    if (int rc = check_layer(b, layer)) return rc;
    if (b->prep.empty() || !b->prep[layer].set)
        return b->fail(ITK_ERR_INVALID_ARGUMENT, "attention preparation: layer " + zu(layer) +
                                                     " has no configuration (itk_layer_prep_set)");
    std::vector<SeqDesc> seqs;
    if (int rc = validate_step(b, layer, n_seqs, slots, positions, rows, &seqs)) return rc;
    const size_t total_rows = static_cast<size_t>(n_seqs) * rows;
    if (total_rows > b->stage_rows)
        return b->fail(ITK_ERR_CAPACITY, "attention: " + zu(total_rows) + " rows exceed the staging capacity of " +
                                             zu(b->stage_rows));
    const itk_backend::LayerPrep& lp = b->prep[layer];
    itk::PrepLaunch p{};
    p.q_in = d_q;
    p.k_in = d_k;
    p.q_out = b->d_qp;
    p.k_out = b->d_kp;
    p.q_w = lp.q_w;
    p.k_w = lp.k_w;
    p.inv_freq = lp.inv_freq;
    p.eps = lp.eps;
    p.rotary_dim = lp.rotary_dim;
    p.pairing = lp.pairing;
    p.q_heads = b->cfg.q_heads;
    p.kv_heads = b->cfg.kv_heads;
    p.head_dim = b->cfg.head_dim;
    p.rows = rows;
    p.n_seqs = n_seqs;
    for (uint32_t i = 0; i < n_seqs; ++i) p.pos0[i] = static_cast<uint32_t>(positions[i]);
    ITK_CUDA(b, itk::launch_prep(p, b->stream, &b->stats.kernel_launches), "attention preparation launch");
    return step_device(b, layer, n_seqs, slots, positions, rows, b->d_qp, b->d_kp, d_v, d_out);
}

int itk_attention_batch_prep_device(itk_backend* b, uint32_t layer, uint32_t n_seqs, const uint32_t* slots,
                                    const uint64_t* positions, uint32_t rows, const float* d_q, const float* d_k,
                                    const float* d_v, float* d_out) {
    if (!b || !slots || !positions || !d_q || !d_k || !d_v || !d_out) return ITK_ERR_INVALID_ARGUMENT;
    if (int rc = check_device_alignment(b, "attention", d_q, d_k, d_v, d_out)) return rc;
    cudaSetDevice(b->cfg.device);
    return step_prepared(b, layer, n_seqs, slots, positions, rows, d_q, d_k, d_v, d_out);
}

int itk_attention_batch_prep(itk_backend* b, uint32_t layer, uint32_t n_seqs, const uint32_t* slots,
                             const uint64_t* positions, uint32_t rows, const float* q, const float* k, const float* v,
                             float* out) {
    if (!b || !slots || !positions || !q || !k || !v || !out) return ITK_ERR_INVALID_ARGUMENT;
    cudaSetDevice(b->cfg.device);
    std::vector<SeqDesc> seqs;
    if (int rc = validate_step(b, layer, n_seqs, slots, positions, rows, &seqs)) return rc;
    const size_t total_rows = static_cast<size_t>(n_seqs) * rows;
    if (total_rows > b->stage_rows)
        return b->fail(ITK_ERR_CAPACITY, "attention: " + zu(total_rows) + " rows exceed the staging capacity of " +
                                             zu(b->stage_rows));
    const size_t qb = total_rows * b->q_width() * sizeof(float), kb = total_rows * b->row_len() * sizeof(float);
    ITK_CUDA(b, cudaMemcpyAsync(b->d_k, k, kb, cudaMemcpyHostToDevice, b->stream), "k upload");
    ITK_CUDA(b, cudaMemcpyAsync(b->d_v, v, kb, cudaMemcpyHostToDevice, b->stream), "v upload");
    ITK_CUDA(b, cudaMemcpyAsync(b->d_q, q, qb, cudaMemcpyHostToDevice, b->stream), "q upload");
    if (int rc = step_prepared(b, layer, n_seqs, slots, positions, rows, b->d_q, b->d_k, b->d_v, b->d_out)) return rc;
    ITK_CUDA(b, cudaMemcpyAsync(out, b->d_out, qb, cudaMemcpyDeviceToHost, b->stream), "output download");
    queue_status_read(b);
    ITK_CUDA(b, cudaStreamSynchronize(b->stream), "attention");
    return check_status(b);
}

int itk_attention(itk_backend* b, uint32_t slot, uint32_t layer, const float* q, size_t q_len, const float* k,
                  size_t k_len, const float* v, size_t v_len, uint64_t position, float* out) {
    if (!b) return ITK_ERR_INVALID_ARGUMENT;
    // crates/cpu-compute/src/cpu.rs:532-556: whole q rows, then k/v lengths for that row count.
    const size_t qw = b->q_width(), kw = b->row_len();
    if (q_len % qw != 0)
        return b->fail(ITK_ERR_STEP_FAILED, "attention: query projection holds " + zu(q_len) +
                                                " elements, not a whole number of " + zu(qw) + "-wide rows");
    const size_t rows = q_len / qw;
    if (k_len != rows * kw || v_len != rows * kw)
        return b->fail(ITK_ERR_STEP_FAILED, "attention: key/value projections hold " + zu(k_len) + "/" + zu(v_len) +
                                                " elements for " + zu(rows) + " rows, expected " + zu(rows * kw) + "/" +
                                                zu(rows * kw));
    if (rows == 0) return ITK_OK;
    return itk_attention_batch(b, layer, 1, &slot, &position, static_cast<uint32_t>(rows), q, k, v, out);
}

int itk_gqa_attention(itk_backend* b, uint32_t slot, uint32_t layer, const float* q, size_t q_len, uint32_t rows,
                      const uint64_t* query_positions, float* out) {
    if (!b) return ITK_ERR_INVALID_ARGUMENT;
    cudaSetDevice(b->cfg.device);
    if (int rc = check_slot(b, slot)) return rc;
    if (int rc = check_layer(b, layer)) return rc;
    const size_t expected = static_cast<size_t>(rows) * b->q_width();
    if (q_len != expected) return b->fail(ITK_ERR_SHAPE_MISMATCH, "q: got " + zu(q_len) + ", expected " + zu(expected));
    if (rows == 0) return ITK_OK;
    if (!q || !query_positions || !out) return ITK_ERR_INVALID_ARGUMENT;
    const SlotState& st = b->slots[slot];
    const uint64_t appended = st.appended[layer];
    const uint64_t first_visible = appended - b->stored(layer, appended);
    // Each query row becomes its own one-row unit so that positions need not be consecutive.
    std::vector<SeqDesc> seqs(rows);
    for (uint32_t r = 0; r < rows; ++r) {
        const uint64_t p = query_positions[r];
        uint64_t lo = first_visible;
        if (b->window[layer] && p + 1 > b->window[layer] && p + 1 - b->window[layer] > lo) lo = p + 1 - b->window[layer];
        const uint64_t hi = (p + 1 < appended) ? p + 1 : appended;
        if (hi <= lo) return b->fail(ITK_ERR_NO_VISIBLE_KEYS, "query at position " + zu(p) + " has no visible keys");
        seqs[r].slot = slot;
        seqs[r].q_pos0 = static_cast<uint32_t>(hi - 1);  // the row sees [lo, hi); its own position caps hi
        seqs[r].kv_lo = static_cast<uint32_t>(lo);
        seqs[r].kv_hi = static_cast<uint32_t>(hi);
    }
    for (uint32_t at = 0; at < rows; at += static_cast<uint32_t>(b->stage_rows)) {
        const uint32_t m = (rows - at < b->stage_rows) ? rows - at : static_cast<uint32_t>(b->stage_rows);
        const size_t bytes = static_cast<size_t>(m) * b->q_width() * sizeof(float);
        ITK_CUDA(b, cudaMemcpyAsync(b->d_q, q + static_cast<size_t>(at) * b->q_width(), bytes, cudaMemcpyHostToDevice,
                                    b->stream), "q upload");
        if (int rc = run_attention(b, layer, m, seqs.data() + at, 1, b->d_q, b->d_out)) return rc;
        ITK_CUDA(b, cudaMemcpyAsync(out + static_cast<size_t>(at) * b->q_width(), b->d_out, bytes,
                                    cudaMemcpyDeviceToHost, b->stream), "output download");
        ITK_CUDA(b, cudaStreamSynchronize(b->stream), "attention");
    }
    b->stats.attention_calls += 1;
    return ITK_OK;
}

int itk_append_rows(itk_backend* b, uint32_t slot, uint32_t layer, const float* k, const float* v, uint32_t rows,
                    uint64_t start) {
    if (!b) return ITK_ERR_INVALID_ARGUMENT;
    cudaSetDevice(b->cfg.device);
    if (int rc = check_slot(b, slot)) return rc;
    SlotState& st = b->slots[slot];
    // crates/attention/src/cache.rs:445-471: checkpoint range, then layer, then order.
    if (st.live && layer < st.bases.size()) {
        const uint64_t limit = st.bases[layer] + st.max_round;
        if (start + rows > limit && rows > 0) {
            const uint64_t bad = start > limit ? start : limit;
            return b->fail(ITK_ERR_CHECKPOINT_RANGE_EXCEEDED,
                           "layer " + zu(layer) + " append at position " + zu(bad) +
                               " is outside the live checkpoint's saved range (first unsaved position " + zu(limit) +
                               "); refusing so a later rewind cannot meet a slot it cannot restore");
        }
    }
    if (int rc = check_layer(b, layer)) return rc;
    if (start != st.appended[layer])
        return b->fail(ITK_ERR_OUT_OF_ORDER_POSITION, "layer " + zu(layer) + " appends must be in order: expected position " +
                                                          zu(st.appended[layer]) + ", got " + zu(start));
    if (rows == 0) return ITK_OK;
    if (!k || !v) return ITK_ERR_INVALID_ARGUMENT;
    if (b->window[layer] == 0 && start + rows > b->ring[layer])
        return b->fail(ITK_ERR_CAPACITY, "append: position " + zu(start + rows) + " is past the slot's context capacity of " +
                                             zu(b->ring[layer]) + " positions");
    // On a ring layer only the newest `ring` rows of a long append can survive; the older ones would be
    // overwritten inside the same call, so they are skipped (the reference evicts them just the same).
    uint32_t first_row = 0;
    if (b->window[layer] != 0 && rows > b->ring[layer]) first_row = rows - b->ring[layer];
    for (uint32_t at = first_row; at < rows; at += static_cast<uint32_t>(b->stage_rows)) {
        const uint32_t m = (rows - at < b->stage_rows) ? rows - at : static_cast<uint32_t>(b->stage_rows);
        const size_t bytes = static_cast<size_t>(m) * b->row_len() * sizeof(float);
        ITK_CUDA(b, cudaMemcpyAsync(b->d_k, k + static_cast<size_t>(at) * b->row_len(), bytes, cudaMemcpyHostToDevice,
                                    b->stream), "k upload");
        ITK_CUDA(b, cudaMemcpyAsync(b->d_v, v + static_cast<size_t>(at) * b->row_len(), bytes, cudaMemcpyHostToDevice,
                                    b->stream), "v upload");
        SeqDesc d{slot, static_cast<uint32_t>(start + at), 0, static_cast<uint32_t>(start + at + m)};
        if (int rc = run_append(b, layer, 1, &d, m, b->d_k, b->d_v)) return rc;
        ITK_CUDA(b, cudaStreamSynchronize(b->stream), "append");
    }
    st.appended[layer] += rows;
    st.built = true;
    b->stats.rows_appended += rows;
    return ITK_OK;
}

int itk_append_rows_device(itk_backend* b, uint32_t layer, uint32_t n_seqs, const uint32_t* slots,
                           const uint64_t* starts, uint32_t rows, const float* d_k, const float* d_v) {
    if (!b || !slots || !starts || !d_k || !d_v) return ITK_ERR_INVALID_ARGUMENT;
    if (int rc = check_device_alignment(b, "append", d_k, d_v)) return rc;
    cudaSetDevice(b->cfg.device);
    if (int rc = check_layer(b, layer)) return rc;
    if (n_seqs == 0 || rows == 0) return ITK_OK;
    std::vector<SeqDesc> seqs(n_seqs);
    for (uint32_t i = 0; i < n_seqs; ++i) {
        if (int rc = check_slot(b, slots[i])) return rc;
        for (uint32_t j = 0; j < i; ++j)
            if (slots[j] == slots[i])
                return b->fail(ITK_ERR_INVALID_ARGUMENT, "append: slot " + zu(slots[i]) + " listed twice");
        const SlotState& st = b->slots[slots[i]];
        if (st.live) {
            const uint64_t limit = st.bases[layer] + st.max_round;
            if (starts[i] + rows > limit) {
                const uint64_t bad = starts[i] > limit ? starts[i] : limit;
                return b->fail(ITK_ERR_CHECKPOINT_RANGE_EXCEEDED,
                               "layer " + zu(layer) + " append at position " + zu(bad) +
                                   " is outside the live checkpoint's saved range (first unsaved position " + zu(limit) +
                                   "); refusing so a later rewind cannot meet a slot it cannot restore");
            }
        }
        if (starts[i] != st.appended[layer])
            return b->fail(ITK_ERR_OUT_OF_ORDER_POSITION, "layer " + zu(layer) + " appends must be in order: expected position " +
                                                              zu(st.appended[layer]) + ", got " + zu(starts[i]));
        if (b->window[layer] == 0 && starts[i] + rows > b->ring[layer])
            return b->fail(ITK_ERR_CAPACITY, "append: position " + zu(starts[i] + rows) +
                                                 " is past the slot's context capacity of " + zu(b->ring[layer]) + " positions");
        if (b->window[layer] != 0 && rows > b->ring[layer])
            return b->fail(ITK_ERR_CAPACITY, "append: " + zu(rows) + " rows exceed the ring of " + zu(b->ring[layer]));
        if (starts[i] + rows > 0xfffffff0ull) return b->fail(ITK_ERR_CAPACITY, "append: position exceeds 32 bits");
        seqs[i] = SeqDesc{slots[i], static_cast<uint32_t>(starts[i]), 0, static_cast<uint32_t>(starts[i] + rows)};
    }
    if (int rc = run_append(b, layer, n_seqs, seqs.data(), rows, d_k, d_v)) return rc;
    for (uint32_t i = 0; i < n_seqs; ++i) {
        b->slots[slots[i]].appended[layer] += rows;
        b->slots[slots[i]].built = true;
    }
    b->stats.rows_appended += static_cast<uint64_t>(n_seqs) * rows;
    return ITK_OK;
}

int itk_append(itk_backend* b, uint32_t slot, uint32_t layer, const float* k, size_t k_len, const float* v,
               size_t v_len, uint64_t position) {
    if (!b) return ITK_ERR_INVALID_ARGUMENT;
    const size_t row = b->row_len();
    if (k_len != row) return b->fail(ITK_ERR_SHAPE_MISMATCH, "k: got " + zu(k_len) + ", expected " + zu(row));
    if (v_len != row) return b->fail(ITK_ERR_SHAPE_MISMATCH, "v: got " + zu(v_len) + ", expected " + zu(row));
    return itk_append_rows(b, slot, layer, k, v, 1, position);
}

int itk_next_position(const itk_backend* b, uint32_t slot, uint32_t layer, uint64_t* out) {
    if (!b || !out) return ITK_ERR_INVALID_ARGUMENT;
    if (int rc = check_slot(b, slot)) return rc;
    if (int rc = check_layer(b, layer)) return rc;
    *out = b->slots[slot].appended[layer];
    return ITK_OK;
}

int itk_stored_len(const itk_backend* b, uint32_t slot, uint32_t layer, uint64_t* out) {
    if (!b || !out) return ITK_ERR_INVALID_ARGUMENT;
    if (int rc = check_slot(b, slot)) return rc;
    if (int rc = check_layer(b, layer)) return rc;
    *out = b->stored(layer, b->slots[slot].appended[layer]);
    return ITK_OK;
}

int itk_view_gather(itk_backend* b, uint32_t slot, uint32_t layer, void* keys, void* values, uint64_t* first_position,
                    uint64_t* rows) {
    if (!b) return ITK_ERR_INVALID_ARGUMENT;
    cudaSetDevice(b->cfg.device);
    if (int rc = check_slot(b, slot)) return rc;
    if (int rc = check_layer(b, layer)) return rc;
    const uint64_t appended = b->slots[slot].appended[layer];
    const uint64_t n = b->stored(layer, appended);
    if (first_position) *first_position = appended - n;
    if (rows) *rows = n;
    if (n == 0 || (!keys && !values)) return ITK_OK;
    const uint64_t block = n * b->row_len();
    if (int rc = ensure_gather(b, 2 * block * b->elem_bytes)) return rc;
    if (int rc = run_copy(b, slot, b->gather_buf, {layer}, {appended - n}, {n}, {0}, {block}, true)) return rc;
    unsigned char* base = static_cast<unsigned char*>(b->gather_buf);
    if (keys)
        ITK_CUDA(b, cudaMemcpyAsync(keys, base, block * b->elem_bytes, cudaMemcpyDeviceToHost, b->stream), "view download");
    if (values)
        ITK_CUDA(b, cudaMemcpyAsync(values, base + block * b->elem_bytes, block * b->elem_bytes, cudaMemcpyDeviceToHost,
                                    b->stream), "view download");
    ITK_CUDA(b, cudaStreamSynchronize(b->stream), "view gather");
    return ITK_OK;
}

int itk_restore_bulk(itk_backend* b, uint32_t slot, uint32_t layer, uint64_t first_position, const float* keys,
                     size_t keys_len, const float* values, size_t values_len) {
    if (!b) return ITK_ERR_INVALID_ARGUMENT;
    cudaSetDevice(b->cfg.device);
    if (int rc = check_slot(b, slot)) return rc;
    // crates/attention/src/cache.rs:520-557, same order.
    const size_t row = b->row_len();
    if (keys_len != values_len || keys_len % row != 0)
        return b->fail(ITK_ERR_SHAPE_MISMATCH, "bulk restore rows: got " + zu(keys_len) + ", expected " + zu(values_len));
    const uint64_t rows = keys_len / row;
    if (int rc = check_layer(b, layer)) return rc;
    SlotState& st = b->slots[slot];
    if (st.appended[layer] != 0)
        return b->fail(ITK_ERR_BULK_RESTORE_NOT_FRESH, "layer " + zu(layer) + " already holds " + zu(st.appended[layer]) +
                                                           " appended positions; bulk restore installs into a fresh layer only");
    if (b->window[layer] == 0) {
        if (first_position != 0)
            return b->fail(ITK_ERR_SHAPE_MISMATCH,
                           "bulk restore first position (global layer): got " + zu(first_position) + ", expected 0");
        if (rows > b->ring[layer])
            return b->fail(ITK_ERR_CAPACITY, "bulk restore: " + zu(rows) + " rows exceed the context capacity of " +
                                                 zu(b->ring[layer]));
    } else if (rows > b->window[layer]) {
        return b->fail(ITK_ERR_SHAPE_MISMATCH, "bulk restore rows (windowed layer): got " + zu(rows) + ", expected " +
                                                   zu(b->window[layer]));
    }
    if (first_position + rows > 0xfffffff0ull) return b->fail(ITK_ERR_CAPACITY, "bulk restore: position exceeds 32 bits");
    // Install = the append scatter at positions first_position.. (same storage-row law), without the order check.
    for (uint64_t at = 0; at < rows; at += b->stage_rows) {
        const uint32_t m = static_cast<uint32_t>((rows - at < b->stage_rows) ? rows - at : b->stage_rows);
        const size_t bytes = static_cast<size_t>(m) * row * sizeof(float);
        ITK_CUDA(b, cudaMemcpyAsync(b->d_k, keys + at * row, bytes, cudaMemcpyHostToDevice, b->stream), "k upload");
        ITK_CUDA(b, cudaMemcpyAsync(b->d_v, values + at * row, bytes, cudaMemcpyHostToDevice, b->stream), "v upload");
        SeqDesc d{slot, static_cast<uint32_t>(first_position + at), 0, static_cast<uint32_t>(first_position + at + m)};
        if (int rc = run_append(b, layer, 1, &d, m, b->d_k, b->d_v)) return rc;
        ITK_CUDA(b, cudaStreamSynchronize(b->stream), "bulk restore");
    }
    st.appended[layer] = first_position + rows;
    st.built = true;
    return ITK_OK;
}

int itk_reset(itk_backend* b, uint32_t slot) {
    if (!b) return ITK_ERR_INVALID_ARGUMENT;
    cudaSetDevice(b->cfg.device);
    if (int rc = check_slot(b, slot)) return rc;
    b->tc_chain_live = false;
    // Ring layers read as zero-filled until written, like a fresh reference cache.
    for (uint32_t l = 0; l < b->cfg.n_layers; ++l)
        if (b->window[l] && b->slots[slot].appended[l] != 0) {
            const size_t bytes = static_cast<size_t>(b->ring[l]) * b->row_len() * b->elem_bytes;
            const size_t off = static_cast<size_t>(slot) * b->ring[l] * b->row_len() * b->elem_bytes;
            cudaMemsetAsync(static_cast<unsigned char*>(b->layer_ptr(b->k_slab, l)) + off, 0, bytes, b->stream);
            cudaMemsetAsync(static_cast<unsigned char*>(b->layer_ptr(b->v_slab, l)) + off, 0, bytes, b->stream);
        }
    drop_slot(b, slot);
    return ITK_OK;
}

int itk_cache_checkpoint(itk_backend* b, uint32_t slot, uint64_t max_round_tokens, itk_checkpoint* out) {
    if (!b || !out) return ITK_ERR_INVALID_ARGUMENT;
    if (int rc = check_slot(b, slot)) return rc;
    SlotState& st = b->slots[slot];
    if (!st.built)
        return b->fail(ITK_ERR_STEP_FAILED,
                       "cache_checkpoint: no KV state exists yet: a speculative round checkpoints after a first forward "
                       "has built the cache (the spec's prefill), not before");
    if (st.live)
        return b->fail(ITK_ERR_CHECKPOINT_BUSY,
                       "a checkpoint is already outstanding on this cache; release it before taking another");
    if (max_round_tokens == 0) return b->fail(ITK_ERR_ZERO_DIMENSION, "max_round_tokens must be positive, got 0");
    uint32_t smallest = 0;
    for (uint32_t w : b->window)
        if (w && (smallest == 0 || w < smallest)) smallest = w;
    if (smallest && max_round_tokens > smallest)
        return b->fail(ITK_ERR_CHECKPOINT_TOO_DEEP,
                       "checkpoint round bound " + zu(max_round_tokens) + " exceeds the smallest sliding window " +
                           zu(smallest) + ": a round that long would overwrite a ring slot twice and no rewind could be exact");
    if (smallest && max_round_tokens > b->cfg.chunk_cap)
        return b->fail(ITK_ERR_CHECKPOINT_TOO_DEEP,
                       "checkpoint round bound " + zu(max_round_tokens) + " exceeds the ring headroom (chunk cap " +
                           zu(b->cfg.chunk_cap) + "): discarded rows could alias rows a later query still sees");
    st.next_serial += 1;
    st.live = true;
    st.live_serial = st.next_serial;
    st.max_round = max_round_tokens;
    st.bases = st.appended;
    out->id = st.id;
    out->serial = st.live_serial;
    out->base = st.bases[0];
    out->max_round_tokens = max_round_tokens;
    return ITK_OK;
}

int itk_cache_rewind(itk_backend* b, uint32_t slot, const itk_checkpoint* cp, uint64_t target) {
    if (!b || !cp) return ITK_ERR_INVALID_ARGUMENT;
    if (int rc = check_slot(b, slot)) return rc;
    SlotState& st = b->slots[slot];
    if (int rc = check_live(b, st, cp)) return rc;
    for (uint32_t l = 0; l < b->cfg.n_layers; ++l)
        if (target < st.bases[l] || target > st.appended[l])
            return b->fail(ITK_ERR_REWIND_OUT_OF_RANGE, "rewind target " + zu(target) + " is outside layer " + zu(l) +
                                                            "'s checkpoint range [" + zu(st.bases[l]) + ", " +
                                                            zu(st.appended[l]) + "]");
    // Rows live at position % ring and every view derives from the position, so
    // truncation is the counter alone: rows past `target` are never read and the
    // next append overwrites them in place.
    for (uint32_t l = 0; l < b->cfg.n_layers; ++l) st.appended[l] = target;
    return ITK_OK;
}

int itk_cache_release(itk_backend* b, uint32_t slot, const itk_checkpoint* cp) {
    if (!b || !cp) return ITK_ERR_INVALID_ARGUMENT;
    if (int rc = check_slot(b, slot)) return rc;
    SlotState& st = b->slots[slot];
    if (int rc = check_live(b, st, cp)) return rc;
    st.live = false;
    return ITK_OK;
}

int itk_snapshot_capture(itk_backend* b, uint32_t slot, itk_snapshot** out) {
    if (!b || !out) return ITK_ERR_INVALID_ARGUMENT;
    cudaSetDevice(b->cfg.device);
    if (int rc = check_slot(b, slot)) return rc;
    const SlotState& st = b->slots[slot];
    const uint64_t tokens = st.appended[0];
    for (uint32_t l = 0; l < b->cfg.n_layers; ++l)
        if (st.appended[l] != tokens)
            return b->fail(ITK_ERR_INCOHERENT_CACHE, "incoherent cache: layer 0 has appended " + zu(tokens) +
                                                         " positions but layer " + zu(l) + " has appended " +
                                                         zu(st.appended[l]) + "; a snapshot is one sequence");
    itk_snapshot* s = new (std::nothrow) itk_snapshot();
    if (!s) return b->fail(ITK_ERR_CUDA, "out of host memory");
    s->device = b->cfg.device;
    s->f16 = b->f16;
    s->kv_heads = b->cfg.kv_heads;
    s->head_dim = b->cfg.head_dim;
    s->window = b->window;
    s->token_count = tokens;
    std::vector<uint32_t> layers;
    uint64_t at = 0;
    for (uint32_t l = 0; l < b->cfg.n_layers; ++l) {
        const uint64_t rows = b->stored(l, tokens);
        s->first.push_back(tokens - rows);
        s->rows.push_back(rows);
        s->k_off.push_back(at);
        at += rows * b->row_len();
        s->v_off.push_back(at);
        at += rows * b->row_len();
        layers.push_back(l);
    }
    s->total_elems = at;
    if (at) {
        cudaError_t e = cudaMalloc(&s->data, at * b->elem_bytes);
        if (e != cudaSuccess) {
            delete s;
            return b->cuda_fail(e, "snapshot allocation");
        }
        if (int rc = run_copy(b, slot, s->data, layers, s->first, s->rows, s->k_off, s->v_off, true)) {
            itk_snapshot_free(s);
            return rc;
        }
    }
    b->stats.prefix_captures += 1;
    *out = s;
    return ITK_OK;
}

int itk_snapshot_restore(itk_backend* b, uint32_t slot, const itk_snapshot* s) {
    if (!b || !s) return ITK_ERR_INVALID_ARGUMENT;
    cudaSetDevice(b->cfg.device);
    if (int rc = check_slot(b, slot)) return rc;
    // crates/wgpu-compute/src/session.rs:410-467: geometry, then empty, then capacity - all before any state moves.
    if (s->window != b->window || s->kv_heads != b->cfg.kv_heads || s->head_dim != b->cfg.head_dim)
        return b->fail(ITK_ERR_GEOMETRY_MISMATCH,
                       "geometry mismatch: snapshot geometry (" + zu(s->window.size()) + " layers, " + zu(s->kv_heads) +
                           " KV heads, head dim " + zu(s->head_dim) + ") differs from the session geometry (" +
                           zu(b->window.size()) + " layers, " + zu(b->cfg.kv_heads) + " KV heads, head dim " +
                           zu(b->cfg.head_dim) + ")");
    if (s->f16 != b->f16 || s->device != b->cfg.device)
        return b->fail(ITK_ERR_GEOMETRY_MISMATCH, "geometry mismatch: snapshot element type or device differs from the backend's");
    if (s->token_count == 0)
        return b->fail(ITK_ERR_STEP_FAILED, "prefix_install: snapshot covers zero tokens; an empty prefix installs nothing "
                                            "and is refused rather than resetting the session to no effect");
    if (s->token_count > b->cfg.max_context)
        return b->fail(ITK_ERR_STEP_FAILED, "prefix_install: snapshot covers " + zu(s->token_count) +
                                                " tokens, past the session's context capacity of " +
                                                zu(b->cfg.max_context) + " positions");
    if (int rc = itk_reset(b, slot)) return rc;
    std::vector<uint32_t> layers;
    for (uint32_t l = 0; l < b->cfg.n_layers; ++l) layers.push_back(l);
    if (int rc = run_copy(b, slot, s->data, layers, s->first, s->rows, s->k_off, s->v_off, false)) return rc;
    SlotState& st = b->slots[slot];
    for (uint32_t l = 0; l < b->cfg.n_layers; ++l) st.appended[l] = s->token_count;
    st.built = true;
    b->stats.prefix_restores += 1;
    return ITK_OK;
}

void itk_snapshot_free(itk_snapshot* s) {
    if (!s) return;
    if (s->data) {
        cudaSetDevice(s->device);
        cudaFree(s->data);
    }
    delete s;
}

uint64_t itk_snapshot_token_count(const itk_snapshot* s) { return s ? s->token_count : 0; }
uint64_t itk_snapshot_payload_bytes(const itk_snapshot* s) { return s ? s->total_elems * (s->f16 ? 2 : 4) : 0; }

int itk_snapshot_layer_to_host(itk_backend* b, const itk_snapshot* s, uint32_t layer, void* keys, void* values,
                               uint64_t* first_position, uint64_t* rows) {
    if (!b || !s) return ITK_ERR_INVALID_ARGUMENT;
    cudaSetDevice(b->cfg.device);
    if (layer >= s->rows.size())
        return b->fail(ITK_ERR_INVALID_LAYER, "layer " + zu(layer) + " out of range, cache has " + zu(s->rows.size()) + " layers");
    if (first_position) *first_position = s->first[layer];
    if (rows) *rows = s->rows[layer];
    const size_t eb = s->f16 ? 2 : 4;
    const size_t bytes = s->rows[layer] * s->kv_heads * s->head_dim * eb;
    if (bytes == 0) return ITK_OK;
    const unsigned char* base = static_cast<const unsigned char*>(s->data);
    if (keys) ITK_CUDA(b, cudaMemcpyAsync(keys, base + s->k_off[layer] * eb, bytes, cudaMemcpyDeviceToHost, b->stream), "snapshot download");
    if (values) ITK_CUDA(b, cudaMemcpyAsync(values, base + s->v_off[layer] * eb, bytes, cudaMemcpyDeviceToHost, b->stream), "snapshot download");
    ITK_CUDA(b, cudaStreamSynchronize(b->stream), "snapshot download");
    return ITK_OK;
}

int itk_snapshot_from_host_f32(itk_backend* b, uint64_t token_count, const uint64_t* first_position,
                               const uint64_t* rows, const float* const* keys, const float* const* values,
                               itk_snapshot** out) {
    if (!b || !first_position || !rows || !keys || !values || !out) return ITK_ERR_INVALID_ARGUMENT;
    cudaSetDevice(b->cfg.device);
    // crates/itak-kv/src/snapshot.rs:187-236: per-layer rows and first positions follow from the token count.
    for (uint32_t l = 0; l < b->cfg.n_layers; ++l) {
        const uint64_t want_rows = b->stored(l, token_count);
        if (first_position[l] != token_count - want_rows)
            return b->fail(ITK_ERR_INCONSISTENT_SNAPSHOT,
                           "inconsistent snapshot: layer " + zu(l) + ": first stored position is " + zu(first_position[l]) +
                               " but " + zu(token_count - want_rows) + " follows from token count " + zu(token_count));
        if (rows[l] != want_rows)
            return b->fail(ITK_ERR_INCONSISTENT_SNAPSHOT, "inconsistent snapshot: layer " + zu(l) + ": holds " + zu(rows[l]) +
                                                              " rows but " + zu(want_rows) + " rows were expected");
    }
    itk_snapshot* s = new (std::nothrow) itk_snapshot();
    if (!s) return b->fail(ITK_ERR_CUDA, "out of host memory");
    s->device = b->cfg.device;
    s->f16 = b->f16;
    s->kv_heads = b->cfg.kv_heads;
    s->head_dim = b->cfg.head_dim;
    s->window = b->window;
    s->token_count = token_count;
    uint64_t at = 0, largest = 0;
    for (uint32_t l = 0; l < b->cfg.n_layers; ++l) {
        const uint64_t block = rows[l] * b->row_len();
        s->first.push_back(first_position[l]);
        s->rows.push_back(rows[l]);
        s->k_off.push_back(at);
        at += block;
        s->v_off.push_back(at);
        at += block;
        if (block > largest) largest = block;
    }
    s->total_elems = at;
    if (at) {
        cudaError_t e = cudaMalloc(&s->data, at * b->elem_bytes);
        if (e != cudaSuccess) {
            delete s;
            return b->cuda_fail(e, "snapshot allocation");
        }
        float* tmp = nullptr;
        e = cudaMalloc(&tmp, largest * sizeof(float));
        if (e != cudaSuccess) {
            itk_snapshot_free(s);
            return b->cuda_fail(e, "snapshot staging allocation");
        }
        for (uint32_t l = 0; l < b->cfg.n_layers && e == cudaSuccess; ++l) {
            const uint64_t block = rows[l] * b->row_len();
            if (block == 0) continue;
            for (int which = 0; which < 2 && e == cudaSuccess; ++which) {
                const float* src = which ? values[l] : keys[l];
                const uint64_t off = which ? s->v_off[l] : s->k_off[l];
                e = cudaMemcpyAsync(tmp, src, block * sizeof(float), cudaMemcpyHostToDevice, b->stream);
                if (e == cudaSuccess)
                    e = itk::launch_convert(tmp, static_cast<unsigned char*>(s->data) + off * b->elem_bytes, block, b->f16,
                                            b->stream, &b->stats.kernel_launches);
                if (e == cudaSuccess) e = cudaStreamSynchronize(b->stream);
            }
        }
        cudaFree(tmp);
        if (e != cudaSuccess) {
            itk_snapshot_free(s);
            return b->cuda_fail(e, "snapshot import");
        }
    }
    *out = s;
    return ITK_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------
// The ITKV wire format (crates/itak-kv/src/snapshot.rs:13-29).  Host-side byte handling only; the rows move
// through itk_snapshot_layer_to_host / itk_snapshot_from_host_f32.
// ---------------------------------------------------------------------------------------------------------
namespace {

// Exact f16 -> f32 (crates/gguf/src/dequant.rs:12-34).
float half_bits_to_float(uint16_t h) {
    const uint32_t sign = h >> 15, exp = (h >> 10) & 0x1f, frac = h & 0x3ff;
    uint32_t out;
    if (exp == 0x1f) {
        out = (sign << 31) | (frac == 0 ? 0x7f800000u : (0x7fc00000u | (frac << 13)));
    } else if (exp == 0) {
        if (frac == 0) {
            out = sign << 31;
        } else {
            const float v = static_cast<float>(frac) * 5.9604644775390625e-8f;  // frac * 2^-24, exact
            return sign ? -v : v;
        }
    } else {
        out = (sign << 31) | ((exp + 112) << 23) | (frac << 13);
    }
    float f;
    std::memcpy(&f, &out, 4);
    return f;
}

void put_u32(std::vector<uint8_t>& b, uint32_t v) {
    for (int i = 0; i < 4; ++i) b.push_back(static_cast<uint8_t>(v >> (8 * i)));
}
void put_u64(std::vector<uint8_t>& b, uint64_t v) {
    for (int i = 0; i < 8; ++i) b.push_back(static_cast<uint8_t>(v >> (8 * i)));
}

using itk::itkv::fnv1a64;

}  // namespace

extern "C" {

int itk_snapshot_to_itkv(itk_backend* b, const itk_snapshot* s, const char* model_fingerprint, uint8_t* out,
                         size_t capacity, size_t* size) {
    return itk_snapshot_to_itkv_version(b, s, model_fingerprint, itk::itkv::kVersionF32, out, capacity, size);
}

int itk_snapshot_to_itkv_version(itk_backend* b, const itk_snapshot* s, const char* model_fingerprint, uint32_t version,
                                 uint8_t* out, size_t capacity, size_t* size) {
    if (!b || !s || !model_fingerprint || !size) return ITK_ERR_INVALID_ARGUMENT;
    if (version != itk::itkv::kVersionF32 && version != itk::itkv::kVersionTyped)
        return b->fail(ITK_ERR_UNSUPPORTED_VERSION, "snapshot: unsupported format version " + zu(version));
    // version 1 always carries f32 rows; version 2 carries the snapshot's own element type
    const bool halves_out = version == itk::itkv::kVersionTyped && s->f16;
    const size_t out_elem = halves_out ? 2 : 4;
    const size_t fp_len = std::strlen(model_fingerprint);
    const size_t n_layers = s->rows.size();
    const size_t row = static_cast<size_t>(s->kv_heads) * s->head_dim;
    size_t payload = 0;
    for (size_t l = 0; l < n_layers; ++l) payload += static_cast<size_t>(s->rows[l]) * row * 2 * out_elem;
    const size_t total = 4 + 4 + (version == itk::itkv::kVersionTyped ? 4 : 0) + 4 + fp_len + 8 + 4 + 4 + 4 + 28 * n_layers +
                         payload + 8;
    *size = total;
    if (!out) return ITK_OK;
    if (capacity < total)
        return b->fail(ITK_ERR_CAPACITY, "snapshot encode: buffer holds " + zu(capacity) + " bytes, " + zu(total) + " needed");
    std::vector<uint8_t> head;
    head.insert(head.end(), {'I', 'T', 'K', 'V'});
    put_u32(head, version);
    if (version == itk::itkv::kVersionTyped) put_u32(head, s->f16 ? itk::itkv::kElemF16 : itk::itkv::kElemF32);
    put_u32(head, static_cast<uint32_t>(fp_len));
    head.insert(head.end(), model_fingerprint, model_fingerprint + fp_len);
    put_u64(head, s->token_count);
    put_u32(head, s->kv_heads);
    put_u32(head, s->head_dim);
    put_u32(head, static_cast<uint32_t>(n_layers));
    for (size_t l = 0; l < n_layers; ++l) {
        head.push_back(s->window[l] ? 1 : 0);
        head.push_back(0);
        head.push_back(0);
        head.push_back(0);
        put_u64(head, s->window[l]);
        put_u64(head, s->first[l]);
        put_u64(head, s->rows[l]);
    }
    std::memcpy(out, head.data(), head.size());
    size_t at = head.size();
    std::vector<uint16_t> halves;
    for (size_t l = 0; l < n_layers; ++l) {
        const size_t elems = static_cast<size_t>(s->rows[l]) * row;
        if (elems == 0) continue;
        uint8_t* kbytes = out + at;  // may be unaligned for f32: filled through memcpy below
        uint8_t* vbytes = out + at + elems * out_elem;
        if (halves_out) {
            // the half bit patterns as they sit in the cache (this host is little-endian, like the format)
            halves.resize(2 * elems);
            if (int rc = itk_snapshot_layer_to_host(b, s, static_cast<uint32_t>(l), halves.data(), halves.data() + elems, nullptr, nullptr))
                return rc;
            std::memcpy(kbytes, halves.data(), elems * 2);
            std::memcpy(vbytes, halves.data() + elems, elems * 2);
        } else if (!s->f16) {
            // the payload offset is arbitrary, so download to aligned scratch and copy the bytes
            std::vector<float> tmp(2 * elems);
            if (int rc = itk_snapshot_layer_to_host(b, s, static_cast<uint32_t>(l), tmp.data(), tmp.data() + elems, nullptr, nullptr))
                return rc;
            std::memcpy(kbytes, tmp.data(), elems * sizeof(float));
            std::memcpy(vbytes, tmp.data() + elems, elems * sizeof(float));
        } else {
            halves.resize(2 * elems);
            if (int rc = itk_snapshot_layer_to_host(b, s, static_cast<uint32_t>(l), halves.data(), halves.data() + elems, nullptr, nullptr))
                return rc;
            for (size_t i = 0; i < elems; ++i) {
                const float kf = half_bits_to_float(halves[i]), vf = half_bits_to_float(halves[elems + i]);
                std::memcpy(kbytes + 4 * i, &kf, 4);
                std::memcpy(vbytes + 4 * i, &vf, 4);
            }
        }
        at += 2 * elems * out_elem;
    }
    const uint64_t sum = fnv1a64(out, at);
    for (int i = 0; i < 8; ++i) out[at + i] = static_cast<uint8_t>(sum >> (8 * i));
    return ITK_OK;
}

int itk_snapshot_from_itkv(itk_backend* b, const uint8_t* bytes, size_t n, const char* expected_fingerprint,
                           itk_snapshot** out) {
    if (!b || !bytes || !out) return ITK_ERR_INVALID_ARGUMENT;
    itk::itkv::Parsed parsed;
    std::string why;
    if (int rc = itk::itkv::parse(bytes, n, &parsed, &why)) return b->fail(rc, why);
    const uint64_t token_count = parsed.token_count;
    const uint32_t hkv = parsed.kv_heads, hd = parsed.head_dim, layer_count = parsed.layer_count;
    const std::vector<uint64_t>&windows = parsed.windows, &firsts = parsed.firsts, &rows = parsed.rows;
    const std::vector<const uint8_t*>&kptr = parsed.kptr, &vptr = parsed.vptr;
    const uint64_t row = static_cast<uint64_t>(hkv) * hd;
    // restore_checked (snapshot.rs:345-371): geometry, then fingerprint
    bool same = layer_count == b->cfg.n_layers && hkv == b->cfg.kv_heads && hd == b->cfg.head_dim;
    for (uint32_t l = 0; same && l < layer_count; ++l) same = windows[l] == b->window[l];
    if (!same)
        return b->fail(ITK_ERR_GEOMETRY_MISMATCH, "geometry mismatch: snapshot geometry (" + zu(layer_count) + " layers, " +
                                                      zu(hkv) + " KV heads, head dim " + zu(hd) +
                                                      ") differs from the required geometry (" + zu(b->cfg.n_layers) +
                                                      " layers, " + zu(b->cfg.kv_heads) + " KV heads, head dim " +
                                                      zu(b->cfg.head_dim) + ")");
    if (expected_fingerprint) {
        const std::string& have = parsed.fingerprint;
        if (have != expected_fingerprint)
            return b->fail(ITK_ERR_FINGERPRINT_MISMATCH,
                           std::string("fingerprint mismatch: expected ") + expected_fingerprint + ", snapshot has " + have);
    }
    if (parsed.elem_bytes == 2 && b->f16) {
        // Half rows into a half cache: the bit patterns are installed as they are (no conversion, no rounding).
        itk_snapshot* s = new (std::nothrow) itk_snapshot();
        if (!s) return b->fail(ITK_ERR_CUDA, "out of host memory");
        cudaSetDevice(b->cfg.device);
        s->device = b->cfg.device;
        s->f16 = true;
        s->kv_heads = hkv;
        s->head_dim = hd;
        s->window = b->window;
        s->token_count = token_count;
        uint64_t at = 0;
        for (uint32_t l = 0; l < layer_count; ++l) {
            s->first.push_back(firsts[l]);
            s->rows.push_back(rows[l]);
            s->k_off.push_back(at);
            at += rows[l] * row;
            s->v_off.push_back(at);
            at += rows[l] * row;
        }
        s->total_elems = at;
        if (at) {
            cudaError_t e = cudaMalloc(&s->data, at * 2);
            for (uint32_t l = 0; l < layer_count && e == cudaSuccess; ++l) {
                const size_t nbytes = static_cast<size_t>(rows[l] * row) * 2;
                if (nbytes == 0) continue;
                unsigned char* base = static_cast<unsigned char*>(s->data);
                e = cudaMemcpyAsync(base + s->k_off[l] * 2, kptr[l], nbytes, cudaMemcpyHostToDevice, b->stream);
                if (e == cudaSuccess)
                    e = cudaMemcpyAsync(base + s->v_off[l] * 2, vptr[l], nbytes, cudaMemcpyHostToDevice, b->stream);
            }
            if (e == cudaSuccess) e = cudaStreamSynchronize(b->stream);  // the source bytes belong to the caller
            if (e != cudaSuccess) {
                itk_snapshot_free(s);
                return b->cuda_fail(e, "snapshot import");
            }
        }
        *out = s;
        return ITK_OK;
    }
    // the payload sits at arbitrary byte offsets: copy the rows into aligned storage before the upload (half rows
    // bound for an f32 cache are widened exactly on the way)
    std::vector<std::vector<float>> ks(layer_count), vs(layer_count);
    std::vector<const float*> kp(layer_count), vp(layer_count);
    for (uint32_t l = 0; l < layer_count; ++l) {
        const size_t floats = static_cast<size_t>(rows[l] * row);
        ks[l].resize(floats ? floats : 1);
        vs[l].resize(floats ? floats : 1);
        if (floats && parsed.elem_bytes == 4) {
            std::memcpy(ks[l].data(), kptr[l], floats * 4);
            std::memcpy(vs[l].data(), vptr[l], floats * 4);
        } else if (floats) {
            for (size_t i = 0; i < floats; ++i) {
                uint16_t hk, hv;
                std::memcpy(&hk, kptr[l] + 2 * i, 2);
                std::memcpy(&hv, vptr[l] + 2 * i, 2);
                ks[l][i] = half_bits_to_float(hk);
                vs[l][i] = half_bits_to_float(hv);
            }
        }
        kp[l] = ks[l].data();
        vp[l] = vs[l].data();
    }
    return itk_snapshot_from_host_f32(b, token_count, firsts.data(), rows.data(), kp.data(), vp.data(), out);
}

}  // extern "C"
