// C entry points over the CPU oracle (kv_oracle.hpp) so tests and the bench's
// CPU-baseline leg can drive it through ctypes. TEST INFRASTRUCTURE ONLY: the
// shipped library never links or loads this file.
//
// Every call returns an orc::Code; the text of the last refusal on the calling
// thread is available through orc_last_error().
#include "kv_oracle.hpp"

#include <atomic>
#include <chrono>
#include <thread>

using namespace orc;

namespace {
thread_local std::string g_last_error;
int done(const Status& st) {
    g_last_error = st.msg;
    return st.code;
}
std::vector<LayerKind> pattern_of(const int32_t* windowed, const uint64_t* windows, size_t n) {
    std::vector<LayerKind> p;
    for (size_t i = 0; i < n; ++i) p.push_back(LayerKind{windowed[i] != 0, static_cast<size_t>(windows[i])});
    return p;
}
}  // namespace

extern "C" {

struct orc_checkpoint_t {
    uint64_t cache_id;
    uint64_t serial;
    uint64_t max_round_tokens;
    uint64_t saved_bytes;
};

const char* orc_last_error() { return g_last_error.c_str(); }

// ---- conversions and RoPE --------------------------------------------------
void orc_f32_to_f16_bits(const float* in, uint16_t* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = f32_to_f16_bits(in[i]);
}
void orc_f16_bits_to_f32(const uint16_t* in, float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = f16_bits_to_f32(in[i]);
}
void orc_round_through_f16(const float* in, float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = round_through_f16(in[i]);
}
// pairing: 0 = adjacent pairs (2i, 2i+1); 1 = half split (i, i + rotary/2).
int orc_rope(int pairing, const float* in, size_t len, size_t position, float base, size_t head_dim,
             size_t rotary_dim, float* out) {
    return done(pairing == 0 ? rope_interleaved_partial(in, len, position, base, head_dim, rotary_dim, out)
                             : rope_half_partial(in, len, position, base, head_dim, rotary_dim, out));
}
// Rotate `rows` consecutive positions of `[rows][heads][head_dim]` in one call.
int orc_rope_rows(int pairing, const float* in, size_t rows, size_t heads, size_t head_dim, size_t start_position,
                  float base, float* out) {
    for (size_t r = 0; r < rows; ++r)
        for (size_t h = 0; h < heads; ++h) {
            const size_t off = (r * heads + h) * head_dim;
            Status st = pairing == 0
                            ? rope_interleaved_partial(in + off, head_dim, start_position + r, base, head_dim, head_dim, out + off)
                            : rope_half_partial(in + off, head_dim, start_position + r, base, head_dim, head_dim, out + off);
            if (!st.ok()) return done(st);
        }
    return done({});
}
int orc_rms_norm(const float* in, size_t len, const float* weight, size_t weight_len, float eps, float* out) {
    return done(rms_norm(in, len, weight, weight_len, eps, out));
}
int orc_draft_attention(const float* q, size_t rows, size_t q_heads, size_t kv_heads, size_t key_len, size_t value_len,
                        const uint64_t* positions, const uint64_t* committed_positions, size_t committed,
                        const float* committed_k, const float* committed_v, const float* block_k, const float* block_v,
                        int causal, int sliding, uint64_t window, float* out) {
    return done(draft_attention(q, rows, q_heads, kv_heads, key_len, value_len, positions, committed_positions, committed,
                                committed_k, committed_v, block_k, block_v, causal != 0, sliding != 0, window, out));
}
float orc_default_scale(size_t head_dim) { return default_scale(head_dim); }
int orc_kv_head_for_query_head(size_t q_head, size_t hq, size_t hkv, size_t* out) {
    return done(kv_head_for_query_head(q_head, hq, hkv, out));
}

// ---- cache -----------------------------------------------------------------
int orc_cache_new(const int32_t* windowed, const uint64_t* windows, size_t n_layers, size_t num_kv_heads,
                  size_t head_dim, void** out) {
    std::unique_ptr<KvCache> c;
    Status st = KvCache::create(pattern_of(windowed, windows, n_layers), num_kv_heads, head_dim, &c);
    if (st.ok()) *out = c.release();
    return done(st);
}
void orc_cache_free(void* c) { delete static_cast<KvCache*>(c); }
uint64_t orc_cache_id(void* c) { return static_cast<KvCache*>(c)->id(); }
size_t orc_cache_layer_count(void* c) { return static_cast<KvCache*>(c)->layer_count(); }
int orc_cache_layer_kind(void* c, size_t layer, int32_t* windowed, uint64_t* window) {
    LayerKind k;
    Status st = static_cast<KvCache*>(c)->layer_kind(layer, &k);
    if (st.ok()) {
        *windowed = k.windowed;
        *window = k.windowed ? k.window : 0;
    }
    return done(st);
}
int orc_cache_append(void* c, size_t layer, const float* k, size_t klen, const float* v, size_t vlen,
                     size_t position) {
    return done(static_cast<KvCache*>(c)->append(layer, k, klen, v, vlen, position));
}
// Append `rows` consecutive positions of one layer, `[rows][Hkv*D]` each.
int orc_cache_append_rows(void* c, size_t layer, const float* k, const float* v, size_t rows, size_t start) {
    KvCache* cache = static_cast<KvCache*>(c);
    const size_t row = cache->row_len();
    for (size_t r = 0; r < rows; ++r) {
        Status st = cache->append(layer, k + r * row, row, v + r * row, row, start + r);
        if (!st.ok()) return done(st);
    }
    return done({});
}
int orc_cache_restore_bulk(void* c, size_t layer, size_t first_position, const float* keys, size_t klen,
                           const float* values, size_t vlen) {
    return done(static_cast<KvCache*>(c)->restore_bulk(layer, first_position, keys, klen, values, vlen));
}
int orc_cache_stored_len(void* c, size_t layer, size_t* out) {
    return done(static_cast<KvCache*>(c)->stored_len(layer, out));
}
int orc_cache_next_position(void* c, size_t layer, size_t* out) {
    return done(static_cast<KvCache*>(c)->next_position(layer, out));
}
// View accessors; a negative return is Option::None.
int64_t orc_view_len(void* c, size_t layer) {
    KvCache* cache = static_cast<KvCache*>(c);
    if (layer >= cache->layer_count()) return -1;
    return static_cast<int64_t>(cache->view_len(layer));
}
int64_t orc_view_position_at(void* c, size_t layer, size_t vi) {
    KvCache* cache = static_cast<KvCache*>(c);
    if (layer >= cache->layer_count()) return -1;
    auto p = cache->position_at(layer, vi);
    return p ? static_cast<int64_t>(*p) : -1;
}
int64_t orc_view_window(void* c, size_t layer) {
    auto w = static_cast<KvCache*>(c)->window(layer);
    return w ? static_cast<int64_t>(*w) : -1;
}
// Copies head_dim floats; returns 0 when the index or head is out of range.
int orc_view_key(void* c, size_t layer, size_t vi, size_t head, float* out) {
    KvCache* cache = static_cast<KvCache*>(c);
    const float* p = cache->key(layer, vi, head);
    if (!p) return 0;
    std::memcpy(out, p, cache->head_dim() * sizeof(float));
    return 1;
}
int orc_view_value(void* c, size_t layer, size_t vi, size_t head, float* out) {
    KvCache* cache = static_cast<KvCache*>(c);
    const float* p = cache->value(layer, vi, head);
    if (!p) return 0;
    std::memcpy(out, p, cache->head_dim() * sizeof(float));
    return 1;
}
// The whole view of one layer in position order: keys and values as
// `[visible][Hkv][D]`. Returns the visible count.
size_t orc_view_dump(void* c, size_t layer, float* keys, float* values) {
    KvCache* cache = static_cast<KvCache*>(c);
    const size_t n = cache->view_len(layer), h = cache->num_kv_heads(), d = cache->head_dim();
    for (size_t vi = 0; vi < n; ++vi)
        for (size_t head = 0; head < h; ++head) {
            std::memcpy(keys + (vi * h + head) * d, cache->key(layer, vi, head), d * sizeof(float));
            std::memcpy(values + (vi * h + head) * d, cache->value(layer, vi, head), d * sizeof(float));
        }
    return n;
}
void orc_cache_stats(void* c, uint64_t* appended, uint64_t* stored) {
    auto s = static_cast<KvCache*>(c)->stats();
    for (size_t i = 0; i < s.size(); ++i) {
        appended[i] = s[i].appended;
        stored[i] = s[i].stored;
    }
}
int orc_cache_checkpoint_active(void* c) { return static_cast<KvCache*>(c)->checkpoint_active(); }
// `bases` receives one entry per layer.
int orc_cache_checkpoint(void* c, size_t max_round_tokens, orc_checkpoint_t* out, uint64_t* bases) {
    Checkpoint cp;
    Status st = static_cast<KvCache*>(c)->checkpoint(max_round_tokens, &cp);
    if (st.ok()) {
        *out = orc_checkpoint_t{cp.cache_id, cp.serial, cp.max_round_tokens, cp.saved_bytes};
        if (bases)
            for (size_t i = 0; i < cp.bases.size(); ++i) bases[i] = cp.bases[i];
    }
    return done(st);
}
static Checkpoint handle_of(const orc_checkpoint_t* h) {
    Checkpoint cp;
    cp.cache_id = h->cache_id;
    cp.serial = h->serial;
    cp.max_round_tokens = h->max_round_tokens;
    cp.saved_bytes = h->saved_bytes;
    return cp;
}
int orc_cache_rewind(void* c, const orc_checkpoint_t* h, size_t target) {
    return done(static_cast<KvCache*>(c)->rewind_to(handle_of(h), target));
}
int orc_cache_release(void* c, const orc_checkpoint_t* h) {
    return done(static_cast<KvCache*>(c)->release(handle_of(h)));
}

// ---- attention ---------------------------------------------------------------
int orc_gqa_attention(void* c, size_t layer, const float* q, size_t q_len, size_t num_queries, size_t num_q_heads,
                      const uint64_t* positions, size_t num_positions, int has_scale, float scale, float* out) {
    std::vector<size_t> pos(positions, positions + num_positions);
    std::vector<float> o;
    Status st = gqa_attention(q, q_len, num_queries, num_q_heads, pos.data(), pos.size(),
                              *static_cast<KvCache*>(c), layer,
                              has_scale ? std::optional<float>(scale) : std::nullopt, &o);
    if (st.ok() && !o.empty()) std::memcpy(out, o.data(), o.size() * sizeof(float));
    return done(st);
}

// Run one single-query attention per unit, `threads` host threads pulling
// units from a shared counter. Unit u reads cache caches[u], layer layers[u],
// query q + u * q_stride at position positions[u]; its `[Hq][D]` output goes
// to out + u * q_stride. Returns the wall time in seconds through *seconds.
// This is the reference's scalar routine, unchanged, spread over cores the way
// its engine spreads sequences over worker threads.
int orc_attention_units(size_t n_units, void* const* caches, const uint64_t* layers, const float* q,
                        size_t q_stride, const uint64_t* positions, size_t num_q_heads, size_t threads,
                        float* out, double* seconds) {
    std::atomic<size_t> next{0};
    std::atomic<int> failed{0};
    std::vector<std::string> msgs(threads);
    auto work = [&](size_t t) {
        std::vector<float> o;
        for (;;) {
            const size_t u = next.fetch_add(1);
            if (u >= n_units) return;
            const size_t p = positions[u];
            Status st = gqa_attention(q + u * q_stride, q_stride, 1, num_q_heads, &p, 1,
                                      *static_cast<KvCache*>(caches[u]), layers[u], std::nullopt, &o);
            if (!st.ok()) {
                failed.store(st.code);
                msgs[t] = st.msg;
                return;
            }
            std::memcpy(out + u * q_stride, o.data(), q_stride * sizeof(float));
        }
    };
    const auto t0 = std::chrono::steady_clock::now();
    if (threads <= 1) {
        work(0);
    } else {
        std::vector<std::thread> pool;
        for (size_t t = 0; t < threads; ++t) pool.emplace_back(work, t);
        for (auto& th : pool) th.join();
    }
    const auto t1 = std::chrono::steady_clock::now();
    if (seconds) *seconds = std::chrono::duration<double>(t1 - t0).count();
    if (failed.load()) {
        for (auto& m : msgs)
            if (!m.empty()) g_last_error = m;
        return failed.load();
    }
    return done({});
}

// ---- the reference fixtures' generator ----------------------------------------
// f32 in [-0.5, 0.5): state = max(seed, 1); per value state = state * A + C
// (wrapping u64), value = ((state >> 40) as f32) / 2^24 - 0.5
// (crates/wgpu-compute/tests/fused_kernels.rs:45-55,
//  crates/itak-kv/tests/restore_fixture.rs:22-30).
void orc_lcg(uint64_t seed, size_t count, float* out) {
    uint64_t state = seed < 1 ? 1 : seed;
    for (size_t i = 0; i < count; ++i) {
        state = state * 6364136223846793005ull + 1442695040888963407ull;
        out[i] = static_cast<float>(static_cast<uint32_t>(state >> 40)) / static_cast<float>(1u << 24) - 0.5f;
    }
}

// ---- hashes ----------------------------------------------------------------
uint64_t orc_checksum(const uint8_t* bytes, size_t n) { return checksum(bytes, n); }
uint64_t orc_prefix_hash(const uint32_t* tokens, size_t n) { return prefix_hash(tokens, n); }
uint64_t orc_prefix_discriminator(const uint32_t* tokens, size_t n) { return prefix_discriminator(tokens, n); }

// ---- snapshots ---------------------------------------------------------------
int orc_snapshot_capture(void* cache, const char* fingerprint, void** out) {
    auto s = std::make_unique<KvSnapshot>();
    Status st = KvSnapshot::capture(*static_cast<KvCache*>(cache), fingerprint, s.get());
    if (st.ok()) *out = s.release();
    return done(st);
}
// Build a snapshot value directly (the reference's fields are public): layer
// blocks are filled afterwards with orc_snapshot_set_layer.
void* orc_snapshot_new(const int32_t* windowed, const uint64_t* windows, size_t n_layers, size_t num_kv_heads,
                       size_t head_dim, const char* fingerprint, size_t token_count, size_t n_blocks) {
    auto* s = new KvSnapshot();
    s->geometry.layers = pattern_of(windowed, windows, n_layers);
    s->geometry.num_kv_heads = num_kv_heads;
    s->geometry.head_dim = head_dim;
    s->model_fingerprint = fingerprint;
    s->token_count = token_count;
    s->layers.resize(n_blocks);
    return s;
}
void orc_snapshot_set_layer(void* snap, size_t layer, size_t first_position, const float* keys, size_t klen,
                            const float* values, size_t vlen) {
    auto* s = static_cast<KvSnapshot*>(snap);
    s->layers[layer].first_position = first_position;
    s->layers[layer].keys.assign(keys, keys + klen);
    s->layers[layer].values.assign(values, values + vlen);
}
void orc_snapshot_free(void* s) { delete static_cast<KvSnapshot*>(s); }
int orc_snapshot_validate(void* s) { return done(static_cast<KvSnapshot*>(s)->validate()); }
size_t orc_snapshot_token_count(void* s) { return static_cast<KvSnapshot*>(s)->token_count; }
size_t orc_snapshot_layer_count(void* s) { return static_cast<KvSnapshot*>(s)->layers.size(); }
size_t orc_snapshot_layer_first(void* s, size_t layer) { return static_cast<KvSnapshot*>(s)->layers[layer].first_position; }
size_t orc_snapshot_layer_floats(void* s, size_t layer) { return static_cast<KvSnapshot*>(s)->layers[layer].keys.size(); }
void orc_snapshot_layer_copy(void* s, size_t layer, float* keys, float* values) {
    auto& l = static_cast<KvSnapshot*>(s)->layers[layer];
    if (!l.keys.empty()) std::memcpy(keys, l.keys.data(), l.keys.size() * sizeof(float));
    if (!l.values.empty()) std::memcpy(values, l.values.data(), l.values.size() * sizeof(float));
}
int orc_snapshot_equal(void* a, void* b) {
    auto* x = static_cast<KvSnapshot*>(a);
    auto* y = static_cast<KvSnapshot*>(b);
    if (!(x->geometry == y->geometry) || x->model_fingerprint != y->model_fingerprint ||
        x->token_count != y->token_count || x->layers.size() != y->layers.size())
        return 0;
    for (size_t i = 0; i < x->layers.size(); ++i) {
        const auto &l = x->layers[i], &r = y->layers[i];
        if (l.first_position != r.first_position || l.keys.size() != r.keys.size() || l.values.size() != r.values.size())
            return 0;
        if (std::memcmp(l.keys.data(), r.keys.data(), l.keys.size() * 4) != 0) return 0;
        if (std::memcmp(l.values.data(), r.values.data(), l.values.size() * 4) != 0) return 0;
    }
    return 1;
}
int orc_snapshot_restore(void* s, void** cache_out) {
    std::unique_ptr<KvCache> c;
    Status st = static_cast<KvSnapshot*>(s)->restore(&c);
    if (st.ok()) *cache_out = c.release();
    return done(st);
}
int orc_snapshot_restore_checked(void* s, const int32_t* windowed, const uint64_t* windows, size_t n_layers,
                                 size_t num_kv_heads, size_t head_dim, const char* fingerprint, void** cache_out) {
    KvGeometry g;
    g.layers = pattern_of(windowed, windows, n_layers);
    g.num_kv_heads = num_kv_heads;
    g.head_dim = head_dim;
    std::unique_ptr<KvCache> c;
    Status st = static_cast<KvSnapshot*>(s)->restore_checked(g, fingerprint, &c);
    if (st.ok()) *cache_out = c.release();
    return done(st);
}
// Two-call protocol: pass out = NULL to learn the size.
int orc_snapshot_to_bytes(void* s, uint8_t* out, size_t cap, size_t* size) {
    std::vector<uint8_t> b;
    Status st = static_cast<KvSnapshot*>(s)->to_bytes(&b);
    if (st.ok()) {
        *size = b.size();
        if (out && cap >= b.size()) std::memcpy(out, b.data(), b.size());
    }
    return done(st);
}
int orc_snapshot_from_bytes(const uint8_t* bytes, size_t n, void** out) {
    auto s = std::make_unique<KvSnapshot>();
    Status st = KvSnapshot::from_bytes(bytes, n, s.get());
    if (st.ok()) *out = s.release();
    return done(st);
}
uint64_t orc_geometry_bytes_per_token(const int32_t* windowed, const uint64_t* windows, size_t n_layers,
                                      size_t num_kv_heads, size_t head_dim) {
    KvGeometry g;
    g.layers = pattern_of(windowed, windows, n_layers);
    g.num_kv_heads = num_kv_heads;
    g.head_dim = head_dim;
    return g.bytes_per_token();
}
uint64_t orc_geometry_stored_bytes_for(const int32_t* windowed, const uint64_t* windows, size_t n_layers,
                                       size_t num_kv_heads, size_t head_dim, size_t tokens) {
    KvGeometry g;
    g.layers = pattern_of(windowed, windows, n_layers);
    g.num_kv_heads = num_kv_heads;
    g.head_dim = head_dim;
    return g.stored_bytes_for(tokens);
}

// ---- slot/ring laws ----------------------------------------------------------
void orc_prefix_visible_range(int sliding, size_t window, size_t position, size_t* first, size_t* rows) {
    auto r = prefix_visible_range(sliding != 0, window, position);
    *first = r.first;
    *rows = r.second;
}
// Writes up to `cap` runs as (row, slot, count) triples; returns the run count.
size_t orc_prefix_slot_runs(int sliding, size_t first_position, size_t rows, size_t ring, uint64_t* triples,
                            size_t cap) {
    auto runs = prefix_slot_runs(sliding != 0, first_position, rows, ring);
    for (size_t i = 0; i < runs.size() && i < cap; ++i) {
        triples[3 * i] = runs[i].row;
        triples[3 * i + 1] = runs[i].slot;
        triples[3 * i + 2] = runs[i].count;
    }
    return runs.size();
}

// ---- the CPU backend step ------------------------------------------------------
struct orc_backend_config_t {
    const int32_t* sliding;  // per layer
    uint64_t n_layers;
    uint64_t q_heads, kv_heads, key_length, value_length, sliding_window;
    float rope_freq_base_swa;
};
static BackendConfig config_of(const orc_backend_config_t* c) {
    BackendConfig b;
    for (uint64_t i = 0; i < c->n_layers; ++i) b.sliding.push_back(c->sliding[i] != 0);
    b.q_heads = c->q_heads;
    b.kv_heads = c->kv_heads;
    b.key_length = c->key_length;
    b.value_length = c->value_length;
    b.sliding_window = c->sliding_window;
    b.rope_freq_base_swa = c->rope_freq_base_swa;
    return b;
}
void* orc_backend_new() { return new CpuBackend(); }
void orc_backend_free(void* b) { delete static_cast<CpuBackend*>(b); }
void orc_backend_reset(void* b) { static_cast<CpuBackend*>(b)->reset(); }
void* orc_backend_cache(void* b) { return static_cast<CpuBackend*>(b)->cache(); }
// `position` is the caller's sequence position (Cache::position()); `out`
// receives `[rows][q_heads * key_length]`.
int orc_backend_attention(void* b, const orc_backend_config_t* cfg, size_t layer, int request_sliding,
                          const float* q, size_t q_len, const float* k, size_t k_len, const float* v, size_t v_len,
                          size_t position, float* out) {
    PositionCache pos{position};
    std::vector<float> o;
    Status st = static_cast<CpuBackend*>(b)->attention(config_of(cfg), layer, request_sliding != 0, q, q_len, k, k_len,
                                                        v, v_len, pos, &o);
    if (st.ok() && !o.empty()) std::memcpy(out, o.data(), o.size() * sizeof(float));
    return done(st);
}
int orc_backend_checkpoint(void* b, size_t max_round_tokens, orc_checkpoint_t* out, uint64_t* bases) {
    Checkpoint cp;
    Status st = static_cast<CpuBackend*>(b)->cache_checkpoint(max_round_tokens, &cp);
    if (st.ok()) {
        *out = orc_checkpoint_t{cp.cache_id, cp.serial, cp.max_round_tokens, cp.saved_bytes};
        if (bases)
            for (size_t i = 0; i < cp.bases.size(); ++i) bases[i] = cp.bases[i];
    }
    return done(st);
}
int orc_backend_rewind(void* b, const orc_checkpoint_t* h, size_t target) {
    return done(static_cast<CpuBackend*>(b)->cache_rewind(handle_of(h), target));
}
int orc_backend_release(void* b, const orc_checkpoint_t* h) {
    return done(static_cast<CpuBackend*>(b)->cache_release(handle_of(h)));
}

}  // extern "C"
