// CPU oracle for the KV-cache hot path. TEST INFRASTRUCTURE ONLY.
//
// This header restates, in plain C++17, the algorithm of the reference's CPU
// crates for the path "append RoPE'd K/V rows -> GQA attention over the cache
// -> prefix snapshot/restore -> checkpoint/rewind of speculative tokens".
// It exists so the CUDA path can be checked against it; it is never linked
// into, imported by or executed from the shipped library. Only the tests, the
// smoke check and the bench's cpu-baseline/reference legs may use it.
//
// Parity pin: the reference is Rust and cannot be compiled in this build
// environment, so the restatement is pinned against every known-answer test
// the reference holds for this path (tests/test_oracle_*.py list them with
// their file:line).
//
// Each function cites the reference file:line whose behaviour it follows
// (paths are relative to the reference repository root).
#pragma once

#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <memory>
#include <optional>
#include <string>
#include <vector>

namespace orc {

// ---------------------------------------------------------------------------
// Refusal codes. One per variant of the reference's error enums:
//   crates/attention/src/error.rs:9-127      (AttentionError)
//   crates/itak-kv/src/error.rs              (KvError, snapshot subset)
//   crates/cpu-compute/src/cpu.rs:28-33      (StepFailed{step, detail})
// The numeric values are shared with the product's C-ABI by convention; a
// test asserts that the two tables agree.
// ---------------------------------------------------------------------------
enum Code : int {
    kOk = 0,
    kZeroDimension = 1,
    kInvalidWindow = 2,
    kSizeOverflow = 3,
    kShapeMismatch = 4,
    kInvalidLayer = 5,
    kOutOfOrderPosition = 6,
    kNonDivisibleHeads = 7,
    kNoVisibleKeys = 8,
    kCheckpointBusy = 9,
    kStaleCheckpoint = 10,
    kCheckpointTooDeep = 11,
    kCheckpointRangeExceeded = 12,
    kBulkRestoreNotFresh = 13,
    kRewindOutOfRange = 14,
    kIncoherentCache = 32,
    kInconsistentSnapshot = 33,
    kBadMagic = 34,
    kUnsupportedVersion = 35,
    kTruncated = 36,
    kChecksumMismatch = 37,
    kGeometryMismatch = 38,
    kFingerprintMismatch = 39,
    kStepFailed = 64,
};

struct Status {
    int code = kOk;
    std::string msg;
    bool ok() const { return code == kOk; }
    static Status fail(int c, std::string m) { return Status{c, std::move(m)}; }
};

inline std::string zu(size_t v) { return std::to_string(v); }

// Checked multiply standing in for Rust's usize::checked_mul.
inline bool mul_overflows(size_t a, size_t b, size_t* out) {
    return __builtin_mul_overflow(a, b, out);
}

// ---------------------------------------------------------------------------
// f32 <-> f16 bit conversions.
// ---------------------------------------------------------------------------

// Round-to-nearest-even f32 -> f16 bits.
// Follows crates/wgpu-compute/src/kernels/k1_q4k_gemv.rs:285-329:
// inf keeps its class, every NaN becomes sign|0x7e00, exponent >= 31 after
// rebias overflows to inf, results below half the smallest subnormal flush to
// a signed zero, subnormal and normal results round to nearest even with the
// mantissa carry propagating into the exponent.
inline uint16_t f32_to_f16_bits(float x) {
    uint32_t bits;
    std::memcpy(&bits, &x, 4);
    const uint16_t sign = static_cast<uint16_t>((bits >> 16) & 0x8000u);
    const int exp = static_cast<int>((bits >> 23) & 0xffu);
    const uint32_t frac = bits & 0x7fffffu;
    if (exp == 0xff) return sign | (frac == 0 ? 0x7c00 : 0x7e00);
    int e = exp - 112;
    if (e >= 0x1f) return sign | 0x7c00;
    if (e <= 0) {
        if (e < -10) return sign;
        const uint32_t m = frac | 0x800000u;
        const uint32_t shift = static_cast<uint32_t>(14 - e);
        const uint32_t rem = m & ((1u << shift) - 1u);
        const uint32_t halfway = 1u << (shift - 1);
        uint32_t out = m >> shift;
        if (rem > halfway || (rem == halfway && (out & 1u))) out += 1;
        return sign | static_cast<uint16_t>(out);
    }
    uint32_t kept = frac >> 13;
    const uint32_t rem = frac & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (kept & 1u))) {
        kept += 1;
        if (kept == 0x400u) {
            kept = 0;
            e += 1;
            if (e >= 0x1f) return sign | 0x7c00;
        }
    }
    return sign | static_cast<uint16_t>(e << 10) | static_cast<uint16_t>(kept);
}

// Exact f16 bits -> f32. Follows crates/gguf/src/dequant.rs:12-34
// (subnormals are frac * 2^-24, NaN payload shifted into the f32 mantissa).
inline float f16_bits_to_f32(uint16_t h) {
    const uint32_t sign = static_cast<uint32_t>(h >> 15);
    const uint32_t exp = (h >> 10) & 0x1fu;
    const uint32_t frac = h & 0x3ffu;
    uint32_t out;
    if (exp == 0x1f) {
        out = (sign << 31) | (frac == 0 ? 0x7f800000u : (0x7fc00000u | (frac << 13)));
    } else if (exp == 0) {
        if (frac == 0) {
            out = sign << 31;
        } else {
            uint32_t scale_bits = 0x33800000u;  // 2^-24
            float scale;
            std::memcpy(&scale, &scale_bits, 4);
            float v = static_cast<float>(frac) * scale;
            return sign ? -v : v;
        }
    } else {
        out = (sign << 31) | ((exp + 127 - 15) << 23) | (frac << 13);
    }
    float f;
    std::memcpy(&f, &out, 4);
    return f;
}

// The value an f16 cache holds for an f32 input: the definition of the f16
// oracle (the reference states its f16 forms differ from f32 "only in the
// stored values", crates/wgpu-compute/src/kernels/k6_attention.rs:631-641).
inline float round_through_f16(float x) { return f16_bits_to_f32(f32_to_f16_bits(x)); }

// ---------------------------------------------------------------------------
// RoPE, both pairings, angles in f64.
// ---------------------------------------------------------------------------

// Adjacent-pair (llama "NORM") rotation of one head vector.
// Follows crates/torch-math/src/rope_interleaved.rs:65-117: pair i joins
// channels (2i, 2i+1), angle = position * base^(-2i/rotary_dim) computed in
// f64, products formed in f64 and cast to f32; channels past rotary_dim copy.
inline Status rope_interleaved_partial(const float* in, size_t len, size_t position, float base,
                                       size_t head_dim, size_t rotary_dim, float* out) {
    if (head_dim < 2 || head_dim % 2 != 0)
        return Status::fail(kStepFailed, "rope_interleaved: head_dim must be even and >= 2");
    if (len != head_dim)
        return Status::fail(kShapeMismatch, "rope_interleaved: got " + zu(len) + ", expected " + zu(head_dim));
    if (rotary_dim < 2 || rotary_dim % 2 != 0 || rotary_dim > head_dim)
        return Status::fail(kStepFailed, "rope_interleaved: rotary_dim must be even, >= 2, and <= head_dim");
    if (!std::isfinite(base) || base <= 1.0f)
        return Status::fail(kStepFailed, "rope_interleaved: base must be finite and > 1");
    for (size_t i = 0; i < head_dim; ++i) out[i] = in[i];
    const double pos = static_cast<double>(position);
    const double b = static_cast<double>(base);
    for (size_t i = 0; i < rotary_dim / 2; ++i) {
        const double exponent = -static_cast<double>(2 * i) / static_cast<double>(rotary_dim);
        const double angle = pos * std::pow(b, exponent);
        const double s = std::sin(angle), c = std::cos(angle);
        const double x = in[2 * i], y = in[2 * i + 1];
        out[2 * i] = static_cast<float>(x * c - y * s);
        out[2 * i + 1] = static_cast<float>(x * s + y * c);
    }
    return {};
}

// RMSNorm with a weight vector. Follows crates/torch-math/src/norm.rs:21-53: the mean of squares is summed
// in f64 in element order, inv_rms = 1 / sqrt(mean + eps) in f64, and each output is
// (f64(v) * inv_rms * f64(w)) rounded once to f32.  Refusals in the reference's order: empty input, weight
// length, eps not finite and > 0.
inline Status rms_norm(const float* in, size_t len, const float* weight, size_t weight_len, float eps, float* out) {
    if (len == 0) return Status::fail(kStepFailed, "rms_norm: input is empty");
    if (weight_len != len)
        return Status::fail(kShapeMismatch, "rms_norm: got " + zu(weight_len) + ", expected " + zu(len));
    if (!std::isfinite(eps) || eps <= 0.0f) return Status::fail(kStepFailed, "rms_norm: eps must be finite and > 0");
    double sum = 0.0;
    for (size_t i = 0; i < len; ++i) sum += static_cast<double>(in[i]) * static_cast<double>(in[i]);
    const double mean_sq = sum / static_cast<double>(len);
    const double inv_rms = 1.0 / std::sqrt(mean_sq + static_cast<double>(eps));
    for (size_t i = 0; i < len; ++i)
        out[i] = static_cast<float>(static_cast<double>(in[i]) * inv_rms * static_cast<double>(weight[i]));
    return {};
}

// Half-split (NeoX) rotation. Follows crates/torch-math/src/rope.rs:63-117:
// pair i joins channel i with channel i + rotary_dim/2, same f64 angle law.
inline Status rope_half_partial(const float* in, size_t len, size_t position, float base,
                                size_t head_dim, size_t rotary_dim, float* out) {
    if (head_dim < 2 || head_dim % 2 != 0)
        return Status::fail(kStepFailed, "rope: head_dim must be even and >= 2");
    if (len != head_dim)
        return Status::fail(kShapeMismatch, "rope: got " + zu(len) + ", expected " + zu(head_dim));
    if (rotary_dim < 2 || rotary_dim % 2 != 0 || rotary_dim > head_dim)
        return Status::fail(kStepFailed, "rope: rotary_dim must be even, >= 2, and <= head_dim");
    if (!std::isfinite(base) || base <= 1.0f)
        return Status::fail(kStepFailed, "rope: base must be finite and > 1");
    for (size_t i = 0; i < head_dim; ++i) out[i] = in[i];
    const double pos = static_cast<double>(position);
    const double b = static_cast<double>(base);
    const size_t half = rotary_dim / 2;
    for (size_t i = 0; i < half; ++i) {
        const double exponent = -static_cast<double>(2 * i) / static_cast<double>(rotary_dim);
        const double angle = pos * std::pow(b, exponent);
        const double s = std::sin(angle), c = std::cos(angle);
        const double x = in[i], y = in[i + half];
        out[i] = static_cast<float>(x * c - y * s);
        out[i + half] = static_cast<float>(x * s + y * c);
    }
    return {};
}

// ---------------------------------------------------------------------------
// KV cache: crates/attention/src/cache.rs (whole file).
// ---------------------------------------------------------------------------

struct LayerKind {
    bool windowed = false;
    size_t window = 0;  // meaningful when windowed
    bool operator==(const LayerKind& o) const {
        return windowed == o.windowed && (!windowed || window == o.window);
    }
    bool operator!=(const LayerKind& o) const { return !(*this == o); }
};

// The 52-layer pattern with a global layer at every index i % 4 == 3 and
// window-2048 ring layers elsewhere (crates/attention/src/cache.rs:68-84).
inline std::vector<LayerKind> glimmer_layer_pattern() {
    std::vector<LayerKind> p;
    for (int i = 0; i < 52; ++i) p.push_back(i % 4 == 3 ? LayerKind{false, 0} : LayerKind{true, 2048});
    return p;
}

constexpr int64_t kNoPosition = -1;  // Option<usize>::None for ring slots

// Receipt for an outstanding checkpoint (crates/attention/src/cache.rs:229-273).
struct Checkpoint {
    uint64_t cache_id = 0;
    uint64_t serial = 0;
    std::vector<size_t> bases;
    size_t max_round_tokens = 0;
    size_t saved_bytes = 0;
};

struct LayerStats {
    size_t layer;
    LayerKind kind;
    size_t appended;
    size_t stored;
};

class KvCache {
  public:
    // crates/attention/src/cache.rs:327-371 with LayerCache::new at :125-151.
    // Refusal order: empty pattern, zero kv heads, zero head dim, any zero
    // window, then per layer the row product and the ring size overflow.
    static Status create(const std::vector<LayerKind>& pattern, size_t num_kv_heads, size_t head_dim,
                         std::unique_ptr<KvCache>* out) {
        if (pattern.empty()) return Status::fail(kZeroDimension, "layer pattern must be positive, got 0");
        if (num_kv_heads == 0) return Status::fail(kZeroDimension, "num_kv_heads must be positive, got 0");
        if (head_dim == 0) return Status::fail(kZeroDimension, "head_dim must be positive, got 0");
        for (const auto& k : pattern)
            if (k.windowed && k.window == 0)
                return Status::fail(kInvalidWindow, "sliding window must be positive, got 0");
        std::unique_ptr<KvCache> c(new KvCache());
        c->hkv_ = num_kv_heads;
        c->d_ = head_dim;
        for (const auto& k : pattern) {
            size_t row;
            if (mul_overflows(num_kv_heads, head_dim, &row))
                return Status::fail(kSizeOverflow, "kv row length: element count overflows usize");
            Layer l;
            l.kind = k;
            if (k.windowed) {
                size_t slots;
                if (mul_overflows(k.window, row, &slots) || slots > (std::numeric_limits<size_t>::max() / 8))
                    return Status::fail(kSizeOverflow, "windowed layer storage: element count overflows usize");
                l.keys.assign(slots, 0.0f);
                l.values.assign(slots, 0.0f);
                l.slot_position.assign(k.window, kNoPosition);
            }
            c->layers_.push_back(std::move(l));
        }
        c->id_ = next_cache_id()++;
        *out = std::move(c);
        return {};
    }

    size_t layer_count() const { return layers_.size(); }
    size_t num_kv_heads() const { return hkv_; }
    size_t head_dim() const { return d_; }
    size_t row_len() const { return hkv_ * d_; }
    uint64_t id() const { return id_; }

    Status layer_kind(size_t layer, LayerKind* out) const {
        if (auto s = check_layer(layer); !s.ok()) return s;
        *out = layers_[layer].kind;
        return {};
    }
    // crates/attention/src/cache.rs:407-415
    Status stored_len(size_t layer, size_t* out) const {
        if (auto s = check_layer(layer); !s.ok()) return s;
        *out = stored(layers_[layer]);
        return {};
    }
    Status next_position(size_t layer, size_t* out) const {
        if (auto s = check_layer(layer); !s.ok()) return s;
        *out = layers_[layer].appended;
        return {};
    }

    // crates/attention/src/cache.rs:423-474 (+ LayerCache::write :181-203).
    // Check order: k length, v length, live-checkpoint range (only when the
    // layer index is in range), layer index, then position == appended.
    Status append(size_t layer, const float* k, size_t klen, const float* v, size_t vlen, size_t position) {
        const size_t row = row_len();
        if (klen != row) return shape("k", row, klen);
        if (vlen != row) return shape("v", row, vlen);
        if (live_ && layer < live_->bases.size()) {
            const size_t limit = live_->bases[layer] + live_->max_round_tokens;
            if (position >= limit)
                return Status::fail(kCheckpointRangeExceeded,
                                    "layer " + zu(layer) + " append at position " + zu(position) +
                                        " is outside the live checkpoint's saved range (first unsaved position " +
                                        zu(limit) + "); refusing so a later rewind cannot meet a slot it cannot restore");
        }
        if (auto s = check_layer(layer); !s.ok()) return s;
        Layer& l = layers_[layer];
        if (position != l.appended)
            return Status::fail(kOutOfOrderPosition, "layer " + zu(layer) + " appends must be in order: expected position " +
                                                         zu(l.appended) + ", got " + zu(position));
        if (!l.kind.windowed) {
            l.keys.insert(l.keys.end(), k, k + row);
            l.values.insert(l.values.end(), v, v + row);
        } else {
            const size_t slot = position % l.kind.window;
            std::memcpy(&l.keys[slot * row], k, row * sizeof(float));
            std::memcpy(&l.values[slot * row], v, row * sizeof(float));
            l.slot_position[slot] = static_cast<int64_t>(position);
        }
        l.appended += 1;
        return {};
    }

    // crates/attention/src/cache.rs:513-577. Installs a snapshot layer's rows
    // for positions first_position.. directly into their slots on a fresh
    // layer; the resulting state equals an append replay.
    Status restore_bulk(size_t layer, size_t first_position, const float* keys, size_t klen, const float* values,
                        size_t vlen) {
        const size_t row = row_len();
        if (klen != vlen || klen % row != 0) return shape("bulk restore rows", vlen, klen);
        const size_t rows = klen / row;
        if (auto s = check_layer(layer); !s.ok()) return s;
        Layer& l = layers_[layer];
        if (l.appended != 0)
            return Status::fail(kBulkRestoreNotFresh, "layer " + zu(layer) + " already holds " + zu(l.appended) +
                                                          " appended positions; bulk restore installs into a fresh layer only");
        if (!l.kind.windowed) {
            if (first_position != 0) return shape("bulk restore first position (global layer)", 0, first_position);
            l.keys.insert(l.keys.end(), keys, keys + klen);
            l.values.insert(l.values.end(), values, values + vlen);
        } else {
            if (rows > l.kind.window) return shape("bulk restore rows (windowed layer)", l.kind.window, rows);
            for (size_t r = 0; r < rows; ++r) {
                const size_t position = first_position + r;
                const size_t slot = position % l.kind.window;
                std::memcpy(&l.keys[slot * row], keys + r * row, row * sizeof(float));
                std::memcpy(&l.values[slot * row], values + r * row, row * sizeof(float));
                l.slot_position[slot] = static_cast<int64_t>(position);
            }
        }
        l.appended = first_position + rows;
        return {};
    }

    // --- the read view (crates/attention/src/cache.rs:581-585, 836-904) ---
    // Visible index i is the i-th oldest stored position; it names absolute
    // position appended - stored + i.
    size_t view_len(size_t layer) const { return stored(layers_[layer]); }
    std::optional<size_t> position_at(size_t layer, size_t visible_index) const {
        const Layer& l = layers_[layer];
        if (visible_index >= stored(l)) return std::nullopt;
        return l.appended - stored(l) + visible_index;
    }
    const float* key(size_t layer, size_t visible_index, size_t kv_head) const {
        auto p = position_at(layer, visible_index);
        if (!p || kv_head >= hkv_) return nullptr;
        const Layer& l = layers_[layer];
        return &l.keys[(slot_of(l, *p) * hkv_ + kv_head) * d_];
    }
    const float* value(size_t layer, size_t visible_index, size_t kv_head) const {
        auto p = position_at(layer, visible_index);
        if (!p || kv_head >= hkv_) return nullptr;
        const Layer& l = layers_[layer];
        return &l.values[(slot_of(l, *p) * hkv_ + kv_head) * d_];
    }
    std::optional<size_t> window(size_t layer) const {
        const Layer& l = layers_[layer];
        if (l.kind.windowed) return l.kind.window;
        return std::nullopt;
    }

    // crates/attention/src/cache.rs:588-599
    std::vector<LayerStats> stats() const {
        std::vector<LayerStats> out;
        for (size_t i = 0; i < layers_.size(); ++i)
            out.push_back(LayerStats{i, layers_[i].kind, layers_[i].appended, stored(layers_[i])});
        return out;
    }

    bool checkpoint_active() const { return live_.has_value(); }

    // crates/attention/src/cache.rs:634-717. One live checkpoint at a time;
    // the round bound may not exceed the smallest window; the serial advances
    // only after validation; each ring layer saves the max_round_tokens slots
    // starting at appended % window (K row, V row, slot position).
    Status checkpoint(size_t max_round_tokens, Checkpoint* out) {
        if (live_) return Status::fail(kCheckpointBusy,
                                       "a checkpoint is already outstanding on this cache; release it before taking another");
        if (max_round_tokens == 0) return Status::fail(kZeroDimension, "max_round_tokens must be positive, got 0");
        std::optional<size_t> smallest;
        for (const auto& l : layers_)
            if (l.kind.windowed && (!smallest || l.kind.window < *smallest)) smallest = l.kind.window;
        if (smallest && max_round_tokens > *smallest)
            return Status::fail(kCheckpointTooDeep,
                                "checkpoint round bound " + zu(max_round_tokens) + " exceeds the smallest sliding window " +
                                    zu(*smallest) +
                                    ": a round that long would overwrite a ring slot twice and no rewind could be exact");
        next_serial_ += 1;
        Live data;
        data.serial = next_serial_;
        data.max_round_tokens = max_round_tokens;
        const size_t row = row_len();
        size_t saved_bytes = 0;
        for (const auto& l : layers_) {
            data.bases.push_back(l.appended);
            std::vector<Saved> saved;
            if (l.kind.windowed) {
                for (size_t i = 0; i < max_round_tokens; ++i) {
                    Saved s;
                    s.slot = (l.appended + i) % l.kind.window;
                    s.position = l.slot_position[s.slot];
                    s.keys.assign(l.keys.begin() + s.slot * row, l.keys.begin() + (s.slot + 1) * row);
                    s.values.assign(l.values.begin() + s.slot * row, l.values.begin() + (s.slot + 1) * row);
                    saved_bytes += (s.keys.size() + s.values.size()) * 4;
                    saved.push_back(std::move(s));
                }
            }
            data.saved.push_back(std::move(saved));
        }
        out->cache_id = id_;
        out->serial = data.serial;
        out->bases = data.bases;
        out->max_round_tokens = max_round_tokens;
        out->saved_bytes = saved_bytes;
        live_ = std::move(data);
        return {};
    }

    // crates/attention/src/cache.rs:758-818. Validate every layer first, then
    // truncate global layers and put back every saved ring slot that does not
    // currently hold a kept speculative position p with base <= p < target.
    // The checkpoint stays live.
    Status rewind_to(const Checkpoint& cp, size_t target) {
        if (auto s = check_live(cp); !s.ok()) return s;
        const Live& data = *live_;
        for (size_t li = 0; li < layers_.size(); ++li) {
            const size_t base = data.bases[li];
            if (target < base || target > layers_[li].appended)
                return Status::fail(kRewindOutOfRange, "rewind target " + zu(target) + " is outside layer " + zu(li) +
                                                           "'s checkpoint range [" + zu(base) + ", " +
                                                           zu(layers_[li].appended) + "]");
        }
        const size_t row = row_len();
        for (size_t li = 0; li < layers_.size(); ++li) {
            Layer& l = layers_[li];
            const size_t base = data.bases[li];
            if (!l.kind.windowed) {
                l.keys.resize(target * row);
                l.values.resize(target * row);
            } else {
                for (const Saved& s : data.saved[li]) {
                    const int64_t p = l.slot_position[s.slot];
                    const bool keep = p != kNoPosition && static_cast<size_t>(p) >= base && static_cast<size_t>(p) < target;
                    if (!keep) {
                        std::memcpy(&l.keys[s.slot * row], s.keys.data(), row * sizeof(float));
                        std::memcpy(&l.values[s.slot * row], s.values.data(), row * sizeof(float));
                        l.slot_position[s.slot] = s.position;
                    }
                }
            }
            l.appended = target;
        }
        return {};
    }

    // crates/attention/src/cache.rs:824-833
    Status release(const Checkpoint& cp) {
        if (auto s = check_live(cp); !s.ok()) return s;
        live_.reset();
        return {};
    }

  private:
    struct Layer {
        LayerKind kind;
        std::vector<float> keys, values;
        std::vector<int64_t> slot_position;
        size_t appended = 0;
    };
    struct Saved {
        size_t slot = 0;
        int64_t position = kNoPosition;
        std::vector<float> keys, values;
    };
    struct Live {
        uint64_t serial = 0;
        size_t max_round_tokens = 0;
        std::vector<size_t> bases;
        std::vector<std::vector<Saved>> saved;
    };

    // Process-wide id source starting at 1 (crates/attention/src/cache.rs:32).
    static uint64_t& next_cache_id() {
        static uint64_t next = 1;
        return next;
    }
    static size_t stored(const Layer& l) {
        return l.kind.windowed ? std::min(l.appended, l.kind.window) : l.appended;
    }
    static size_t slot_of(const Layer& l, size_t position) {
        return l.kind.windowed ? position % l.kind.window : position;
    }
    Status check_layer(size_t layer) const {
        if (layer >= layers_.size())
            return Status::fail(kInvalidLayer,
                                "layer " + zu(layer) + " out of range, cache has " + zu(layers_.size()) + " layers");
        return {};
    }
    // crates/attention/src/cache.rs:719-728
    Status check_live(const Checkpoint& cp) const {
        if (live_ && live_->serial == cp.serial && cp.cache_id == id_) return {};
        return Status::fail(kStaleCheckpoint, "checkpoint " + std::to_string(cp.serial) +
                                                  " is not this cache's live checkpoint (already released or foreign)");
    }
    static Status shape(const char* what, size_t expected, size_t actual) {
        return Status::fail(kShapeMismatch, std::string(what) + ": got " + zu(actual) + ", expected " + zu(expected));
    }

    std::vector<Layer> layers_;
    size_t hkv_ = 0, d_ = 0;
    uint64_t id_ = 0;
    uint64_t next_serial_ = 0;
    std::optional<Live> live_;
};

// ---------------------------------------------------------------------------
// Grouped-query attention: crates/attention/src/attention.rs:35-215.
// ---------------------------------------------------------------------------

// crates/attention/src/attention.rs:35-37
inline float default_scale(size_t head_dim) { return 1.0f / std::sqrt(static_cast<float>(head_dim)); }

// crates/attention/src/attention.rs:43-72
inline Status kv_head_for_query_head(size_t q_head, size_t num_q_heads, size_t num_kv_heads, size_t* out) {
    if (num_kv_heads == 0) return Status::fail(kZeroDimension, "num_kv_heads must be positive, got 0");
    if (num_q_heads == 0) return Status::fail(kZeroDimension, "num_q_heads must be positive, got 0");
    if (num_q_heads % num_kv_heads != 0)
        return Status::fail(kNonDivisibleHeads, zu(num_q_heads) + " query heads do not divide evenly across " +
                                                    zu(num_kv_heads) + " KV heads");
    if (q_head >= num_q_heads)
        return Status::fail(kShapeMismatch, "q_head: got " + zu(q_head) + ", expected " + zu(num_q_heads));
    *out = q_head / (num_q_heads / num_kv_heads);
    return {};
}

// crates/attention/src/attention.rs:77-85: causal, plus (p - window, p] on
// ring layers, compared in signed arithmetic.
inline bool attends(size_t kp, size_t p, std::optional<size_t> window) {
    if (kp > p) return false;
    if (!window) return true;
    return static_cast<int64_t>(kp) > static_cast<int64_t>(p) - static_cast<int64_t>(*window);
}

// crates/attention/src/attention.rs:104-215. Validation order: positions
// length, q length, zero queries -> empty, zero q heads, divisibility. Per
// query the visible set is resolved once; per head the scores are sequential
// f32 dot products times scale, softmax is max-subtracted with exp and the sum
// accumulated in view order, and the output accumulates (e / sum) * v.
inline Status gqa_attention(const float* q, size_t q_len, size_t num_queries, size_t num_q_heads,
                            const size_t* query_positions, size_t num_positions, const KvCache& cache, size_t layer,
                            std::optional<float> scale_opt, std::vector<float>* out) {
    const size_t head_dim = cache.head_dim();
    const size_t num_kv_heads = cache.num_kv_heads();
    if (num_positions != num_queries)
        return Status::fail(kShapeMismatch,
                            "query_positions: got " + zu(num_positions) + ", expected " + zu(num_queries));
    const size_t expected_q = num_queries * num_q_heads * head_dim;
    if (q_len != expected_q) return Status::fail(kShapeMismatch, "q: got " + zu(q_len) + ", expected " + zu(expected_q));
    out->clear();
    if (num_queries == 0) return {};
    if (num_q_heads == 0) return Status::fail(kZeroDimension, "num_q_heads must be positive, got 0");
    if (num_q_heads % num_kv_heads != 0)
        return Status::fail(kNonDivisibleHeads, zu(num_q_heads) + " query heads do not divide evenly across " +
                                                    zu(num_kv_heads) + " KV heads");
    const size_t group = num_q_heads / num_kv_heads;
    const float scale = scale_opt ? *scale_opt : default_scale(head_dim);
    const auto window = cache.window(layer);
    const size_t view_len = cache.view_len(layer);

    out->assign(q_len, 0.0f);
    std::vector<float> scores;
    std::vector<size_t> visible;
    scores.reserve(view_len);
    for (size_t qi = 0; qi < num_queries; ++qi) {
        const size_t p = query_positions[qi];
        visible.clear();
        for (size_t vi = 0; vi < view_len; ++vi) {
            auto kp = cache.position_at(layer, vi);
            if (kp && attends(*kp, p, window)) visible.push_back(vi);
        }
        if (visible.empty())
            return Status::fail(kNoVisibleKeys, "query at position " + zu(p) + " has no visible keys");
        for (size_t h = 0; h < num_q_heads; ++h) {
            const size_t kv_head = h / group;
            const float* qh = q + (qi * num_q_heads + h) * head_dim;
            scores.clear();
            float max = -std::numeric_limits<float>::infinity();
            for (size_t vi : visible) {
                const float* k = cache.key(layer, vi, kv_head);
                float acc = 0.0f;
                for (size_t d = 0; d < head_dim; ++d) acc += qh[d] * k[d];
                const float s = acc * scale;
                if (s > max) max = s;
                scores.push_back(s);
            }
            float sum = 0.0f;
            for (float& s : scores) {
                s = std::exp(s - max);
                sum += s;
            }
            float* o = out->data() + (qi * num_q_heads + h) * head_dim;
            for (size_t i = 0; i < visible.size(); ++i) {
                const float w = scores[i] / sum;
                const float* v = cache.value(layer, visible[i], kv_head);
                for (size_t d = 0; d < head_dim; ++d) o[d] += w * v[d];
            }
        }
    }
    return {};
}

// ---------------------------------------------------------------------------
// Hashes: crates/itak-kv/src/hash.rs:13-61.
// ---------------------------------------------------------------------------
constexpr uint64_t kFnvOffset = 0xcbf29ce484222325ull;
constexpr uint64_t kFnvPrime = 0x00000100000001b3ull;
constexpr uint64_t kAltOffset = 0x84222325cbf29ce4ull;

inline uint64_t fnv1a(const uint8_t* bytes, size_t n, uint64_t basis) {
    uint64_t h = basis;
    for (size_t i = 0; i < n; ++i) {
        h ^= bytes[i];
        h *= kFnvPrime;
    }
    return h;
}
inline uint64_t checksum(const uint8_t* bytes, size_t n) { return fnv1a(bytes, n, kFnvOffset); }
inline uint64_t fold_tokens(const uint32_t* tokens, size_t n, uint64_t basis) {
    uint64_t h = basis;
    for (size_t i = 0; i < n; ++i)
        for (int b = 0; b < 4; ++b) {
            h ^= (tokens[i] >> (8 * b)) & 0xffu;
            h *= kFnvPrime;
        }
    return h;
}
inline uint64_t prefix_hash(const uint32_t* tokens, size_t n) { return fold_tokens(tokens, n, kFnvOffset); }
inline uint64_t prefix_discriminator(const uint32_t* tokens, size_t n) { return fold_tokens(tokens, n, kAltOffset); }

// ---------------------------------------------------------------------------
// Prefix snapshot: crates/itak-kv/src/snapshot.rs:56-540.
// ---------------------------------------------------------------------------
struct KvGeometry {
    std::vector<LayerKind> layers;
    size_t num_kv_heads = 0;
    size_t head_dim = 0;
    size_t row_floats() const { return num_kv_heads * head_dim; }
    bool operator==(const KvGeometry& o) const {
        return layers == o.layers && num_kv_heads == o.num_kv_heads && head_dim == o.head_dim;
    }
    // crates/itak-kv/src/snapshot.rs:100-103 (saturating)
    uint64_t bytes_per_token() const {
        return sat_mul(sat_mul(static_cast<uint64_t>(row_floats()), 8), static_cast<uint64_t>(layers.size()));
    }
    // crates/itak-kv/src/snapshot.rs:110-120 (saturating)
    uint64_t stored_bytes_for(size_t tokens) const {
        const uint64_t per_row = sat_mul(static_cast<uint64_t>(row_floats()), 8);
        uint64_t rows = 0;
        for (const auto& k : layers) {
            const uint64_t r = k.windowed ? std::min(tokens, k.window) : tokens;
            rows = (rows + r < rows) ? UINT64_MAX : rows + r;
        }
        return sat_mul(rows, per_row);
    }
    static uint64_t sat_mul(uint64_t a, uint64_t b) {
        uint64_t r;
        return __builtin_mul_overflow(a, b, &r) ? UINT64_MAX : r;
    }
};

struct LayerSnapshot {
    size_t first_position = 0;
    std::vector<float> keys, values;
};

struct KvSnapshot {
    KvGeometry geometry;
    std::string model_fingerprint;
    size_t token_count = 0;
    std::vector<LayerSnapshot> layers;

    // crates/itak-kv/src/snapshot.rs:187-236
    Status validate() const {
        if (layers.size() != geometry.layers.size())
            return inconsistent("snapshot carries " + zu(layers.size()) + " layer blocks but its geometry has " +
                                zu(geometry.layers.size()) + " layers");
        if (geometry.num_kv_heads == 0 || geometry.head_dim == 0)
            return inconsistent("geometry has a zero KV head count or head dimension");
        size_t row;
        if (mul_overflows(geometry.num_kv_heads, geometry.head_dim, &row))
            return inconsistent("KV row width overflows: " + zu(geometry.num_kv_heads) + " heads of dim " +
                                zu(geometry.head_dim) + " have no usize product");
        for (size_t i = 0; i < layers.size(); ++i) {
            const auto& kind = geometry.layers[i];
            const size_t expected_rows = kind.windowed ? std::min(token_count, kind.window) : token_count;
            const size_t expected_first = token_count - expected_rows;
            if (layers[i].first_position != expected_first)
                return inconsistent("layer " + zu(i) + ": first stored position is " + zu(layers[i].first_position) +
                                    " but " + zu(expected_first) + " follows from token count " + zu(token_count));
            size_t expected_floats;
            if (mul_overflows(expected_rows, row, &expected_floats))
                return inconsistent("layer " + zu(i) + ": " + zu(expected_rows) + " rows of " + zu(row) +
                                    " floats overflow the float count");
            if (layers[i].keys.size() != expected_floats || layers[i].values.size() != expected_floats)
                return inconsistent("layer " + zu(i) + ": holds " + zu(layers[i].keys.size()) + " key and " +
                                    zu(layers[i].values.size()) + " value floats but " + zu(expected_rows) +
                                    " rows of " + zu(row) + " floats were expected");
        }
        return {};
    }

    // crates/itak-kv/src/snapshot.rs:247-302: gather every layer's visible
    // rows in position order; all layers must sit at the same position.
    static Status capture(const KvCache& cache, const std::string& fingerprint, KvSnapshot* out) {
        KvSnapshot s;
        s.geometry.num_kv_heads = cache.num_kv_heads();
        s.geometry.head_dim = cache.head_dim();
        for (size_t i = 0; i < cache.layer_count(); ++i) {
            LayerKind k;
            cache.layer_kind(i, &k);
            s.geometry.layers.push_back(k);
        }
        size_t token_count = 0;
        cache.next_position(0, &token_count);
        const size_t d = cache.head_dim();
        for (size_t i = 0; i < cache.layer_count(); ++i) {
            size_t appended = 0;
            cache.next_position(i, &appended);
            if (appended != token_count)
                return Status::fail(kIncoherentCache, "incoherent cache: layer 0 has appended " + zu(token_count) +
                                                          " positions but layer " + zu(i) + " has appended " +
                                                          zu(appended) + "; a snapshot is one sequence");
            LayerSnapshot ls;
            const size_t visible = cache.view_len(i);
            for (size_t slot = 0; slot < visible; ++slot)
                for (size_t head = 0; head < cache.num_kv_heads(); ++head) {
                    const float* k = cache.key(i, slot, head);
                    const float* v = cache.value(i, slot, head);
                    ls.keys.insert(ls.keys.end(), k, k + d);
                    ls.values.insert(ls.values.end(), v, v + d);
                }
            ls.first_position = token_count - visible;
            s.layers.push_back(std::move(ls));
        }
        s.model_fingerprint = fingerprint;
        s.token_count = token_count;
        if (auto st = s.validate(); !st.ok()) return st;
        *out = std::move(s);
        return {};
    }

    // crates/itak-kv/src/snapshot.rs:321-334: validate, then a fresh cache via
    // restore_bulk; handed out only on full success.
    Status restore(std::unique_ptr<KvCache>* out) const {
        if (auto st = validate(); !st.ok()) return st;
        std::unique_ptr<KvCache> cache;
        if (auto st = KvCache::create(geometry.layers, geometry.num_kv_heads, geometry.head_dim, &cache); !st.ok())
            return st;
        for (size_t i = 0; i < layers.size(); ++i) {
            auto st = cache->restore_bulk(i, layers[i].first_position, layers[i].keys.data(), layers[i].keys.size(),
                                          layers[i].values.data(), layers[i].values.size());
            if (!st.ok()) return st;
        }
        *out = std::move(cache);
        return {};
    }

    // crates/itak-kv/src/snapshot.rs:345-371
    Status restore_checked(const KvGeometry& expected, const std::string& fingerprint,
                           std::unique_ptr<KvCache>* out) const {
        if (!(geometry == expected))
            return Status::fail(kGeometryMismatch,
                                "geometry mismatch: snapshot geometry (" + zu(geometry.layers.size()) + " layers, " +
                                    zu(geometry.num_kv_heads) + " KV heads, head dim " + zu(geometry.head_dim) +
                                    ") differs from the required geometry (" + zu(expected.layers.size()) + " layers, " +
                                    zu(expected.num_kv_heads) + " KV heads, head dim " + zu(expected.head_dim) + ")");
        if (model_fingerprint != fingerprint)
            return Status::fail(kFingerprintMismatch,
                                "fingerprint mismatch: expected " + fingerprint + ", snapshot has " + model_fingerprint);
        return restore(out);
    }

    // crates/itak-kv/src/snapshot.rs:13-29, 381-415: the ITKV byte format.
    Status to_bytes(std::vector<uint8_t>* out) const {
        if (auto st = validate(); !st.ok()) return st;
        std::vector<uint8_t>& b = *out;
        b.clear();
        const char magic[4] = {'I', 'T', 'K', 'V'};
        b.insert(b.end(), magic, magic + 4);
        put_u32(b, 1);
        put_u32(b, static_cast<uint32_t>(model_fingerprint.size()));
        b.insert(b.end(), model_fingerprint.begin(), model_fingerprint.end());
        put_u64(b, token_count);
        put_u32(b, static_cast<uint32_t>(geometry.num_kv_heads));
        put_u32(b, static_cast<uint32_t>(geometry.head_dim));
        put_u32(b, static_cast<uint32_t>(geometry.layers.size()));
        const size_t row = geometry.row_floats();
        for (size_t i = 0; i < layers.size(); ++i) {
            const auto& kind = geometry.layers[i];
            b.push_back(kind.windowed ? 1 : 0);
            b.push_back(0);
            b.push_back(0);
            b.push_back(0);
            put_u64(b, kind.windowed ? kind.window : 0);
            put_u64(b, layers[i].first_position);
            put_u64(b, row ? layers[i].keys.size() / row : 0);
        }
        for (const auto& l : layers) {
            put_f32s(b, l.keys);
            put_f32s(b, l.values);
        }
        put_u64(b, checksum(b.data(), b.size()));
        return {};
    }

    // crates/itak-kv/src/snapshot.rs:425-540: strict decoder. The layer count
    // is bounded by remaining/28 before it sizes anything; trailing bytes
    // refuse; the checksum covers every byte before it.
    static Status from_bytes(const uint8_t* bytes, size_t n, KvSnapshot* out) {
        Reader r{bytes, n, 0};
        const uint8_t* m;
        if (auto st = r.take(4, &m); !st.ok()) return st;
        if (std::memcmp(m, "ITKV", 4) != 0) return Status::fail(kBadMagic, "snapshot: bad magic");
        uint32_t version;
        if (auto st = r.u32(&version); !st.ok()) return st;
        if (version != 1)
            return Status::fail(kUnsupportedVersion, "snapshot: unsupported format version " + std::to_string(version));
        uint32_t fp_len;
        if (auto st = r.u32(&fp_len); !st.ok()) return st;
        const uint8_t* fp;
        if (auto st = r.take(fp_len, &fp); !st.ok()) return st;
        if (!valid_utf8(fp, fp_len)) return inconsistent("model fingerprint is not valid UTF-8");
        KvSnapshot s;
        s.model_fingerprint.assign(reinterpret_cast<const char*>(fp), fp_len);
        uint64_t token_count;
        if (auto st = r.u64(&token_count); !st.ok()) return st;
        s.token_count = static_cast<size_t>(token_count);
        uint32_t hkv, hd, layer_count;
        if (auto st = r.u32(&hkv); !st.ok()) return st;
        if (auto st = r.u32(&hd); !st.ok()) return st;
        if (auto st = r.u32(&layer_count); !st.ok()) return st;
        if (layer_count > r.remaining() / 28)
            return inconsistent("snapshot declares " + std::to_string(layer_count) + " layers but only " +
                                zu(r.remaining()) + " bytes remain, not enough for the layer headers alone");
        s.geometry.num_kv_heads = hkv;
        s.geometry.head_dim = hd;
        std::vector<std::pair<size_t, size_t>> blocks;
        for (uint32_t i = 0; i < layer_count; ++i) {
            const uint8_t* tag;
            if (auto st = r.take(1, &tag); !st.ok()) return st;
            const uint8_t* reserved;
            if (auto st = r.take(3, &reserved); !st.ok()) return st;
            if (reserved[0] || reserved[1] || reserved[2]) return inconsistent("layer header reserved bytes are not zero");
            uint64_t window, first, rows;
            if (auto st = r.u64(&window); !st.ok()) return st;
            if (auto st = r.u64(&first); !st.ok()) return st;
            if (auto st = r.u64(&rows); !st.ok()) return st;
            LayerKind kind;
            if (*tag == 0) {
                kind = LayerKind{false, 0};
            } else if (*tag == 1) {
                if (window == 0) return inconsistent("windowed layer carries a zero window");
                kind = LayerKind{true, static_cast<size_t>(window)};
            } else {
                return inconsistent("layer kind tag " + std::to_string(*tag) + " is not a known kind");
            }
            s.geometry.layers.push_back(kind);
            blocks.emplace_back(static_cast<size_t>(first), static_cast<size_t>(rows));
        }
        size_t row;
        if (mul_overflows(s.geometry.num_kv_heads, s.geometry.head_dim, &row))
            return inconsistent("KV row width overflows");
        for (auto [first, rows] : blocks) {
            size_t floats;
            if (mul_overflows(rows, row, &floats)) return inconsistent("layer row count overflows the row width");
            LayerSnapshot ls;
            ls.first_position = first;
            if (auto st = r.f32s(floats, &ls.keys); !st.ok()) return st;
            if (auto st = r.f32s(floats, &ls.values); !st.ok()) return st;
            s.layers.push_back(std::move(ls));
        }
        uint64_t stored;
        if (auto st = r.u64(&stored); !st.ok()) return st;
        if (r.remaining() != 0) return inconsistent(zu(r.remaining()) + " trailing bytes after the checksum");
        const uint64_t computed = checksum(bytes, n - 8);
        if (stored != computed)
            return Status::fail(kChecksumMismatch, "snapshot: checksum mismatch (stored " + std::to_string(stored) +
                                                       ", computed " + std::to_string(computed) + ")");
        if (auto st = s.validate(); !st.ok()) return st;
        *out = std::move(s);
        return {};
    }

  private:
    static Status inconsistent(std::string detail) {
        return Status::fail(kInconsistentSnapshot, "inconsistent snapshot: " + std::move(detail));
    }
    static void put_u32(std::vector<uint8_t>& b, uint32_t v) {
        for (int i = 0; i < 4; ++i) b.push_back(static_cast<uint8_t>(v >> (8 * i)));
    }
    static void put_u64(std::vector<uint8_t>& b, uint64_t v) {
        for (int i = 0; i < 8; ++i) b.push_back(static_cast<uint8_t>(v >> (8 * i)));
    }
    static void put_f32s(std::vector<uint8_t>& b, const std::vector<float>& f) {
        const size_t at = b.size();
        b.resize(at + f.size() * 4);
        if (!f.empty()) std::memcpy(&b[at], f.data(), f.size() * 4);  // little-endian host
    }
    static bool valid_utf8(const uint8_t* s, size_t n) {
        size_t i = 0;
        while (i < n) {
            const uint8_t c = s[i];
            size_t extra;
            uint32_t cp;
            if (c < 0x80) { i++; continue; }
            else if ((c & 0xe0) == 0xc0) { extra = 1; cp = c & 0x1f; }
            else if ((c & 0xf0) == 0xe0) { extra = 2; cp = c & 0x0f; }
            else if ((c & 0xf8) == 0xf0) { extra = 3; cp = c & 0x07; }
            else return false;
            if (i + extra >= n) return false;
            for (size_t k = 1; k <= extra; ++k) {
                if ((s[i + k] & 0xc0) != 0x80) return false;
                cp = (cp << 6) | (s[i + k] & 0x3f);
            }
            if ((extra == 1 && cp < 0x80) || (extra == 2 && cp < 0x800) || (extra == 3 && cp < 0x10000)) return false;
            if (cp > 0x10ffff || (cp >= 0xd800 && cp <= 0xdfff)) return false;
            i += extra + 1;
        }
        return true;
    }
    // crates/itak-kv/src/snapshot.rs:546-607
    struct Reader {
        const uint8_t* bytes;
        size_t len;
        size_t at;
        size_t remaining() const { return len - at; }
        Status take(size_t n, const uint8_t** out) {
            if (remaining() < n)
                return Status::fail(kTruncated, "snapshot: truncated, needed " + zu(at + n) + " bytes, have " + zu(len));
            *out = bytes + at;
            at += n;
            return {};
        }
        Status u32(uint32_t* v) {
            const uint8_t* p;
            if (auto st = take(4, &p); !st.ok()) return st;
            *v = 0;
            for (int i = 0; i < 4; ++i) *v |= static_cast<uint32_t>(p[i]) << (8 * i);
            return {};
        }
        Status u64(uint64_t* v) {
            const uint8_t* p;
            if (auto st = take(8, &p); !st.ok()) return st;
            *v = 0;
            for (int i = 0; i < 8; ++i) *v |= static_cast<uint64_t>(p[i]) << (8 * i);
            return {};
        }
        Status f32s(size_t count, std::vector<float>* out) {
            size_t nbytes;
            if (mul_overflows(count, 4, &nbytes))
                return Status::fail(kInconsistentSnapshot, "inconsistent snapshot: float count overflows the byte count");
            const uint8_t* p;
            if (auto st = take(nbytes, &p); !st.ok()) return st;
            out->resize(count);
            if (count) std::memcpy(out->data(), p, nbytes);
            return {};
        }
    };
};

// ---------------------------------------------------------------------------
// Slot/ring laws of the device-resident session
// (crates/wgpu-compute/src/session.rs:235-249, 284-346).
// ---------------------------------------------------------------------------
struct SlotRun {
    size_t row, slot, count;
};

// session.rs:284-292: what a snapshot stores of one layer at `position`.
inline std::pair<size_t, size_t> prefix_visible_range(bool sliding, size_t window, size_t position) {
    if (!sliding) return {0, position};
    const size_t rows = std::min(position, window);
    return {position - rows, rows};
}

// session.rs:320-346: maximal runs of consecutive device slots for stored
// rows first_position.. (global = one run; ring = at most two).
inline std::vector<SlotRun> prefix_slot_runs(bool sliding, size_t first_position, size_t rows, size_t ring) {
    std::vector<SlotRun> runs;
    for (size_t r = 0; r < rows; ++r) {
        const size_t position = first_position + r;
        const size_t slot = sliding ? position % ring : position;
        if (!runs.empty() && runs.back().slot + runs.back().count == slot) {
            runs.back().count += 1;
            continue;
        }
        runs.push_back(SlotRun{r, slot, 1});
    }
    return runs;
}

// ---------------------------------------------------------------------------
// The CPU backend's attention step and speculation seam:
// crates/cpu-compute/src/cpu.rs:171-339, 506-655, with the position contract
// of crates/muse-glimmer/src/cache.rs:18-74.
// ---------------------------------------------------------------------------
struct BackendConfig {
    std::vector<bool> sliding;  // per layer: true = sliding-window layer
    size_t q_heads = 0, kv_heads = 0, key_length = 0, value_length = 0;
    size_t sliding_window = 0;
    float rope_freq_base_swa = 10000.0f;
    bool operator==(const BackendConfig& o) const {
        return sliding == o.sliding && kv_heads == o.kv_heads && key_length == o.key_length &&
               value_length == o.value_length && sliding_window == o.sliding_window;
    }
};

struct PositionCache {
    size_t position = 0;
    void advance(size_t tokens) { position += tokens; }
    void rewind_to(size_t p) { position = p; }
};

class CpuBackend {
  public:
    // crates/cpu-compute/src/cpu.rs:264-267
    void reset() {
        cache_.reset();
        shape_.reset();
    }

    // crates/cpu-compute/src/cpu.rs:506-655. One position at a time: rotate q
    // and k (sliding layers only, adjacent pairing), append, view, attend.
    Status attention(const BackendConfig& cfg, size_t layer, bool request_sliding, const float* q, size_t q_len,
                     const float* k, size_t k_len, const float* v, size_t v_len, const PositionCache& pos,
                     std::vector<float>* out) {
        // A refusal that originates in the cache or the attention math keeps its
        // own code and gains the step name; the backend's own refusals are
        // kStepFailed (the reference wraps both as StepFailed{step, detail}).
        auto fail = [](std::string d) { return Status::fail(kStepFailed, "attention: " + std::move(d)); };
        auto wrap = [](const Status& st) { return Status::fail(st.code, "attention: " + st.msg); };
        if (cfg.key_length != cfg.value_length)
            return fail("key_length " + zu(cfg.key_length) + " != value_length " + zu(cfg.value_length) +
                        ": the attention crate's KvCache stores keys and values at one head dimension");
        if (layer >= cfg.sliding.size() || cfg.sliding[layer] != request_sliding)
            return fail("request kind does not match the config's kind for layer " + zu(layer));
        const size_t q_width = cfg.q_heads * cfg.key_length;
        const size_t k_width = cfg.kv_heads * cfg.key_length;
        const size_t v_width = cfg.kv_heads * cfg.value_length;
        if (q_width == 0 || q_len % q_width != 0)
            return fail("query projection holds " + zu(q_len) + " elements, not a whole number of " + zu(q_width) +
                        "-wide rows");
        const size_t rows = q_len / q_width;
        if (k_len != rows * k_width || v_len != rows * v_width)
            return fail("key/value projections hold " + zu(k_len) + "/" + zu(v_len) + " elements for " + zu(rows) +
                        " rows, expected " + zu(rows * k_width) + "/" + zu(rows * v_width));
        const size_t start = pos.position;
        if (!cache_) {
            std::vector<LayerKind> pattern;
            for (bool s : cfg.sliding) pattern.push_back(s ? LayerKind{true, cfg.sliding_window} : LayerKind{false, 0});
            std::unique_ptr<KvCache> c;
            if (auto st = KvCache::create(pattern, cfg.kv_heads, cfg.key_length, &c); !st.ok()) return wrap(st);
            cache_ = std::move(c);
            shape_ = cfg;
        }
        if (!(*shape_ == cfg))
            return fail("this CpuCompute already serves a model of a different shape; construct a fresh CpuCompute per "
                        "model (or reset this one) instead of retargeting it mid-sequence");
        size_t appended;
        if (auto st = cache_->next_position(layer, &appended); !st.ok()) return wrap(st);
        if (appended != start)
            return fail("KV state for layer " + zu(layer) + " is at position " + zu(appended) +
                        " but the sequence cache is at position " + zu(start) + ": the two disagree");
        const size_t d = cfg.key_length;
        out->clear();
        std::vector<float> q_rot(q_width), k_rot(k_width), row_out;
        for (size_t i = 0; i < rows; ++i) {
            const size_t position = start + i;
            const float* qi = q + i * q_width;
            const float* ki = k + i * k_width;
            if (request_sliding) {
                for (size_t h = 0; h < cfg.q_heads; ++h)
                    if (auto st = rope_interleaved_partial(qi + h * d, d, position, cfg.rope_freq_base_swa, d, d,
                                                           q_rot.data() + h * d);
                        !st.ok())
                        return wrap(st);
                for (size_t h = 0; h < cfg.kv_heads; ++h)
                    if (auto st = rope_interleaved_partial(ki + h * d, d, position, cfg.rope_freq_base_swa, d, d,
                                                           k_rot.data() + h * d);
                        !st.ok())
                        return wrap(st);
            } else {
                std::memcpy(q_rot.data(), qi, q_width * sizeof(float));
                std::memcpy(k_rot.data(), ki, k_width * sizeof(float));
            }
            if (auto st = cache_->append(layer, k_rot.data(), k_width, v + i * v_width, v_width, position); !st.ok())
                return wrap(st);
            if (auto st = gqa_attention(q_rot.data(), q_width, 1, cfg.q_heads, &position, 1, *cache_, layer,
                                        std::nullopt, &row_out);
                !st.ok())
                return wrap(st);
            out->insert(out->end(), row_out.begin(), row_out.end());
        }
        return {};
    }

    // crates/cpu-compute/src/cpu.rs:281-339
    Status cache_checkpoint(size_t max_round_tokens, Checkpoint* out) {
        if (!cache_)
            return Status::fail(kStepFailed, "cache_checkpoint: no KV state exists yet: a speculative round checkpoints "
                                             "after a first forward has built the cache (the spec's prefill), not before");
        auto st = cache_->checkpoint(max_round_tokens, out);
        if (!st.ok()) st.msg = "cache_checkpoint: " + st.msg;
        return st;
    }
    Status cache_rewind(const Checkpoint& cp, size_t target) {
        if (!cache_)
            return Status::fail(kStepFailed,
                                "cache_rewind: no KV state exists: the sequence was reset after the checkpoint was taken");
        auto st = cache_->rewind_to(cp, target);
        if (!st.ok()) st.msg = "cache_rewind: " + st.msg;
        return st;
    }
    Status cache_release(const Checkpoint& cp) {
        if (!cache_)
            return Status::fail(kStepFailed,
                                "cache_release: no KV state exists: the sequence was reset after the checkpoint was taken");
        auto st = cache_->release(cp);
        if (!st.ok()) st.msg = "cache_release: " + st.msg;
        return st;
    }
    KvCache* cache() { return cache_.get(); }

  private:
    std::unique_ptr<KvCache> cache_;
    std::optional<BackendConfig> shape_;
};

// ---------------------------------------------------------------------------
// Draft-model (DFlash) attention.  Follows crates/dflash/src/model.rs:388-466: for query row r at positions[r],
// the visible set is the committed rows in ascending position order, then the block's own rows in order, each
// kept unless (causal and kp > p) or (sliding and kp <= p - window, signed); per query head: scores = dot * scale
// with scale = 1 / sqrt(key_len as f32) (sequential f32 dot, :585-587), max, e = exp(s - max) summed in order,
// out += (e / sum) * v.  `committed_k` / `committed_v` are compact here ([committed][kv_heads * len], in the order
// of `committed_positions`), as the CPU cache's map iteration yields them (crates/dflash/src/cache.rs:96-104).
inline Status draft_attention(const float* q, size_t rows, size_t q_heads, size_t kv_heads, size_t key_len,
                              size_t value_len, const uint64_t* positions, const uint64_t* committed_positions,
                              size_t committed, const float* committed_k, const float* committed_v,
                              const float* block_k, const float* block_v, bool causal, bool sliding, uint64_t window,
                              float* out) {
    if (q_heads == 0 || kv_heads == 0 || q_heads % kv_heads != 0)
        return Status::fail(kNonDivisibleHeads, "q_heads " + zu(q_heads) + " must be a whole multiple of kv_heads " +
                                                    zu(kv_heads) + ", both non-zero");
    if (key_len == 0 || value_len == 0) return Status::fail(kZeroDimension, "key_len / value_len is zero");
    const size_t group = q_heads / kv_heads;
    const size_t k_w = kv_heads * key_len, v_w = kv_heads * value_len;
    const float scale = 1.0f / std::sqrt(static_cast<float>(key_len));
    for (size_t i = 0; i < rows * q_heads * value_len; ++i) out[i] = 0.0f;
    std::vector<std::pair<const float*, const float*>> visible;
    std::vector<float> scores;
    for (size_t r = 0; r < rows; ++r) {
        const int64_t p = static_cast<int64_t>(positions[r]);
        const int64_t w = static_cast<int64_t>(window);
        visible.clear();
        for (size_t c = 0; c < committed; ++c) {
            const int64_t kp = static_cast<int64_t>(committed_positions[c]);
            if (causal && kp > p) continue;
            if (sliding && kp <= p - w) continue;
            visible.emplace_back(committed_k + c * k_w, committed_v + c * v_w);
        }
        for (size_t m = 0; m < rows; ++m) {
            const int64_t mp = static_cast<int64_t>(positions[m]);
            if (causal && mp > p) continue;
            if (sliding && mp <= p - w) continue;
            visible.emplace_back(block_k + m * k_w, block_v + m * v_w);
        }
        for (size_t head = 0; head < q_heads; ++head) {
            const size_t kv_head = head / group;
            const float* qh = q + (r * q_heads + head) * key_len;
            scores.clear();
            float max = -INFINITY;
            for (const auto& kv : visible) {
                const float* kh = kv.first + kv_head * key_len;
                float dot = 0.0f;
                for (size_t d = 0; d < key_len; ++d) dot += qh[d] * kh[d];
                const float s = dot * scale;
                if (s > max) max = s;
                scores.push_back(s);
            }
            float sum = 0.0f;
            for (float& s : scores) {
                s = std::exp(s - max);
                sum += s;
            }
            float* o = out + (r * q_heads + head) * value_len;
            for (size_t i = 0; i < visible.size(); ++i) {
                const float weight = scores[i] / sum;
                const float* vh = visible[i].second + kv_head * value_len;
                for (size_t d = 0; d < value_len; ++d) o[d] += weight * vh[d];
            }
        }
    }
    return {};
}

}  // namespace orc
