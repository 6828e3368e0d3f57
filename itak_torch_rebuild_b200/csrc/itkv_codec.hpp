// Host-side byte handling of the ITKV snapshot wire format (crates/itak-kv/src/snapshot.rs:13-29, strict decoder
// :381-540) and the FNV-1a hashes that key prefix entries (crates/itak-kv/src/hash.rs:13-61).  Shared by the
// device snapshot codec and the on-disk prefix store; nothing here touches the GPU.
#pragma once

#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/itak_cuda_compute.h"

namespace itk {
namespace itkv {

constexpr uint64_t kFnvOffset = 0xcbf29ce484222325ull;  // hash.rs:13-16
constexpr uint64_t kFnvPrime = 0x00000100000001b3ull;
constexpr uint64_t kAltOffset = 0x84222325cbf29ce4ull;  // hash.rs:21 (filename discriminator)

inline uint64_t fnv1a64(const uint8_t* p, size_t n, uint64_t basis = kFnvOffset) {
    uint64_t h = basis;
    for (size_t i = 0; i < n; ++i) {
        h ^= p[i];
        h *= kFnvPrime;
    }
    return h;
}

// hash.rs:44-56: every token id folded as its four little-endian bytes.
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

// Strict little-endian cursor (snapshot.rs:546-607).
struct Reader {
    const uint8_t* bytes;
    size_t len, at;
    size_t remaining() const { return len - at; }
    bool take(size_t n, const uint8_t** out) {
        if (remaining() < n) return false;
        *out = bytes + at;
        at += n;
        return true;
    }
    bool u32(uint32_t* v) {
        const uint8_t* p;
        if (!take(4, &p)) return false;
        *v = 0;
        for (int i = 0; i < 4; ++i) *v |= static_cast<uint32_t>(p[i]) << (8 * i);
        return true;
    }
    bool u64(uint64_t* v) {
        const uint8_t* p;
        if (!take(8, &p)) return false;
        *v = 0;
        for (int i = 0; i < 8; ++i) *v |= static_cast<uint64_t>(p[i]) << (8 * i);
        return true;
    }
};

inline bool valid_utf8(const uint8_t* s, size_t n) {
    size_t i = 0;
    while (i < n) {
        const uint8_t c = s[i];
        size_t extra;
        uint32_t cp;
        if (c < 0x80) { ++i; continue; }
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

// Format versions.  Version 1 is the reference's: f32 rows.  Version 2 (this library's extension for f16 caches,
// which the reference refuses to snapshot, crates/wgpu-compute/src/session.rs:383-398) is the same layout with one
// more header field - a u32 element type directly after the version, 0 = f32, 1 = IEEE half - and rows stored in
// that type, little-endian; everything else, the checksum included, is unchanged.
constexpr uint32_t kVersionF32 = 1, kVersionTyped = 2;
constexpr uint32_t kElemF32 = 0, kElemF16 = 1;

// A decoded, validated snapshot: geometry, per-layer headers and where each layer's rows sit in the bytes.
struct Parsed {
    uint32_t version = kVersionF32;
    uint32_t elem_bytes = 4;  // 4 = f32 rows, 2 = half rows (version 2 only)
    std::string fingerprint;
    uint64_t token_count = 0;
    uint32_t kv_heads = 0, head_dim = 0, layer_count = 0;
    std::vector<uint64_t> windows, firsts, rows;  // per layer: 0 = global or the window; first position; row count
    std::vector<const uint8_t*> kptr, vptr;       // per layer: little-endian rows inside `bytes` (unaligned)
};

// KvSnapshot::from_bytes followed by KvSnapshot::validate (snapshot.rs:187-236, 381-540).  Returns ITK_OK or the
// refusal's code with its text in *why.
inline int parse(const uint8_t* bytes, size_t n, Parsed* out, std::string* why) {
    auto zu = [](unsigned long long v) { return std::to_string(v); };
    auto fail = [&](int code, std::string msg) {
        *why = std::move(msg);
        return code;
    };
    auto truncated = [&](const Reader& r, size_t want) {
        return fail(ITK_ERR_TRUNCATED, "snapshot: truncated, needed " + zu(r.at + want) + " bytes, have " + zu(r.len));
    };
    auto inconsistent = [&](std::string d) { return fail(ITK_ERR_INCONSISTENT_SNAPSHOT, "inconsistent snapshot: " + d); };
    Reader r{bytes, n, 0};
    const uint8_t* p;
    if (!r.take(4, &p)) return truncated(r, 4);
    if (std::memcmp(p, "ITKV", 4) != 0) return fail(ITK_ERR_BAD_MAGIC, "snapshot: bad magic");
    uint32_t version;
    if (!r.u32(&version)) return truncated(r, 4);
    if (version != kVersionF32 && version != kVersionTyped)
        return fail(ITK_ERR_UNSUPPORTED_VERSION, "snapshot: unsupported format version " + zu(version));
    uint64_t elem_bytes = 4;
    if (version == kVersionTyped) {
        uint32_t elem;
        if (!r.u32(&elem)) return truncated(r, 4);
        if (elem == kElemF16) elem_bytes = 2;
        else if (elem != kElemF32) return inconsistent("element type tag " + zu(elem) + " is not a known type");
    }
    uint32_t fp_len;
    if (!r.u32(&fp_len)) return truncated(r, 4);
    const uint8_t* fp;
    if (!r.take(fp_len, &fp)) return truncated(r, fp_len);
    if (!valid_utf8(fp, fp_len)) return inconsistent("model fingerprint is not valid UTF-8");
    uint64_t token_count;
    uint32_t hkv, hd, layer_count;
    if (!r.u64(&token_count)) return truncated(r, 8);
    if (!r.u32(&hkv)) return truncated(r, 4);
    if (!r.u32(&hd)) return truncated(r, 4);
    if (!r.u32(&layer_count)) return truncated(r, 4);
    if (layer_count > r.remaining() / 28)
        return inconsistent("snapshot declares " + zu(layer_count) + " layers but only " + zu(r.remaining()) +
                            " bytes remain, not enough for the layer headers alone");
    std::vector<uint64_t> windows(layer_count), firsts(layer_count), rows(layer_count);
    for (uint32_t l = 0; l < layer_count; ++l) {
        const uint8_t *tag, *reserved;
        if (!r.take(1, &tag)) return truncated(r, 1);
        if (!r.take(3, &reserved)) return truncated(r, 3);
        if (reserved[0] || reserved[1] || reserved[2]) return inconsistent("layer header reserved bytes are not zero");
        uint64_t window;
        if (!r.u64(&window)) return truncated(r, 8);
        if (!r.u64(&firsts[l])) return truncated(r, 8);
        if (!r.u64(&rows[l])) return truncated(r, 8);
        if (*tag == 0) {
            windows[l] = 0;
        } else if (*tag == 1) {
            if (window == 0) return inconsistent("windowed layer carries a zero window");
            windows[l] = window;
        } else {
            return inconsistent("layer kind tag " + zu(*tag) + " is not a known kind");
        }
    }
    uint64_t row;
    if (__builtin_mul_overflow(static_cast<uint64_t>(hkv), static_cast<uint64_t>(hd), &row))
        return inconsistent("KV row width overflows");
    std::vector<const uint8_t*> kptr(layer_count), vptr(layer_count);
    for (uint32_t l = 0; l < layer_count; ++l) {
        uint64_t floats, nbytes;
        if (__builtin_mul_overflow(rows[l], row, &floats)) return inconsistent("layer row count overflows the row width");
        if (__builtin_mul_overflow(floats, elem_bytes, &nbytes))
            return inconsistent("float count overflows the byte count");
        if (!r.take(nbytes, &kptr[l])) return truncated(r, nbytes);
        if (!r.take(nbytes, &vptr[l])) return truncated(r, nbytes);
    }
    uint64_t stored;
    if (!r.u64(&stored)) return truncated(r, 8);
    if (r.remaining() != 0) return inconsistent(zu(r.remaining()) + " trailing bytes after the checksum");
    const uint64_t computed = fnv1a64(bytes, n - 8);
    if (stored != computed)
        return fail(ITK_ERR_CHECKSUM_MISMATCH,
                    "snapshot: checksum mismatch (stored " + zu(stored) + ", computed " + zu(computed) + ")");
    // KvSnapshot::validate (snapshot.rs:187-236)
    if (hkv == 0 || hd == 0) return inconsistent("geometry has a zero KV head count or head dimension");
    for (uint32_t l = 0; l < layer_count; ++l) {
        const uint64_t want_rows = windows[l] ? (token_count < windows[l] ? token_count : windows[l]) : token_count;
        if (firsts[l] != token_count - want_rows)
            return inconsistent("layer " + zu(l) + ": first stored position is " + zu(firsts[l]) + " but " +
                                zu(token_count - want_rows) + " follows from token count " + zu(token_count));
        if (rows[l] != want_rows)
            return inconsistent("layer " + zu(l) + ": holds " + zu(rows[l]) + " rows but " + zu(want_rows) + " rows were expected");
    }
    out->version = version;
    out->elem_bytes = static_cast<uint32_t>(elem_bytes);
    out->fingerprint.assign(reinterpret_cast<const char*>(fp), fp_len);
    out->token_count = token_count;
    out->kv_heads = hkv;
    out->head_dim = hd;
    out->layer_count = layer_count;
    out->windows = std::move(windows);
    out->firsts = std::move(firsts);
    out->rows = std::move(rows);
    out->kptr = std::move(kptr);
    out->vptr = std::move(vptr);
    return ITK_OK;
}

}  // namespace itkv
}  // namespace itk
