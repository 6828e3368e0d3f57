// Prefix snapshots kept on disk between runs.  Each stored prefix is a file of its own inside one directory; a
// lookup finds the longest stored run of token ids that starts the query; a byte budget caps the directory and the
// entries that were used longest ago are deleted first when it is exceeded.  Everything here runs on the host: an
// entry's payload is an ITKV snapshot, which itk_snapshot_to_itkv / itk_snapshot_from_itkv carry to and from the GPU.
//
// Stands in for crates/itak-kv/src/store.rs (entry layout :5-21, trust model :23-33, atomic writes :35-39,
// last-used stamping and eviction :41-46, index by scan at open :48-52) and writes the same bytes under the same
// file names, so a directory can be shared with the reference's own store.
//
// Entry file (all integers little-endian), store.rs:5-21:
//   preamble, 72 bytes: "ITKVPENT", u32 version (1), u32 zero, u64 created, u64 last used (offset 24, rewritten in
//   place on a verified hit), u64 prefix hash, u64 token count, u64 tokens bytes (4 x count), u64 payload bytes,
//   u64 zero; then the token ids (u32 each); then the snapshot bytes.
// File name: {prefix_hash:016x}-{token_count}-{discriminator:016x}[-c{n}].kv (store.rs:459-502); temp files start
// with ".tmp-" and are never indexed.
#include <dirent.h>
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cinttypes>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "itkv_codec.hpp"

namespace {

constexpr size_t kPreambleLen = 72;
constexpr uint64_t kLastUsedOffset = 24;
constexpr uint32_t kEntryVersion = 1;
const char kEntryMagic[9] = "ITKVPENT";
const char kEntrySuffix[] = ".kv";
const char kTempPrefix[] = ".tmp-";

std::string zu(unsigned long long v) { return std::to_string(v); }
std::string hex18(uint64_t v) {  // Rust's {:#018x}
    char buf[32];
    snprintf(buf, sizeof buf, "0x%016" PRIx64, v);
    return buf;
}
std::string hexx(uint64_t v) {  // Rust's {:#x}
    char buf[32];
    snprintf(buf, sizeof buf, "0x%" PRIx64, v);
    return buf;
}

struct EntryMeta {
    std::string file_name;
    uint64_t prefix_hash = 0, token_count = 0, bytes = 0, created = 0, last_used = 0;
};

struct Preamble {
    uint64_t created = 0, last_used = 0, prefix_hash = 0, token_count = 0, payload_bytes = 0;
};

uint64_t le64(const uint8_t* p) {
    uint64_t v = 0;
    for (int i = 0; i < 8; ++i) v |= static_cast<uint64_t>(p[i]) << (8 * i);
    return v;
}
void put64(uint8_t* p, uint64_t v) {
    for (int i = 0; i < 8; ++i) p[i] = static_cast<uint8_t>(v >> (8 * i));
}

// store.rs:556-567
void encode_preamble(const Preamble& pr, uint8_t out[kPreambleLen]) {
    std::memset(out, 0, kPreambleLen);
    std::memcpy(out, kEntryMagic, 8);
    for (int i = 0; i < 4; ++i) out[8 + i] = static_cast<uint8_t>(kEntryVersion >> (8 * i));
    put64(out + 16, pr.created);
    put64(out + 24, pr.last_used);
    put64(out + 32, pr.prefix_hash);
    put64(out + 40, pr.token_count);
    put64(out + 48, pr.token_count * 4);
    put64(out + 56, pr.payload_bytes);
}

struct Refusal {
    int code = ITK_OK;
    std::string text;
    explicit operator bool() const { return code != ITK_OK; }
};
Refusal refuse(int code, std::string text) { return Refusal{code, std::move(text)}; }
Refusal io_refusal(const std::string& context) { return refuse(ITK_ERR_IO, context + ": " + std::strerror(errno)); }

// store.rs:569-609
Refusal parse_preamble(const uint8_t* bytes, size_t n, Preamble* out) {
    if (n < kPreambleLen)
        return refuse(ITK_ERR_TRUNCATED, "entry: truncated, needs " + zu(kPreambleLen) + " bytes, has " + zu(n));
    if (std::memcmp(bytes, kEntryMagic, 8) != 0) return refuse(ITK_ERR_BAD_MAGIC, "entry: bad magic");
    uint32_t version = 0;
    for (int i = 0; i < 4; ++i) version |= static_cast<uint32_t>(bytes[8 + i]) << (8 * i);
    if (version != kEntryVersion)
        return refuse(ITK_ERR_UNSUPPORTED_VERSION, "entry: unsupported format version " + zu(version));
    const uint64_t token_count = le64(bytes + 40), tokens_bytes = le64(bytes + 48);
    uint64_t expected;
    if (__builtin_mul_overflow(token_count, static_cast<uint64_t>(4), &expected)) expected = ~0ull;  // saturating
    if (tokens_bytes != expected)
        return refuse(ITK_ERR_INCONSISTENT_SNAPSHOT, "inconsistent snapshot: entry tokens_bytes is " + zu(tokens_bytes) +
                                                         " but token count " + zu(token_count) + " implies " + zu(expected));
    out->created = le64(bytes + 16);
    out->last_used = le64(bytes + 24);
    out->prefix_hash = le64(bytes + 32);
    out->token_count = token_count;
    out->payload_bytes = le64(bytes + 56);
    return {};
}

Refusal read_file(const std::string& path, const std::string& context, std::vector<uint8_t>* out) {
    const int fd = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
    if (fd < 0) return io_refusal(context);
    struct stat st;
    if (fstat(fd, &st) != 0) {
        const Refusal r = io_refusal(context);
        ::close(fd);
        return r;
    }
    out->resize(static_cast<size_t>(st.st_size));
    size_t at = 0;
    while (at < out->size()) {
        const ssize_t got = ::read(fd, out->data() + at, out->size() - at);
        if (got < 0 && errno == EINTR) continue;
        if (got <= 0) break;
        at += static_cast<size_t>(got);
    }
    ::close(fd);
    out->resize(at);
    return {};
}

// store.rs:611-634: the preamble only, plus the file size
Refusal read_preamble(const std::string& dir, const std::string& name, EntryMeta* out) {
    const std::string path = dir + "/" + name;
    const int fd = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
    if (fd < 0) return io_refusal("open " + path);
    uint8_t head[kPreambleLen];
    size_t at = 0;
    while (at < kPreambleLen) {
        const ssize_t got = ::read(fd, head + at, kPreambleLen - at);
        if (got < 0 && errno == EINTR) continue;
        if (got <= 0) break;
        at += static_cast<size_t>(got);
    }
    struct stat st;
    const bool stat_ok = fstat(fd, &st) == 0;
    ::close(fd);
    if (at < kPreambleLen) return refuse(ITK_ERR_IO, "read preamble of " + path + ": failed to fill whole buffer");
    Preamble pr;
    if (Refusal r = parse_preamble(head, kPreambleLen, &pr)) return r;
    if (!stat_ok) return io_refusal("stat " + path);
    out->file_name = name;
    out->prefix_hash = pr.prefix_hash;
    out->token_count = pr.token_count;
    out->bytes = static_cast<uint64_t>(st.st_size);
    out->created = pr.created;
    out->last_used = pr.last_used;
    return {};
}

// store.rs:636-653
bool read_entry_tokens(const std::string& path, std::vector<uint32_t>* out) {
    std::vector<uint8_t> bytes;
    if (read_file(path, "read " + path, &bytes)) return false;
    Preamble pr;
    if (parse_preamble(bytes.data(), bytes.size(), &pr)) return false;
    uint64_t end;
    if (__builtin_mul_overflow(pr.token_count, static_cast<uint64_t>(4), &end) ||
        __builtin_add_overflow(end, static_cast<uint64_t>(kPreambleLen), &end) || bytes.size() < end)
        return false;
    out->resize(pr.token_count);
    for (uint64_t i = 0; i < pr.token_count; ++i) {
        const uint8_t* p = bytes.data() + kPreambleLen + 4 * i;
        (*out)[i] = static_cast<uint32_t>(p[0]) | (static_cast<uint32_t>(p[1]) << 8) | (static_cast<uint32_t>(p[2]) << 16) |
                    (static_cast<uint32_t>(p[3]) << 24);
    }
    return true;
}

bool ends_with(const std::string& s, const char* suffix) {
    const size_t n = std::strlen(suffix);
    return s.size() >= n && s.compare(s.size() - n, n, suffix) == 0;
}

std::string g_open_error;  // text of the last failed open

}  // namespace

struct itk_prefix_store {
    std::string root;
    uint64_t max_bytes = 0;
    std::vector<EntryMeta> entries;
    std::string err;           // last refusal of a call
    std::string last_refusal;  // last candidate or scanned file refused by name (the reference's diag line)
    std::vector<uint8_t> hit;  // bytes of the last verified hit
    std::vector<uint32_t> hit_tokens;

    int fail(const Refusal& r) {
        err = r.text;
        return r.code;
    }
    uint64_t total_bytes() const {
        uint64_t t = 0;
        for (const EntryMeta& e : entries) t += e.bytes;
        return t;
    }

    // store.rs:205-228
    Refusal rescan() {
        DIR* d = opendir(root.c_str());
        if (!d) return io_refusal("list store root " + root);
        std::vector<EntryMeta> found;
        while (dirent* item = readdir(d)) {
            const std::string name = item->d_name;
            if (name == "." || name == "..") continue;
            if (name.rfind(kTempPrefix, 0) == 0 || !ends_with(name, kEntrySuffix)) continue;
            EntryMeta meta;
            if (Refusal r = read_preamble(root, name, &meta)) {
                last_refusal = "prefix store refuses entry " + name + ": " + r.text;
                continue;
            }
            found.push_back(std::move(meta));
        }
        closedir(d);
        entries = std::move(found);
        return {};
    }

    // store.rs:459-502
    Refusal pick_file_name(const uint32_t* tokens, size_t n, uint64_t key, std::string* out) {
        char base[80];
        snprintf(base, sizeof base, "%016" PRIx64 "-%zu-%016" PRIx64, key, n, itk::itkv::prefix_discriminator(tokens, n));
        const std::vector<uint32_t> want(tokens, tokens + n);
        for (uint32_t counter = 0; counter < 1024; ++counter) {
            const std::string name = counter == 0 ? std::string(base) + kEntrySuffix
                                                  : std::string(base) + "-c" + zu(counter) + kEntrySuffix;
            const std::string path = root + "/" + name;
            const bool indexed =
                std::any_of(entries.begin(), entries.end(), [&](const EntryMeta& e) { return e.file_name == name; });
            std::vector<uint32_t> existing;
            if (!indexed) {
                // The name may still exist on disk from a writer this instance has not indexed; check the ids.
                if (::access(path.c_str(), F_OK) == 0 && read_entry_tokens(path, &existing)) {
                    if (existing == want) {
                        *out = name;
                        return {};
                    }
                    continue;
                }
                *out = name;
                return {};
            }
            if (read_entry_tokens(path, &existing) && existing == want) {
                *out = name;
                return {};
            }
        }
        return refuse(ITK_ERR_INVALID_CONFIG, "invalid config: no free filename for prefix hash " + hexx(key) +
                                                  " after 1024 collisions; the store directory is not behaving like a prefix store");
    }

    // store.rs:518-546
    Refusal evict_except(const std::string& keep) {
        while (total_bytes() > max_bytes) {
            const EntryMeta* victim = nullptr;
            for (const EntryMeta& e : entries) {
                if (e.file_name == keep) continue;
                if (!victim || e.last_used < victim->last_used ||
                    (e.last_used == victim->last_used && e.file_name < victim->file_name))
                    victim = &e;
            }
            if (!victim) break;
            const std::string name = victim->file_name;
            if (::unlink((root + "/" + name).c_str()) != 0) return io_refusal("evict entry " + name);
            entries.erase(std::remove_if(entries.begin(), entries.end(), [&](const EntryMeta& e) { return e.file_name == name; }),
                          entries.end());
        }
        return {};
    }

    // store.rs:364-452.  *matched: the entry is this query's prefix and passed every trust check.
    Refusal verify_candidate(const EntryMeta& meta, const uint32_t* query, const itk_config* geometry,
                             const char* fingerprint, std::vector<uint8_t>* bytes, std::vector<uint32_t>* tokens,
                             bool* matched) {
        *matched = false;
        if (Refusal r = read_file(root + "/" + meta.file_name, "read entry " + meta.file_name, bytes)) return r;
        Preamble pr;
        if (Refusal r = parse_preamble(bytes->data(), bytes->size(), &pr)) return r;
        if (pr.prefix_hash != meta.prefix_hash || pr.token_count != meta.token_count)
            return refuse(ITK_ERR_INCONSISTENT_SNAPSHOT,
                          "inconsistent snapshot: entry " + meta.file_name + " changed between scan and read (index hash " +
                              hexx(meta.prefix_hash) + " / " + zu(meta.token_count) + " tokens, file hash " +
                              hexx(pr.prefix_hash) + " / " + zu(pr.token_count) + " tokens)");
        const uint64_t tokens_end = kPreambleLen + pr.token_count * 4;  // token_count <= query length here
        if (bytes->size() < tokens_end)
            return refuse(ITK_ERR_TRUNCATED, "entry: truncated, needs " + zu(tokens_end) + " bytes, has " + zu(bytes->size()));
        tokens->resize(pr.token_count);
        for (uint64_t i = 0; i < pr.token_count; ++i) {
            const uint8_t* p = bytes->data() + kPreambleLen + 4 * i;
            (*tokens)[i] = static_cast<uint32_t>(p[0]) | (static_cast<uint32_t>(p[1]) << 8) |
                           (static_cast<uint32_t>(p[2]) << 16) | (static_cast<uint32_t>(p[3]) << 24);
        }
        // Trust check 1: the stored ids must hash back to the key.
        const uint64_t computed = itk::itkv::prefix_hash(tokens->data(), tokens->size());
        if (computed != pr.prefix_hash)
            return refuse(ITK_ERR_PREFIX_HASH_MISMATCH, "stored token ids hash to " + hex18(computed) + ", not the entry key " +
                                                            hex18(pr.prefix_hash) + "; entry refused");
        // Prefix check: not an error, just not this query's branch.
        if (!std::equal(tokens->begin(), tokens->end(), query)) return {};
        // Trust check 2: the payload must decode whole and agree with the preamble.
        const uint64_t payload_len = bytes->size() - tokens_end;
        if (payload_len != pr.payload_bytes)
            return refuse(ITK_ERR_TRUNCATED,
                          "entry payload: truncated, needs " + zu(pr.payload_bytes) + " bytes, has " + zu(payload_len));
        itk::itkv::Parsed snap;
        std::string why;
        if (int rc = itk::itkv::parse(bytes->data() + tokens_end, payload_len, &snap, &why)) return refuse(rc, why);
        if (snap.token_count != pr.token_count)
            return refuse(ITK_ERR_SNAPSHOT_TOKEN_MISMATCH, "entry preamble covers " + zu(pr.token_count) +
                                                               " tokens but its snapshot covers " + zu(snap.token_count));
        // Trust check 3: caller-required geometry and fingerprint.
        if (geometry) {
            bool same = snap.layer_count == geometry->n_layers && snap.kv_heads == geometry->kv_heads &&
                        snap.head_dim == geometry->head_dim;
            for (uint32_t l = 0; same && l < snap.layer_count; ++l)
                same = snap.windows[l] == (geometry->layer_window ? geometry->layer_window[l] : 0u);
            if (!same)
                return refuse(ITK_ERR_GEOMETRY_MISMATCH, "geometry mismatch: entry " + meta.file_name +
                                                             " snapshot geometry differs from the required geometry");
        }
        if (fingerprint && snap.fingerprint != fingerprint)
            return refuse(ITK_ERR_FINGERPRINT_MISMATCH, std::string("model fingerprint mismatch: need ") + fingerprint +
                                                            ", snapshot carries " + snap.fingerprint);
        *matched = true;
        return {};
    }
};

extern "C" {

// PrefixStore::open (store.rs:147-170)
int itk_prefix_store_open(const char* root, uint64_t max_bytes, itk_prefix_store** out) {
    if (!root || !out) return ITK_ERR_INVALID_ARGUMENT;
    if (max_bytes == 0) {
        g_open_error = "invalid config: the store byte cap is zero";
        return ITK_ERR_INVALID_CONFIG;
    }
    // create_dir_all
    std::string path(root), partial;
    for (size_t i = 0; i <= path.size(); ++i) {
        if (i == path.size() || path[i] == '/') {
            partial = path.substr(0, i);
            if (!partial.empty() && ::mkdir(partial.c_str(), 0777) != 0 && errno != EEXIST) {
                g_open_error = "create store root " + path + ": " + std::strerror(errno);
                return ITK_ERR_IO;
            }
        }
    }
    auto* s = new itk_prefix_store;
    s->root = path;
    s->max_bytes = max_bytes;
    if (Refusal r = s->rescan()) {
        g_open_error = r.text;
        delete s;
        return r.code;
    }
    *out = s;
    return ITK_OK;
}

void itk_prefix_store_close(itk_prefix_store* s) { delete s; }

const char* itk_prefix_store_last_error(const itk_prefix_store* s) { return s ? s->err.c_str() : g_open_error.c_str(); }
const char* itk_prefix_store_last_refusal(const itk_prefix_store* s) { return s ? s->last_refusal.c_str() : ""; }

int itk_prefix_store_rescan(itk_prefix_store* s) {
    if (!s) return ITK_ERR_INVALID_ARGUMENT;
    if (Refusal r = s->rescan()) return s->fail(r);
    return ITK_OK;
}

// PrefixStore::put (store.rs:236-303).  `itkv` is the snapshot's encoding (KvSnapshot::to_bytes).
int itk_prefix_store_put(itk_prefix_store* s, const uint32_t* tokens, size_t n_tokens, const uint8_t* itkv, size_t itkv_len,
                         uint64_t now) {
    if (!s || (!tokens && n_tokens) || !itkv) return ITK_ERR_INVALID_ARGUMENT;
    if (n_tokens == 0) return s->fail(refuse(ITK_ERR_EMPTY_PREFIX, "empty token prefix refused"));
    itk::itkv::Parsed snap;
    std::string why;
    if (int rc = itk::itkv::parse(itkv, itkv_len, &snap, &why)) return s->fail(refuse(rc, why));
    if (snap.token_count != n_tokens)
        return s->fail(refuse(ITK_ERR_TOKEN_COUNT_MISMATCH, "snapshot covers " + zu(snap.token_count) +
                                                                " tokens but was offered under " + zu(n_tokens) + " token ids"));
    const uint64_t key = itk::itkv::prefix_hash(tokens, n_tokens);
    const uint64_t entry_bytes = kPreambleLen + n_tokens * 4 + itkv_len;
    if (entry_bytes > s->max_bytes)
        return s->fail(refuse(ITK_ERR_ENTRY_TOO_LARGE, "entry of " + zu(entry_bytes) + " bytes exceeds the store cap of " +
                                                           zu(s->max_bytes) + " bytes"));
    std::string file_name;
    if (Refusal r = s->pick_file_name(tokens, n_tokens, key, &file_name)) return s->fail(r);
    // Atomic write: temp file in the same directory, sync, rename over the final name.
    const std::string temp_name = std::string(kTempPrefix) + file_name + "-" + zu(static_cast<unsigned long long>(getpid()));
    const std::string temp_path = s->root + "/" + temp_name, path = s->root + "/" + file_name;
    std::vector<uint8_t> head(kPreambleLen + n_tokens * 4);
    Preamble pr;
    pr.created = pr.last_used = now;
    pr.prefix_hash = key;
    pr.token_count = n_tokens;
    pr.payload_bytes = itkv_len;
    encode_preamble(pr, head.data());
    for (size_t i = 0; i < n_tokens; ++i)
        for (int b = 0; b < 4; ++b) head[kPreambleLen + 4 * i + b] = static_cast<uint8_t>(tokens[i] >> (8 * b));
    const int fd = ::open(temp_path.c_str(), O_WRONLY | O_CREAT | O_TRUNC | O_CLOEXEC, 0666);
    if (fd < 0) return s->fail(io_refusal("create temp entry " + temp_name));
    auto write_all = [&](const uint8_t* p, size_t n) {
        while (n) {
            const ssize_t put = ::write(fd, p, n);
            if (put < 0 && errno == EINTR) continue;
            if (put <= 0) return false;
            p += put;
            n -= static_cast<size_t>(put);
        }
        return true;
    };
    if (!write_all(head.data(), head.size()) || !write_all(itkv, itkv_len) || fsync(fd) != 0) {
        const Refusal r = io_refusal("write temp entry " + temp_name);
        ::close(fd);
        ::unlink(temp_path.c_str());
        return s->fail(r);
    }
    ::close(fd);
    if (::rename(temp_path.c_str(), path.c_str()) != 0) {
        const Refusal r = io_refusal("rename entry " + file_name);
        ::unlink(temp_path.c_str());
        return s->fail(r);
    }
    s->entries.erase(std::remove_if(s->entries.begin(), s->entries.end(),
                                    [&](const EntryMeta& e) { return e.file_name == file_name; }),
                     s->entries.end());
    EntryMeta meta;
    meta.file_name = file_name;
    meta.prefix_hash = key;
    meta.token_count = n_tokens;
    meta.bytes = entry_bytes;
    meta.created = meta.last_used = now;
    s->entries.push_back(meta);
    if (Refusal r = s->evict_except(file_name)) return s->fail(r);
    return ITK_OK;
}

// PrefixStore::lookup (store.rs:314-356).  On a hit *token_count is the matched prefix length and *itkv / *itkv_len
// name the verified snapshot bytes, owned by the store until its next call; on a clean miss *token_count is 0.
int itk_prefix_store_lookup(itk_prefix_store* s, const uint32_t* query, size_t n_query, const itk_config* required_geometry,
                            const char* required_fingerprint, uint64_t now, uint64_t* token_count, const uint8_t** itkv,
                            size_t* itkv_len) {
    if (!s || (!query && n_query) || !token_count || !itkv || !itkv_len) return ITK_ERR_INVALID_ARGUMENT;
    *token_count = 0;
    *itkv = nullptr;
    *itkv_len = 0;
    std::vector<EntryMeta> candidates;
    for (const EntryMeta& e : s->entries)
        if (e.token_count <= n_query) candidates.push_back(e);
    std::stable_sort(candidates.begin(), candidates.end(),
                     [](const EntryMeta& a, const EntryMeta& b) { return a.token_count > b.token_count; });
    for (const EntryMeta& c : candidates) {
        bool matched = false;
        if (Refusal r = s->verify_candidate(c, query, required_geometry, required_fingerprint, &s->hit, &s->hit_tokens, &matched)) {
            s->last_refusal = "prefix store refuses entry " + c.file_name + ": " + r.text;
            continue;
        }
        if (!matched) continue;
        // touch (store.rs:504-515): the 8-byte stamp, in place
        const std::string path = s->root + "/" + c.file_name;
        const int fd = ::open(path.c_str(), O_WRONLY | O_CLOEXEC);
        if (fd < 0) return s->fail(io_refusal("open entry " + c.file_name + " to restamp"));
        uint8_t stamp[8];
        put64(stamp, now);
        const bool ok = ::pwrite(fd, stamp, 8, static_cast<off_t>(kLastUsedOffset)) == 8;
        const Refusal r = ok ? Refusal{} : io_refusal("restamp entry " + c.file_name);
        ::close(fd);
        if (r) return s->fail(r);
        for (EntryMeta& e : s->entries)
            if (e.file_name == c.file_name) e.last_used = now;
        put64(s->hit.data() + kLastUsedOffset, now);
        const size_t tokens_end = kPreambleLen + static_cast<size_t>(c.token_count) * 4;
        *token_count = c.token_count;
        *itkv = s->hit.data() + tokens_end;
        *itkv_len = s->hit.size() - tokens_end;
        return ITK_OK;
    }
    return ITK_OK;
}

// StoreStats (store.rs:108-118, 187-193)
int itk_prefix_store_stats(const itk_prefix_store* s, uint64_t* entries, uint64_t* total_bytes, uint64_t* max_bytes) {
    if (!s) return ITK_ERR_INVALID_ARGUMENT;
    if (entries) *entries = s->entries.size();
    if (total_bytes) *total_bytes = s->total_bytes();
    if (max_bytes) *max_bytes = s->max_bytes;
    return ITK_OK;
}

// PrefixStore::entries (store.rs:179-184): index `i` of the entries sorted longest prefix first.
int itk_prefix_store_entry(const itk_prefix_store* s, uint64_t i, char* file_name, size_t file_name_cap, uint64_t* prefix_hash,
                           uint64_t* token_count, uint64_t* bytes, uint64_t* created_unix, uint64_t* last_used_unix) {
    if (!s || i >= s->entries.size()) return ITK_ERR_INVALID_ARGUMENT;
    std::vector<const EntryMeta*> sorted;
    for (const EntryMeta& e : s->entries) sorted.push_back(&e);
    std::stable_sort(sorted.begin(), sorted.end(), [](const EntryMeta* a, const EntryMeta* b) { return a->token_count > b->token_count; });
    const EntryMeta& e = *sorted[i];
    if (file_name && file_name_cap) snprintf(file_name, file_name_cap, "%s", e.file_name.c_str());
    if (prefix_hash) *prefix_hash = e.prefix_hash;
    if (token_count) *token_count = e.token_count;
    if (bytes) *bytes = e.bytes;
    if (created_unix) *created_unix = e.created;
    if (last_used_unix) *last_used_unix = e.last_used;
    return ITK_OK;
}

// KvSnapshot::from_bytes + validate (crates/itak-kv/src/snapshot.rs:187-236, 425-540) without a device: the strict
// decode alone, for callers that want to vet bytes before handing them to a backend.
int itk_itkv_check(const uint8_t* bytes, size_t n, uint32_t* version, uint64_t* token_count, uint32_t* elem_bytes,
                   char* why, size_t why_len) {
    if (why && why_len) why[0] = '\0';
    if (!bytes) return ITK_ERR_INVALID_ARGUMENT;
    itk::itkv::Parsed parsed;
    std::string text;
    const int rc = itk::itkv::parse(bytes, n, &parsed, &text);
    if (rc != ITK_OK) {
        if (why && why_len) snprintf(why, why_len, "%s", text.c_str());
        return rc;
    }
    if (version) *version = parsed.version;
    if (token_count) *token_count = parsed.token_count;
    if (elem_bytes) *elem_bytes = parsed.elem_bytes;
    return ITK_OK;
}

}  // extern "C"
